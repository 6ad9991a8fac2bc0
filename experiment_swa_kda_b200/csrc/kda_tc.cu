// Tensor-core lane (K = V = 128, bf16 operands, fp32 accumulation and state): the sequential state scans
// on tcgen05 / TMEM, fed by TMA.
//
// One CTA owns one (sequence, head) and walks its chunks in order with the full 128x128 state held in
// registers in V-first form (thread v owns row v, i.e. S[v][0..127]); all products are written transposed so
// that M = 128 (value index) for every UMMA:
//     [ (W H)^T | (R H)^T ]  = H^T [ W^T | R^T ]          M=128, N=128, K=128   (one UMMA chain, MN-major B)
//     Z^T = U^T - (W H)^T                                  registers
//     [ dH^T | (A Z)^T ]     = Z^T [ E | A^T ]             M=128, N=192, K=64    (one UMMA chain, MN-major B)
//     H'^T = exp(G_end) . H^T + dH^T ,  O^T = (R H)^T + (A Z)^T
// so the chunk output falls out of the same two UMMA chains as the state update.
// Restates reference chunk_wy_forward.cu:940-1275 (state scan) and 1498-1588 (output).

#include "common.cuh"
#include "simt_ws.cuh"
#include "tc_common.cuh"
#include "tc_ws.cuh"

namespace kda {
namespace tc {

// ---------------------------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeFn)p;
    }
    return fn;
}

// 2-D bf16 row-major tensor [rows][cols]; box = box_cols x box_rows; 128-byte swizzle (box_cols must be 64).
int make_map_bf16(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
    EncodeFn enc = encode_fn();
    if (!enc) return KDA_ERR_CUDA;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t es[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {
        // a host thread that has made no runtime call yet (e.g. an autograd worker) has no context bound:
        // bind the current device's primary context and try once more
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess && cudaFree(nullptr) == cudaSuccess)
            r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS && getenv("KDA_B200_VERBOSE"))
        fprintf(stderr, "libkda_b200: cuTensorMapEncodeTiled failed (%d): ptr %p rows %llu cols %llu box %u x %u\n", (int)r, ptr,
                (unsigned long long)rows, (unsigned long long)cols, box_cols, box_rows);
    return r == CUDA_SUCCESS ? KDA_OK : KDA_ERR_CUDA;
}

// ---------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 t = __bfloat1622float2(h[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
    }
}

// ---------------------------------------------------------------------------------------------
// forward scan + fused chunk output
// ---------------------------------------------------------------------------------------------
struct ScanFwdArgs {
    const int* seq_chunk0;
    const int* chunk_tok0;
    const int* chunk_len;
    const float* decay_end;   // [nch][128] exp(G_end)
    const float* h0;          // V-first or null
    float* final_state;       // V-first or null
    __nv_bfloat16* o;         // [tokens][H][128]
    int H;
    int save;                 // publish H and Z^T panels for the backward
    int* status;
};

constexpr int kStageBytes = 32768 + 24576 + 16384 + 512;   // [W^T|R^T] + [E|A^T] + U^T + exp(G_end)
constexpr int kStageStride = 32768 + 24576 + 16384 + 1024; // keeps every stage 1024-byte aligned
constexpr int kScanFwdSmem = 2 * kStageStride + 32768 + 16384 + 1024;

// barrier over the 256 state threads only (the output warpgroup never joins it)
__device__ __forceinline__ void state_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// 384 threads.  Warpgroups 0 and 1 hold the state: thread (kh, v) owns S[v][64*kh .. 64*kh+63] in registers and does
// half of every per-step conversion.  Warpgroup 2 only drains the output accumulators and stores o, off the
// critical path.  TMEM: D1 = [(W H)^T | (R H)^T] double-buffered at columns 0 / 320, D2 = [dH^T | (A Z)^T] at 128.
__global__ void __launch_bounds__(384, 1)
    tc_scan_fwd_kernel(const __grid_constant__ CUtensorMap mW, const __grid_constant__ CUtensorMap mR,
                       const __grid_constant__ CUtensorMap mE, const __grid_constant__ CUtensorMap mAT,
                       const __grid_constant__ CUtensorMap mUT, const __grid_constant__ CUtensorMap mH,
                       const __grid_constant__ CUtensorMap mZT, ScanFwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* Hop = sm + 2 * kStageStride;         // [2 k-blocks][128 rows x 128 B]
    uint8_t* Zop = Hop + 32768;                   // [128 rows x 128 B]
    __shared__ uint64_t bar_full[2], bar_mma1, bar_mma2, bar_o;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag, go_flag;   // any thread may raise abort; only thread 0 writes go

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wg = warp >> 2;                      // 0,1: state (key half), 2: output
    const int v = (warp & 3) * 32 + lane;          // value row = TMEM lane
    const int seq = blockIdx.x, h = blockIdx.y, H = p.H;
    const int c_begin = p.seq_chunk0[seq], c_end = p.seq_chunk0[seq + 1];
    const int n = c_end - c_begin;

    if (tid == 0) {
        mbar_init(&bar_full[0], 1);
        mbar_init(&bar_full[1], 1);
        mbar_init(&bar_mma1, 1);
        mbar_init(&bar_mma2, 1);
        mbar_init(&bar_o, 128);
        mbar_fence_init();
        abort_flag = 0;
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    constexpr uint32_t cD2 = 128;

    if (wg == 2) {
        // ------------------------------------------------------------------ output warpgroup
        for (int c = 0; c < n; ++c) {
            const int slot = c_begin + c;
            const int len = p.chunk_len[slot], tok0 = p.chunk_tok0[slot];
            if (!mbar_wait(&bar_mma2, c & 1, p.status, 14)) { abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t d1 = tmem + lane_base + ((c & 1) ? 320u : 0u) + 64;
            float ov[64];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint32_t r1[32], r2[32];
                tmem_ld32(d1 + b * 32, r1);
                tmem_ld32(tmem + lane_base + cD2 + 128 + b * 32, r2);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) ov[32 * b + j] = __uint_as_float(r1[j]) + __uint_as_float(r2[j]);
            }
            tc_fence_before();
            mbar_arrive(&bar_o);               // accumulators drained: the issuer may overwrite them
            __nv_bfloat16* orow = p.o + ((size_t)tok0 * H + h) * 128 + v;
#pragma unroll
            for (int i = 0; i < 64; ++i)
                if (i < len) orow[(size_t)i * H * 128] = __float2bfloat16(ov[i]);
        }
    } else {
        // ------------------------------------------------------------------ state warpgroups
        const int kh = wg;
        float hs[64];
        if (p.h0) {
            const float4* src = reinterpret_cast<const float4*>(p.h0 + (((size_t)seq * H + h) * 128 + v) * 128 + 64 * kh);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float4 x = src[j];
                hs[4 * j] = x.x; hs[4 * j + 1] = x.y; hs[4 * j + 2] = x.z; hs[4 * j + 3] = x.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) hs[j] = 0.f;
        }
        auto issue_loads = [&](int c) {   // thread 0 only
            const int st = c & 1;
            const int ch = (c_begin + c) * H + h;
            uint8_t* b = sm + st * kStageStride;
            mbar_expect_tx(&bar_full[st], kStageBytes);
            bulk_load_1d(b + 73728, p.decay_end + (size_t)ch * 128, 512, &bar_full[st]);
            tma_load_2d(b, &mW, &bar_full[st], 0, ch * 128);            // W^T [key][token]: n-block 0
            tma_load_2d(b + 16384, &mR, &bar_full[st], 0, ch * 128);    // R^T [key][token]: n-block 1
            for (int nb = 0; nb < 2; ++nb) tma_load_2d(b + 32768 + nb * 8192, &mE, &bar_full[st], nb * 64, ch * 64);
            tma_load_2d(b + 32768 + 16384, &mAT, &bar_full[st], 0, ch * 64);
            tma_load_2d(b + 32768 + 24576, &mUT, &bar_full[st], 0, ch * 128);
        };
        int loads_issued = 0;
        if (n > 0) {
            if (tid == 0) issue_loads(0);
            loads_issued = 1;
        }
        const uint32_t idesc1 = umma_idesc_bf16(128, 128, kMajorK, kMajorMN);
        const uint32_t idesc2 = umma_idesc_bf16(128, 192, kMajorK, kMajorMN);

        for (int c = 0; c < n; ++c) {
            const int st = c & 1;
            const int ch = (c_begin + c) * H + h;
            uint8_t* sb = sm + st * kStageStride;
            const uint32_t cD1 = (c & 1) ? 320u : 0u;
            if (tid == 0) {
                if (p.save) tma_store_wait_read();            // the previous chunk's panel stores have read Hop / Zop
                go_flag = abort_flag ? 0 : 1;                 // one uniform decision per step
            }
            state_sync();
            if (!go_flag) break;
            if (c + 1 < n) {                                  // prefetch: that stage was last read by chunk c-1
                if (tid == 0) issue_loads(c + 1);
                loads_issued = c + 2;
            }
            // ---- this thread's half of the state row -> bf16 A operand (K-major, 128-byte swizzle)
#pragma unroll
            for (int c16 = 0; c16 < 8; ++c16) {
                uint4 u;
                u.x = pack_bf16(hs[8 * c16 + 0], hs[8 * c16 + 1]);
                u.y = pack_bf16(hs[8 * c16 + 2], hs[8 * c16 + 3]);
                u.z = pack_bf16(hs[8 * c16 + 4], hs[8 * c16 + 5]);
                u.w = pack_bf16(hs[8 * c16 + 6], hs[8 * c16 + 7]);
                *reinterpret_cast<uint4*>(Hop + kh * 16384 + sw128_off(v, c16)) = u;
            }
            fence_async_smem();
            tc_fence_before();
            state_sync();
            if (tid == 0) {
                if (!mbar_wait(&bar_full[st], (c >> 1) & 1, p.status, 11)) abort_flag = 1;
                else {
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(Hop), b0 = smem_u32(sb);
#pragma unroll
                    for (int k16 = 0; k16 < 8; ++k16)
                        umma_bf16_ss(tmem + cD1, umma_smem_desc_sw128(a0 + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                                     umma_smem_desc_sw128(b0 + k16 * 2048, 16384, 1024), idesc1, k16 > 0);
                    umma_commit(&bar_mma1);
                    if (p.save) {
                        tma_store_2d(&mH, Hop, 0, ch * 128);
                        tma_store_2d(&mH, Hop + 16384, 64, ch * 128);
                        tma_store_commit();
                    }
                }
            }
            // ---- Z^T = U^T - (W H)^T: this thread converts tokens 32*kh .. 32*kh+31 of its row
            if (!mbar_wait(&bar_mma1, c & 1, p.status, 12)) abort_flag = 1;
            tc_fence_after();
            {
                const uint8_t* UTs = sb + 32768 + 24576;
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + cD1 + 32 * kh, r);
                tmem_ld_wait();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int c16 = kh * 4 + q4;
                    float u[8];
                    unpack_bf16x8(*reinterpret_cast<const uint4*>(UTs + sw128_off(v, c16)), u);
                    uint4 z;
                    z.x = pack_bf16(u[0] - __uint_as_float(r[8 * q4 + 0]), u[1] - __uint_as_float(r[8 * q4 + 1]));
                    z.y = pack_bf16(u[2] - __uint_as_float(r[8 * q4 + 2]), u[3] - __uint_as_float(r[8 * q4 + 3]));
                    z.z = pack_bf16(u[4] - __uint_as_float(r[8 * q4 + 4]), u[5] - __uint_as_float(r[8 * q4 + 5]));
                    z.w = pack_bf16(u[6] - __uint_as_float(r[8 * q4 + 6]), u[7] - __uint_as_float(r[8 * q4 + 7]));
                    *reinterpret_cast<uint4*>(Zop + sw128_off(v, c16)) = z;
                }
            }
            fence_async_smem();
            tc_fence_before();
            state_sync();
            if (tid == 0) {
                // the output warpgroup must have drained chunk c-1's accumulators before they are overwritten
                if (c > 0 && !mbar_wait(&bar_o, (c - 1) & 1, p.status, 15)) abort_flag = 1;
                else {
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(Zop), b0 = smem_u32(sb + 32768);
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)
                        umma_bf16_ss(tmem + cD2, umma_smem_desc_sw128(a0 + k16 * 32, 16, 1024),
                                     umma_smem_desc_sw128(b0 + k16 * 2048, 8192, 1024), idesc2, k16 > 0);
                    umma_commit(&bar_mma2);
                    if (p.save) {
                        tma_store_2d(&mZT, Zop, 0, ch * 128);
                        tma_store_commit();
                    }
                }
            }
            // ---- state update for this thread's 64 key columns
            if (!mbar_wait(&bar_mma2, c & 1, p.status, 13)) abort_flag = 1;
            tc_fence_after();
            const float* dc = reinterpret_cast<const float*>(sb + 73728) + 64 * kh;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + cD2 + 64 * kh + b * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 dv = *reinterpret_cast<const float4*>(dc + 32 * b + 4 * j4);
                    hs[32 * b + 4 * j4 + 0] = dv.x * hs[32 * b + 4 * j4 + 0] + __uint_as_float(r[4 * j4 + 0]);
                    hs[32 * b + 4 * j4 + 1] = dv.y * hs[32 * b + 4 * j4 + 1] + __uint_as_float(r[4 * j4 + 1]);
                    hs[32 * b + 4 * j4 + 2] = dv.z * hs[32 * b + 4 * j4 + 2] + __uint_as_float(r[4 * j4 + 2]);
                    hs[32 * b + 4 * j4 + 3] = dv.w * hs[32 * b + 4 * j4 + 3] + __uint_as_float(r[4 * j4 + 3]);
                }
            }
            tc_fence_before();
        }
        // ---- unwind
        state_sync();
        const bool ok = abort_flag == 0;
        if (!ok && tid == 0) {
            for (int c = 0; c < loads_issued; ++c)
                if (c >= loads_issued - 2) mbar_wait(&bar_full[c & 1], (c >> 1) & 1, nullptr, 0);
        }
        if (p.save && tid == 0) tma_store_wait_all();
        if (ok && p.final_state) {
            float4* dst = reinterpret_cast<float4*>(p.final_state + (((size_t)seq * H + h) * 128 + v) * 128 + 64 * kh);
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[j] = make_float4(hs[4 * j], hs[4 * j + 1], hs[4 * j + 2], hs[4 * j + 3]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------
// reverse scan of the state adjoint (restates reference chunk_wy_backward.cu:2445-2562)
//   dZ^T = dO^T A + dH'^T E^T                      [v x i]   UMMA chain 1: M=128, N=64
//   dH^T = exp(G_end) . dH'^T + dO^T R - dZ^T W    [v x k]   UMMA chain 2: M=128, N=128 (second part with -A)
// dO arrives token-major [s][v], i.e. as an MN-major A operand; R and W [i][k] are MN-major B operands.
// ---------------------------------------------------------------------------------------------
struct ScanBwdArgs {
    const int* seq_chunk0;
    const int* chunk_tok0;
    const float* decay_end;
    const float* d_final;   // V-first cotangent of the final state, or null
    float* dh0;             // V-first, or null
    int H;
    int* status;
};

constexpr int kScanBwdSmem = 2 * kStageStride + 32768 + 16384 + 1024;

// 256 threads: thread (kh, v) owns dH'[v][64*kh .. 64*kh+63] in registers and does half of every per-step conversion.
__global__ void __launch_bounds__(256, 1)
    tc_scan_bwd_kernel(const __grid_constant__ CUtensorMap mW, const __grid_constant__ CUtensorMap mR,
                       const __grid_constant__ CUtensorMap mE, const __grid_constant__ CUtensorMap mAT,
                       const __grid_constant__ CUtensorMap mdO, const __grid_constant__ CUtensorMap mdH,
                       const __grid_constant__ CUtensorMap mdZT, ScanBwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* dHop = sm + 2 * kStageStride;   // [2 k-blocks][128 rows x 128 B]
    uint8_t* dZop = dHop + 32768;            // [128 rows x 128 B]
    __shared__ uint64_t bar_full[2], bar_mma1, bar_mma2;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag, go_flag;   // any thread may raise abort; only thread 0 writes go

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kh = warp >> 2;                     // key half of this thread
    const int v = (warp & 3) * 32 + lane;         // value row = TMEM lane
    const int seq = blockIdx.x, h = blockIdx.y, H = p.H;
    const int c_begin = p.seq_chunk0[seq], c_end = p.seq_chunk0[seq + 1];
    const int n = c_end - c_begin;

    if (tid == 0) {
        mbar_init(&bar_full[0], 1);
        mbar_init(&bar_full[1], 1);
        mbar_init(&bar_mma1, 1);
        mbar_init(&bar_mma2, 1);
        mbar_fence_init();
        abort_flag = 0;
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t D1 = tmem + lane_base;         // cols [0,64)   dZ^T
    const uint32_t D2 = tmem + lane_base + 64;    // cols [64,192) dO^T R - dZ^T W

    float dh[64];
    if (p.d_final) {
        const float4* src = reinterpret_cast<const float4*>(p.d_final + (((size_t)seq * H + h) * 128 + v) * 128 + 64 * kh);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float4 x = src[j];
            dh[4 * j] = x.x; dh[4 * j + 1] = x.y; dh[4 * j + 2] = x.z; dh[4 * j + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) dh[j] = 0.f;
    }

    // step j = 0 .. n-1 walks the chunks from the last to the first
    auto issue_loads = [&](int j) {   // thread 0 only
        const int st = j & 1;
        const int slot = c_end - 1 - j;
        const int ch = slot * H + h;
        const int tok0 = p.chunk_tok0[slot];
        uint8_t* b = sm + st * kStageStride;
        mbar_expect_tx(&bar_full[st], kStageBytes);
        bulk_load_1d(b + 73728, p.decay_end + (size_t)ch * 128, 512, &bar_full[st]);
        for (int kb = 0; kb < 2; ++kb) {
            tma_load_2d(b + kb * 8192, &mE, &bar_full[st], kb * 64, ch * 64);
            tma_load_2d(b + 57344 + kb * 8192, &mdO, &bar_full[st], h * 128 + kb * 64, tok0);
        }
        tma_load_2d(b + 24576, &mR, &bar_full[st], 0, ch * 128);    // R^T [key][token], K-major B
        tma_load_2d(b + 40960, &mW, &bar_full[st], 0, ch * 128);    // W^T [key][token], K-major B
        tma_load_2d(b + 16384, &mAT, &bar_full[st], 0, ch * 64);
    };

    int loads_issued = 0;
    if (n > 0) {
        if (tid == 0) issue_loads(0);
        loads_issued = 1;
    }
    const uint32_t id1a = umma_idesc_bf16(128, 64, kMajorMN, kMajorK);
    const uint32_t id1b = umma_idesc_bf16(128, 64, kMajorK, kMajorK);
    const uint32_t id2a = umma_idesc_bf16(128, 128, kMajorMN, kMajorK);
    const uint32_t id2b = umma_idesc_bf16(128, 128, kMajorK, kMajorK, 1);

    for (int j = 0; j < n; ++j) {
        const int st = j & 1;
        const int slot = c_end - 1 - j;
        const int ch = slot * H + h;
        uint8_t* sb = sm + st * kStageStride;
        if (tid == 0) {
            tma_store_wait_read();                    // the previous step's panel stores have read dHop / dZop
            go_flag = abort_flag ? 0 : 1;             // one uniform decision per step
        }
        __syncthreads();
        if (!go_flag) break;
        if (j + 1 < n) {
            if (tid == 0) issue_loads(j + 1);
            loads_issued = j + 2;
        }
        // ---- this thread's half of dH' -> bf16 A operand
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {
            uint4 u;
            u.x = pack_bf16(dh[8 * c16 + 0], dh[8 * c16 + 1]);
            u.y = pack_bf16(dh[8 * c16 + 2], dh[8 * c16 + 3]);
            u.z = pack_bf16(dh[8 * c16 + 4], dh[8 * c16 + 5]);
            u.w = pack_bf16(dh[8 * c16 + 6], dh[8 * c16 + 7]);
            *reinterpret_cast<uint4*>(dHop + kh * 16384 + sw128_off(v, c16)) = u;
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            if (!mbar_wait(&bar_full[st], (j >> 1) & 1, p.status, 21)) abort_flag = 1;
            else {
                tc_fence_after();
                const uint32_t s0 = smem_u32(sb), a_dh = smem_u32(dHop);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)     // dO^T A
                    umma_bf16_ss(tmem, umma_smem_desc_sw128(s0 + 57344 + k16 * 2048, 8192, 1024),
                                 umma_smem_desc_sw128(s0 + 16384 + k16 * 32, 16, 1024), id1a, k16 > 0);
#pragma unroll
                for (int k16 = 0; k16 < 8; ++k16)     // + dH'^T E^T
                    umma_bf16_ss(tmem, umma_smem_desc_sw128(a_dh + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                                 umma_smem_desc_sw128(s0 + (k16 >> 2) * 8192 + (k16 & 3) * 32, 16, 1024), id1b, 1);
                umma_commit(&bar_mma1);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)     // dO^T R   (runs while the threads convert dZ)
                    umma_bf16_ss(tmem + 64, umma_smem_desc_sw128(s0 + 57344 + k16 * 2048, 8192, 1024),
                                 umma_smem_desc_sw128(s0 + 24576 + k16 * 32, 16, 1024), id2a, k16 > 0);
                tma_store_2d(&mdH, dHop, 0, ch * 128);
                tma_store_2d(&mdH, dHop + 16384, 64, ch * 128);
                tma_store_commit();
            }
        }
        if (!mbar_wait(&bar_mma1, j & 1, p.status, 22)) abort_flag = 1;
        tc_fence_after();
        {   // dZ^T: this thread converts tokens 32*kh .. 32*kh+31 of its row
            uint32_t r[32];
            tmem_ld32(D1 + 32 * kh, r);
            tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                uint4 z;
                z.x = pack_bf16(__uint_as_float(r[8 * q4 + 0]), __uint_as_float(r[8 * q4 + 1]));
                z.y = pack_bf16(__uint_as_float(r[8 * q4 + 2]), __uint_as_float(r[8 * q4 + 3]));
                z.z = pack_bf16(__uint_as_float(r[8 * q4 + 4]), __uint_as_float(r[8 * q4 + 5]));
                z.w = pack_bf16(__uint_as_float(r[8 * q4 + 6]), __uint_as_float(r[8 * q4 + 7]));
                *reinterpret_cast<uint4*>(dZop + sw128_off(v, kh * 4 + q4)) = z;
            }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const uint32_t s0 = smem_u32(sb), a_dz = smem_u32(dZop);
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16)         // - dZ^T W
                umma_bf16_ss(tmem + 64, umma_smem_desc_sw128(a_dz + k16 * 32, 16, 1024),
                             umma_smem_desc_sw128(s0 + 40960 + k16 * 32, 16, 1024), id2b, 1);
            umma_commit(&bar_mma2);
            tma_store_2d(&mdZT, dZop, 0, ch * 128);
            tma_store_commit();
        }
        if (!mbar_wait(&bar_mma2, j & 1, p.status, 23)) abort_flag = 1;
        tc_fence_after();
        const float* dc = reinterpret_cast<const float*>(sb + 73728) + 64 * kh;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            uint32_t r[32];
            tmem_ld32(D2 + 64 * kh + b * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
                const float4 dv = *reinterpret_cast<const float4*>(dc + 32 * b + 4 * j4);
                dh[32 * b + 4 * j4 + 0] = dv.x * dh[32 * b + 4 * j4 + 0] + __uint_as_float(r[4 * j4 + 0]);
                dh[32 * b + 4 * j4 + 1] = dv.y * dh[32 * b + 4 * j4 + 1] + __uint_as_float(r[4 * j4 + 1]);
                dh[32 * b + 4 * j4 + 2] = dv.z * dh[32 * b + 4 * j4 + 2] + __uint_as_float(r[4 * j4 + 2]);
                dh[32 * b + 4 * j4 + 3] = dv.w * dh[32 * b + 4 * j4 + 3] + __uint_as_float(r[4 * j4 + 3]);
            }
        }
        tc_fence_before();
    }

    __syncthreads();
    const bool ok = abort_flag == 0;
    if (!ok && tid == 0) {
        for (int j = 0; j < loads_issued; ++j)
            if (j >= loads_issued - 2) mbar_wait(&bar_full[j & 1], (j >> 1) & 1, nullptr, 0);
    }
    if (tid == 0) tma_store_wait_all();
    if (ok && p.dh0) {
        float4* dst = reinterpret_cast<float4*>(p.dh0 + (((size_t)seq * H + h) * 128 + v) * 128 + 64 * kh);
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j] = make_float4(dh[4 * j], dh[4 * j + 1], dh[4 * j + 2], dh[4 * j + 3]);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 256);
}

}  // namespace tc

// ---------------------------------------------------------------------------------------------
// host entry used by the chunk forward when the tensor-core lane is selected
// ---------------------------------------------------------------------------------------------
int tc_scan_forward(const simt::Ws& w, const tc::TcWs& t, int n_seq, const float* h0, float* final_state, void* o,
                    cudaStream_t st) {
    using namespace tc;
    const uint64_t nch = (uint64_t)w.nslots * w.H;
    CUtensorMap mW, mR, mE, mAT, mUT, mH, mZT;
    int rc = 0;
    rc |= make_map_bf16(&mW, t.WT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mR, t.RT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mE, t.E, nch * 64, 128, 64, 64);
    rc |= make_map_bf16(&mAT, t.AT, nch * 64, 64, 64, 64);
    rc |= make_map_bf16(&mUT, t.UT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mH, t.Hp, nch * 128, 128, 64, 128);
    rc |= make_map_bf16(&mZT, t.ZT, nch * 128, 64, 64, 128);
    if (rc) return KDA_ERR_CUDA;
    ScanFwdArgs a;
    a.seq_chunk0 = w.seq_chunk0; a.chunk_tok0 = w.chunk_tok0; a.chunk_len = w.chunk_len;
    a.decay_end = t.decay_end; a.h0 = h0; a.final_state = final_state; a.o = static_cast<__nv_bfloat16*>(o);
    a.H = w.H; a.save = 1; a.status = t.status;
    if (cudaFuncSetAttribute(tc_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanFwdSmem) != cudaSuccess)
        return KDA_ERR_CUDA;
    KDA_LAUNCH("tc_scan_fwd_kernel", st,
               tc_scan_fwd_kernel<<<dim3(n_seq, w.H), 384, kScanFwdSmem, st>>>(mW, mR, mE, mAT, mUT, mH, mZT, a));
    return launch_status();
}

int tc_scan_backward(const simt::Ws& w, const simt::Scr& s, const tc::TcWs& t, int n_seq, int tokens, const void* d_o,
                     const float* d_final, float* dh0, cudaStream_t st) {
    using namespace tc;
    const uint64_t nch = (uint64_t)w.nslots * w.H;
    CUtensorMap mW, mR, mE, mAT, mdO, mdH, mdZT;
    int rc = 0;
    rc |= make_map_bf16(&mW, t.WT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mR, t.RT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mE, t.E, nch * 64, 128, 64, 64);
    rc |= make_map_bf16(&mAT, t.AT, nch * 64, 64, 64, 64);
    rc |= make_map_bf16(&mdO, d_o, (uint64_t)tokens, (uint64_t)w.H * 128, 64, 64);
    rc |= make_map_bf16(&mdH, t.dHp, nch * 128, 128, 64, 128);
    rc |= make_map_bf16(&mdZT, t.dZT, nch * 128, 64, 64, 128);
    if (rc) return KDA_ERR_CUDA;
    ScanBwdArgs a;
    a.seq_chunk0 = w.seq_chunk0; a.chunk_tok0 = w.chunk_tok0; a.decay_end = t.decay_end;
    a.d_final = d_final; a.dh0 = dh0; a.H = w.H; a.status = t.status;
    if (cudaFuncSetAttribute(tc_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanBwdSmem) != cudaSuccess)
        return KDA_ERR_CUDA;
    KDA_LAUNCH("tc_scan_bwd_kernel", st,
               tc_scan_bwd_kernel<<<dim3(n_seq, w.H), 256, kScanBwdSmem, st>>>(mW, mR, mE, mAT, mdO, mdH, mdZT, a));
    return launch_status();
}

}  // namespace kda
