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

constexpr int kStageData = 32768 + 24576 + 16384;          // [W^T|R^T] + [E|A^T] + U^T
constexpr int kStageBytes = kStageData + 512;              // + exp(G_end), which lands in a ring of its own
constexpr int kStageStride = kStageData;                   // 73,728: every stage stays 1024-byte aligned
constexpr int kScanFwdSmem = 2 * kStageStride + 32768 + 16384 + 1024;

#ifdef KDA_PHASE_TIMING
#define KDA_TICKS(n) do { if (tid == 0) { long long t_ = clock64(); acc[n] += t_ - tlast; tlast = t_; } } while (0)
#else
#define KDA_TICKS(n) do { } while (0)
#endif

// 448 threads, specialised by warp; nothing on the recurrence's critical path waits for work that only feeds the output.
//   warps 0-7   state: thread (kh, v) owns S[v][64*kh .. 64*kh+63] in registers and does half of every conversion
//   warps 8-11  output: drain the output accumulators and store o
//   warp 12     one lane issues the TMA loads, two chunks ahead
//   warp 13     one lane issues every UMMA and the TMA stores of the panels the backward needs
// The threads meet only through mbarriers.  Each UMMA chain is split so that the part the recurrence waits for is
// committed first:
//   chain 1:  (W H)^T -> commit -> (R H)^T            D1 = [(W H)^T | (R H)^T], double-buffered at columns 0 / 320
//   chain 2:  dH^T    -> commit -> (A Z)^T -> commit  D2 = [dH^T | (A Z)^T] at column 128
__global__ void __launch_bounds__(448, 1)
    tc_scan_fwd_kernel(const __grid_constant__ CUtensorMap mW, const __grid_constant__ CUtensorMap mR,
                       const __grid_constant__ CUtensorMap mE, const __grid_constant__ CUtensorMap mAT,
                       const __grid_constant__ CUtensorMap mUT, const __grid_constant__ CUtensorMap mH,
                       const __grid_constant__ CUtensorMap mZT, ScanFwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* Hop = sm + 2 * kStageStride;         // [2 k-blocks][128 rows x 128 B]
    uint8_t* Zop = Hop + 32768;                   // [128 rows x 128 B]
    __shared__ __align__(16) float dec_ring[4][128];   // exp(G_end) of chunk c in slot c % 4
    // full: a stage has landed.  hop / zop: all 256 state threads have written their part of the state / Z panel.
    // mma1 / mma2: the product the recurrence waits for is complete.  out: every product of the chunk is complete.
    // o: the output warpgroup has drained the chunk's accumulators.
    // free: every product that reads a stage is complete (per stage, so that the load thread can never miss a phase).
    __shared__ uint64_t bar_full[2], bar_free[2], bar_hop, bar_zop, bar_mma1, bar_mma2, bar_out, bar_o;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int v = (warp & 3) * 32 + lane;          // value row = TMEM lane
    const int seq = blockIdx.x, h = blockIdx.y, H = p.H;
    const int c_begin = p.seq_chunk0[seq], c_end = p.seq_chunk0[seq + 1];
    const int n = c_end - c_begin;

    if (tid == 0) {
        mbar_init(&bar_full[0], 1);
        mbar_init(&bar_full[1], 1);
        mbar_init(&bar_free[0], 1);
        mbar_init(&bar_free[1], 1);
        mbar_init(&bar_hop, 256);
        mbar_init(&bar_zop, 256);
        mbar_init(&bar_mma1, 1);
        mbar_init(&bar_mma2, 1);
        mbar_init(&bar_out, 1);
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

    if (warp == 12) {
        // ------------------------------------------------------------------ load warp
        if (lane == 0) {
            auto issue_loads = [&](int c) {
                const int st = c & 1;
                const int ch = (c_begin + c) * H + h;
                uint8_t* b = sm + st * kStageStride;
                mbar_expect_tx(&bar_full[st], kStageBytes);
                bulk_load_1d(dec_ring[c & 3], p.decay_end + (size_t)ch * 128, 512, &bar_full[st]);
                tma_load_2d(b, &mW, &bar_full[st], 0, ch * 128);            // W^T [key][token]
                tma_load_2d(b + 16384, &mR, &bar_full[st], 0, ch * 128);    // R^T [key][token]
                for (int nb = 0; nb < 2; ++nb) tma_load_2d(b + 32768 + nb * 8192, &mE, &bar_full[st], nb * 64, ch * 64);
                tma_load_2d(b + 32768 + 16384, &mAT, &bar_full[st], 0, ch * 64);
                tma_load_2d(b + 32768 + 24576, &mUT, &bar_full[st], 0, ch * 128);
            };
            int issued = 0;
            for (; issued < 2 && issued < n; ++issued) issue_loads(issued);
            bool ok = true;
            // stage c % 2 is free once every product of chunk c has completed
            for (int c = 0; c + 2 < n && ok; ++c) {
                ok = mbar_wait(&bar_free[c & 1], (c >> 1) & 1, p.status, 16);
                if (ok) { issue_loads(c + 2); issued = c + 3; }
                else abort_flag = 1;
            }
            if (!ok)   // unwinding: the copies in flight must land before the block may exit
                for (int c = issued > 2 ? issued - 2 : 0; c < issued; ++c) mbar_wait(&bar_full[c & 1], (c >> 1) & 1, nullptr, 0);
        }
    } else if (warp == 13) {
        // ------------------------------------------------------------------ UMMA / panel-store thread
        if (lane == 0) {
            const uint32_t idesc_n64 = umma_idesc_bf16(128, 64, kMajorK, kMajorMN);
            const uint32_t idesc_n128 = umma_idesc_bf16(128, 128, kMajorK, kMajorMN);
            const uint32_t a_h = smem_u32(Hop), a_z = smem_u32(Zop);
            for (int c = 0; c < n; ++c) {
                const int st = c & 1;
                const int ch = (c_begin + c) * H + h;
                const uint32_t b0 = smem_u32(sm + st * kStageStride);
                const uint32_t cD1 = (c & 1) ? 320u : 0u;
                // Every panel store is waited for (its read of shared memory) before the commit that lets the state
                // threads rewrite that panel: the Z panel before mma1, the state panel before mma2.
                if (p.save) tma_store_wait_read();
                if (!mbar_wait(&bar_full[st], (c >> 1) & 1, p.status, 11) || !mbar_wait(&bar_hop, c & 1, p.status, 17)) {
                    abort_flag = 1;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < 8; ++k16)         // (W H)^T: the recurrence waits for this half only
                    umma_bf16_ss(tmem + cD1, umma_smem_desc_sw128(a_h + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                                 umma_smem_desc_sw128(b0 + k16 * 2048, 16384, 1024), idesc_n64, k16 > 0);
                umma_commit(&bar_mma1);
#pragma unroll
                for (int k16 = 0; k16 < 8; ++k16)         // (R H)^T: read by the output warpgroup
                    umma_bf16_ss(tmem + cD1 + 64, umma_smem_desc_sw128(a_h + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                                 umma_smem_desc_sw128(b0 + 16384 + k16 * 2048, 16384, 1024), idesc_n64, k16 > 0);
                if (p.save) {
                    tma_store_2d(&mH, Hop, 0, ch * 128);
                    tma_store_2d(&mH, Hop + 16384, 64, ch * 128);
                    tma_store_commit();
                    tma_store_wait_read();
                }
                if (!mbar_wait(&bar_zop, c & 1, p.status, 18)) { abort_flag = 1; break; }
                tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)         // dH^T = Z^T E
                    umma_bf16_ss(tmem + cD2, umma_smem_desc_sw128(a_z + k16 * 32, 16, 1024),
                                 umma_smem_desc_sw128(b0 + 32768 + k16 * 2048, 8192, 1024), idesc_n128, k16 > 0);
                umma_commit(&bar_mma2);
                // the output warpgroup must have drained chunk c-1's accumulators before (A Z)^T overwrites them
                if (c > 0 && !mbar_wait(&bar_o, (c - 1) & 1, p.status, 15)) { abort_flag = 1; break; }
                tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)         // (A Z)^T
                    umma_bf16_ss(tmem + cD2 + 128, umma_smem_desc_sw128(a_z + k16 * 32, 16, 1024),
                                 umma_smem_desc_sw128(b0 + 32768 + 16384 + k16 * 2048, 8192, 1024), idesc_n64, k16 > 0);
                umma_commit(&bar_out);
                umma_commit(&bar_free[st]);
                if (p.save) {
                    tma_store_2d(&mZT, Zop, 0, ch * 128);
                    tma_store_commit();
                }
            }
            if (p.save) tma_store_wait_all();
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ output warpgroup
        for (int c = 0; c < n; ++c) {
            const int slot = c_begin + c;
            const int len = p.chunk_len[slot], tok0 = p.chunk_tok0[slot];
            if (!mbar_wait(&bar_out, c & 1, p.status, 14)) { abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t d1 = tmem + lane_base + ((c & 1) ? 320u : 0u) + 64;
            __nv_bfloat16* orow = p.o + ((size_t)tok0 * H + h) * 128 + v;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint32_t r1[32], r2[32];
                tmem_ld32(d1 + b * 32, r1);
                tmem_ld32(tmem + lane_base + cD2 + 128 + b * 32, r2);
                tmem_ld_wait();
                if (b == 1) {
                    tc_fence_before();
                    mbar_arrive(&bar_o);       // accumulators drained: the issuer may overwrite them
                }
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (32 * b + j < len)
                        orow[(size_t)(32 * b + j) * H * 128] = __float2bfloat16(__uint_as_float(r1[j]) + __uint_as_float(r2[j]));
            }
        }
    } else {
        // ------------------------------------------------------------------ state warpgroups
        const int kh = warp >> 2;
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
        // this thread's half of the state row -> bf16 A operand (K-major, 128-byte swizzle)
        auto pack_state = [&]() {
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
            mbar_arrive(&bar_hop);
        };
#ifdef KDA_PHASE_TIMING
        long long acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tlast = clock64();
#endif
        bool ok = true;
        if (n > 0) pack_state();
        for (int c = 0; c < n; ++c) {
            const int st = c & 1;
            const uint8_t* sb = sm + st * kStageStride;
            const uint32_t cD1 = (c & 1) ? 320u : 0u;
            KDA_TICKS(0);
            // ---- Z^T = U^T - (W H)^T: this thread converts tokens 32*kh .. 32*kh+31 of its row
            if (!mbar_wait(&bar_mma1, c & 1, p.status, 12) || !mbar_wait(&bar_full[st], (c >> 1) & 1, p.status, 19)) {
                abort_flag = 1; ok = false;
                break;
            }
            tc_fence_after();
            KDA_TICKS(1);
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
            mbar_arrive(&bar_zop);
            KDA_TICKS(2);
            // ---- state update for this thread's 64 key columns
            if (!mbar_wait(&bar_mma2, c & 1, p.status, 13)) { abort_flag = 1; ok = false; break; }
            tc_fence_after();
            KDA_TICKS(3);
            const float* dc = dec_ring[c & 3] + 64 * kh;
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
            KDA_TICKS(4);
            if (c + 1 < n) pack_state();
            KDA_TICKS(5);
        }
#ifdef KDA_PHASE_TIMING
        if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && n > 0)
            printf("scan_fwd per step: loop %lld | wait1 %lld | Z conv %lld | wait2 %lld | update %lld | pack %lld\n",
                   acc[0] / n, acc[1] / n, acc[2] / n, acc[3] / n, acc[4] / n, acc[5] / n);
#endif
        if (ok && abort_flag == 0 && p.final_state) {
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

// 320 threads, specialised by warp like the forward scan:
//   warps 0-7  state: thread (kh, v) owns dH'[v][64*kh .. 64*kh+63] in registers and does half of every conversion
//   warp 8     one lane issues the TMA loads, two chunks ahead
//   warp 9     one lane issues every UMMA and the TMA stores of the dH' / dZ^T panels
// The products that do not depend on dH' (dO^T A and dO^T R) are issued one step early, into accumulators that the
// dependent products then add to: D1 = dZ^T at columns [0,64); D2 = dO^T R - dZ^T W double-buffered at 64 / 192.
__global__ void __launch_bounds__(320, 1)
    tc_scan_bwd_kernel(const __grid_constant__ CUtensorMap mW, const __grid_constant__ CUtensorMap mR,
                       const __grid_constant__ CUtensorMap mE, const __grid_constant__ CUtensorMap mAT,
                       const __grid_constant__ CUtensorMap mdO, const __grid_constant__ CUtensorMap mdH,
                       const __grid_constant__ CUtensorMap mdZT, ScanBwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* dHop = sm + 2 * kStageStride;   // [2 k-blocks][128 rows x 128 B]
    uint8_t* dZop = dHop + 32768;            // [128 rows x 128 B]
    __shared__ __align__(16) float dec_ring[4][128];   // exp(G_end) of step j in slot j % 4
    __shared__ uint64_t bar_full[2], bar_free[2], bar_hop, bar_zop, bar_mma1, bar_mma2;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int v = (warp & 3) * 32 + lane;         // value row = TMEM lane
    const int seq = blockIdx.x, h = blockIdx.y, H = p.H;
    const int c_begin = p.seq_chunk0[seq], c_end = p.seq_chunk0[seq + 1];
    const int n = c_end - c_begin;

    if (tid == 0) {
        mbar_init(&bar_full[0], 1);
        mbar_init(&bar_full[1], 1);
        mbar_init(&bar_free[0], 1);
        mbar_init(&bar_free[1], 1);
        mbar_init(&bar_hop, 256);
        mbar_init(&bar_zop, 256);
        mbar_init(&bar_mma1, 1);
        mbar_init(&bar_mma2, 1);
        mbar_fence_init();
        abort_flag = 0;
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

    // step j = 0 .. n-1 walks the chunks from the last to the first
    if (warp == 8) {
        // ------------------------------------------------------------------ load warp
        if (lane == 0) {
            auto issue_loads = [&](int j) {
                const int st = j & 1;
                const int slot = c_end - 1 - j;
                const int ch = slot * H + h;
                const int tok0 = p.chunk_tok0[slot];
                uint8_t* b = sm + st * kStageStride;
                mbar_expect_tx(&bar_full[st], kStageBytes);
                bulk_load_1d(dec_ring[j & 3], p.decay_end + (size_t)ch * 128, 512, &bar_full[st]);
                for (int kb = 0; kb < 2; ++kb) {
                    tma_load_2d(b + kb * 8192, &mE, &bar_full[st], kb * 64, ch * 64);
                    tma_load_2d(b + 57344 + kb * 8192, &mdO, &bar_full[st], h * 128 + kb * 64, tok0);
                }
                tma_load_2d(b + 24576, &mR, &bar_full[st], 0, ch * 128);    // R^T [key][token], K-major B
                tma_load_2d(b + 40960, &mW, &bar_full[st], 0, ch * 128);    // W^T [key][token], K-major B
                tma_load_2d(b + 16384, &mAT, &bar_full[st], 0, ch * 64);
            };
            int issued = 0;
            for (; issued < 2 && issued < n; ++issued) issue_loads(issued);
            bool ok = true;
            for (int j = 0; j + 2 < n && ok; ++j) {
                ok = mbar_wait(&bar_free[j & 1], (j >> 1) & 1, p.status, 24);
                if (ok) { issue_loads(j + 2); issued = j + 3; }
                else abort_flag = 1;
            }
            if (!ok)   // unwinding: the copies in flight must land before the block may exit
                for (int j = issued > 2 ? issued - 2 : 0; j < issued; ++j) mbar_wait(&bar_full[j & 1], (j >> 1) & 1, nullptr, 0);
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ UMMA / panel-store thread
        if (lane == 0 && n > 0) {
            const uint32_t id1a = umma_idesc_bf16(128, 64, kMajorMN, kMajorK);
            const uint32_t id1b = umma_idesc_bf16(128, 64, kMajorK, kMajorK);
            const uint32_t id2a = umma_idesc_bf16(128, 128, kMajorMN, kMajorK);
            const uint32_t id2b = umma_idesc_bf16(128, 128, kMajorK, kMajorK, 1);
            const uint32_t a_dh = smem_u32(dHop), a_dz = smem_u32(dZop);
            // the products of step j that do not depend on dH': dO^T A -> D1, dO^T R -> D2[j % 2]
            auto issue_early = [&](int j) {
                const uint32_t s0 = smem_u32(sm + (j & 1) * kStageStride);
                const uint32_t d2 = tmem + 64 + 128 * (j & 1);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)
                    umma_bf16_ss(tmem, umma_smem_desc_sw128(s0 + 57344 + k16 * 2048, 8192, 1024),
                                 umma_smem_desc_sw128(s0 + 16384 + k16 * 32, 16, 1024), id1a, k16 > 0);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)
                    umma_bf16_ss(d2, umma_smem_desc_sw128(s0 + 57344 + k16 * 2048, 8192, 1024),
                                 umma_smem_desc_sw128(s0 + 24576 + k16 * 32, 16, 1024), id2a, k16 > 0);
            };
            bool ok = mbar_wait(&bar_full[0], 0, p.status, 21);
            if (ok) {
                tc_fence_after();
                issue_early(0);
            } else abort_flag = 1;
            for (int j = 0; j < n && ok; ++j) {
                const int st = j & 1;
                const int ch = (c_end - 1 - j) * H + h;
                const uint32_t s0 = smem_u32(sm + st * kStageStride);
                // Every panel store is waited for (its read of shared memory) before the commit that lets the state
                // threads rewrite that panel: the dZ panel before mma1, the dH' panel before mma2.
                tma_store_wait_read();
                if (!mbar_wait(&bar_hop, j & 1, p.status, 25)) { abort_flag = 1; break; }
                tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < 8; ++k16)     // dZ^T += dH'^T E^T
                    umma_bf16_ss(tmem, umma_smem_desc_sw128(a_dh + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                                 umma_smem_desc_sw128(s0 + (k16 >> 2) * 8192 + (k16 & 3) * 32, 16, 1024), id1b, 1);
                umma_commit(&bar_mma1);
                tma_store_2d(&mdH, dHop, 0, ch * 128);
                tma_store_2d(&mdH, dHop + 16384, 64, ch * 128);
                tma_store_commit();
                tma_store_wait_read();
                if (!mbar_wait(&bar_zop, j & 1, p.status, 26)) { abort_flag = 1; break; }
                tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)     // D2 -= dZ^T W
                    umma_bf16_ss(tmem + 64 + 128 * st, umma_smem_desc_sw128(a_dz + k16 * 32, 16, 1024),
                                 umma_smem_desc_sw128(s0 + 40960 + k16 * 32, 16, 1024), id2b, 1);
                umma_commit(&bar_mma2);
                umma_commit(&bar_free[st]);
                tma_store_2d(&mdZT, dZop, 0, ch * 128);
                tma_store_commit();
                if (j + 1 < n) {
                    if (!mbar_wait(&bar_full[(j + 1) & 1], ((j + 1) >> 1) & 1, p.status, 21)) { abort_flag = 1; break; }
                    tc_fence_after();
                    issue_early(j + 1);
                }
            }
            tma_store_wait_all();
        }
    } else {
        // ------------------------------------------------------------------ state warpgroups
        const int kh = warp >> 2;                 // key half of this thread
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
        // this thread's half of dH' -> bf16 A operand
        auto pack_state = [&]() {
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
            mbar_arrive(&bar_hop);
        };
#ifdef KDA_PHASE_TIMING
        long long acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tlast = clock64();
#endif
        bool ok = true;
        if (n > 0) pack_state();
        for (int j = 0; j < n; ++j) {
            const int st = j & 1;
            KDA_TICKS(0);
            if (!mbar_wait(&bar_mma1, j & 1, p.status, 22) || !mbar_wait(&bar_full[st], (j >> 1) & 1, p.status, 27)) {
                abort_flag = 1; ok = false;
                break;
            }
            tc_fence_after();
            KDA_TICKS(1);
            {   // dZ^T: this thread converts tokens 32*kh .. 32*kh+31 of its row
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + 32 * kh, r);
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
            mbar_arrive(&bar_zop);
            KDA_TICKS(2);
            if (!mbar_wait(&bar_mma2, j & 1, p.status, 23)) { abort_flag = 1; ok = false; break; }
            tc_fence_after();
            KDA_TICKS(3);
            const float* dc = dec_ring[j & 3] + 64 * kh;
            const uint32_t D2 = tmem + lane_base + 64 + 128 * st + 64 * kh;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint32_t r[32];
                tmem_ld32(D2 + b * 32, r);
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
            KDA_TICKS(4);
            if (j + 1 < n) pack_state();
            KDA_TICKS(5);
        }
#ifdef KDA_PHASE_TIMING
        if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && n > 0)
            printf("scan_bwd per step: loop %lld | wait1 %lld | dZ conv %lld | wait2 %lld | update %lld | pack %lld\n",
                   acc[0] / n, acc[1] / n, acc[2] / n, acc[3] / n, acc[4] / n, acc[5] / n);
#endif
        if (ok && abort_flag == 0 && p.dh0) {
            float4* dst = reinterpret_cast<float4*>(p.dh0 + (((size_t)seq * H + h) * 128 + v) * 128 + 64 * kh);
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[j] = make_float4(dh[4 * j], dh[4 * j + 1], dh[4 * j + 2], dh[4 * j + 3]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
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
               tc_scan_fwd_kernel<<<dim3(n_seq, w.H), 448, kScanFwdSmem, st>>>(mW, mR, mE, mAT, mUT, mH, mZT, a));
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
               tc_scan_bwd_kernel<<<dim3(n_seq, w.H), 320, kScanBwdSmem, st>>>(mW, mR, mE, mAT, mdO, mdH, mdZT, a));
    return launch_status();
}

}  // namespace kda
