// Tensor-core lane, chunk-parallel part of the forward: one CTA (256 threads, two CTAs per SM) per (chunk, head) builds
// every operand panel the scans consume.  K = V = 128, chunk = 64 tokens, bf16 UMMA operands, fp32 accumulation.
//
//   norms, cumulative log-decay G (fp32)                                       CUDA cores, thread = 4 rows x 8 channels
//   A[t][s], M~[t][s] = sum_d (q|k)[t,d] e^{G_t-c} * k[s,d] e^{c-G_s}         tcgen05, M=128 N=64 K=128, two chains
//       c = G at the first row of the 16-row target block, so both factors stay in range for any g in [-5, 0]
//       (restates the per-tile decay centre of reference chunk_wy_forward.cu:312-376, 447-450)
//   T = (I + beta M~)^-1                                                       fp32, block forward substitution
//   U^T = P^T T^T,  W^T = Q^T T^T   (P = beta v, Q = beta e^G k)                tcgen05, M=128 N=64 K=64, MN-major A
//   R^T = (q e^G)^T, E = k e^{G_end-G}, e^{G_end}, A^T, T                       panels for the scans / backward
//   Pn = W^T E,  Rm^T = R^T - W^T A^T   (the chunk's state transition)         tcgen05, M=128 N=128|64 K=64, at the end:
//       W^T is still staged in shared memory for its store, E and A^T come back by TMA into the dead value / Q tiles
// Every operand panel is written as 16-byte pieces of the 128-byte-swizzled layout the UMMA descriptors read: a thread
// owns 8 adjacent channels of 4 consecutive rows, takes q, k, g straight from global memory (a half-warp reads one
// 256-byte row segment) and needs two exponentials and one reciprocal per element.  The source panels of the two
// chains share one buffer (the second is written once the first chain has completed), which together with 256 threads
// keeps the CTA at 105 KB / <= 128 registers so that two CTAs share an SM and fill each other's waits.
// Restates reference chunk_wy_forward.cu:125-405 and 761-858.

#include <cstdio>

#include "common.cuh"
#include "simt_ws.cuh"
#include "tc_common.cuh"
#include "tc_ws.cuh"

namespace kda {
namespace tc {

int make_map_bf16(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows);

namespace {

constexpr int kLDs = 68;      // leading dimension (floats) of the 64x64 fp32 tiles of the inverse
constexpr int kNT = 256;

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}
// byte offset of the 16-byte piece holding channels 8*cg .. 8*cg+7 of row r in a K-major / MN-major swizzled panel whose
// 64-column blocks are blk_bytes apart
__device__ __forceinline__ uint32_t piece_off(int r, int cg, uint32_t blk_bytes) {
    return (uint32_t)(cg >> 3) * blk_bytes + sw128_off(r, cg & 7);
}
__device__ __forceinline__ void ld8(const void* base, size_t idx, int bf16, float (&f)[8]) {
    if (bf16) {
        unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx)), f);
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx));
        const float4 b = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx + 4));
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
}
__device__ __forceinline__ void lds8(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void sts8(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
// Per-channel tables (rows of 128 floats read 8 channels per lane): channel ch sits at ((ch >> 2) & 1) * 64 +
// (ch >> 3) * 4 + (ch & 3), i.e. the two float4 halves of a lane's 8 channels live in separate 64-float halves of the
// row, so that each of the two 16-byte accesses has a 16-byte lane stride (32 bytes would use half the banks).
// `row + 4 * cg` is the lane's address for channels 8 cg .. 8 cg + 7; element-wise passes over whole rows need no change
// as long as every table of the pass is in this order.
__device__ __forceinline__ void lds8c(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 64);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void sts8c(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 64) = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// dst = alpha * A * B for NP independent S x S problems (row-major fp32, leading dimension kLDs), all 256 threads busy:
// a thread owns one row piece of CW adjacent columns of one product.
template <int S, int NP, class PA, class PB, class PD>
__device__ __forceinline__ void tile_mm(PA pa, PB pb, PD pd, float alpha) {
    constexpr int CW = S * S * NP / kNT;          // columns per thread: 1 (8x8x4), 2 (16x16x2), 4 (32x32x1)
    constexpr int TPR = S / CW;                   // threads per row
    const int tid = threadIdx.x;
    const int prob = tid / (S * TPR), rem = tid % (S * TPR);
    const int i = rem / TPR, j0 = (rem % TPR) * CW;
    const float* A = pa(prob) + i * kLDs;
    const float* B = pb(prob) + j0;
    float acc[CW];
#pragma unroll
    for (int c = 0; c < CW; ++c) acc[c] = 0.f;
#pragma unroll
    for (int t = 0; t < S; ++t) {
        const float a = A[t];
        if (CW == 4) {
            const float4 b = *reinterpret_cast<const float4*>(B + t * kLDs);
            acc[0] += a * b.x; acc[1 % CW] += a * b.y; acc[2 % CW] += a * b.z; acc[3 % CW] += a * b.w;
        } else if (CW == 2) {
            const float2 b = *reinterpret_cast<const float2*>(B + t * kLDs);
            acc[0] += a * b.x; acc[1 % CW] += a * b.y;
        } else {
            acc[0] += a * B[t * kLDs];
        }
    }
    float* D = pd(prob) + i * kLDs + j0;
#pragma unroll
    for (int c = 0; c < CW; ++c) D[c] = alpha * acc[c];
}

// D = alpha * A * B for S x S fp32 tiles in shared memory (leading dimension kLDs) on the warp-level tensor-core path:
// mma.sync m16n8k8 with every operand split into two TF32 terms (hi + lo; lo*lo dropped), which keeps float32-class
// accuracy - T feeds every later product - while one product costs a warp S/8 short steps instead of S dependent
// shared-memory round trips.  These few 16..32-wide dependent products are latency-bound; a tcgen05 round trip
// (stage operands, issue, commit, read tensor memory back) costs more than the whole product does here.
// NP problems of S x S; a warp owns one 16 x 8 output tile; warps beyond the tile count idle.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    const float r = x - __uint_as_float(hi);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <int S, int NP, class PA, class PB, class PD>
__device__ __forceinline__ void warp_mm(PA pa, PB pb, PD pd, float alpha) {
    constexpr int TR = S / 16, TC = S / 8;         // output tiles per problem
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= NP * TR * TC) return;
    const int prob = warp / (TR * TC), tile = warp % (TR * TC);
    const int r0 = 16 * (tile / TC), c0 = 8 * (tile % TC);
    const int g = lane >> 2, tig = lane & 3;
    const float* A = pa(prob) + (r0 + g) * kLDs + tig;
    const float* B = pb(prob) + tig * kLDs + c0 + g;
    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < S / 8; ++ks) {
        uint32_t ah[4], al[4], bh[2], bl[2];
        split_tf32(A[8 * ks], ah[0], al[0]);
        split_tf32(A[8 * kLDs + 8 * ks], ah[1], al[1]);
        split_tf32(A[8 * ks + 4], ah[2], al[2]);
        split_tf32(A[8 * kLDs + 8 * ks + 4], ah[3], al[3]);
        split_tf32(B[(8 * ks) * kLDs], bh[0], bl[0]);
        split_tf32(B[(8 * ks + 4) * kLDs], bh[1], bl[1]);
        mma_tf32(d, al, bh);
        mma_tf32(d, ah, bl);
        mma_tf32(d, ah, bh);
    }
    float* D = pd(prob) + (r0 + g) * kLDs + c0 + 2 * tig;
    *reinterpret_cast<float2*>(D) = make_float2(alpha * d[0], alpha * d[1]);
    *reinterpret_cast<float2*>(D + 8 * kLDs) = make_float2(alpha * d[2], alpha * d[3]);
}

// Ts = (I + Ms)^-1 for strictly lower-triangular Ms (64x64): 8x8 diagonal solves (a short dependent chain per thread),
// then merges to 16 (CUDA cores), 32 and 64 (warp-level tensor cores) with
//   inv([[A,0],[C,B]]) = [[Ai,0],[-Bi C Ai, Bi]].
__device__ __forceinline__ void unit_lower_inverse(const float* Ms, float* Ts, float* tmp) {
    const int tid = threadIdx.x;
    for (int idx = tid; idx < 64 * kLDs / 4; idx += kNT) reinterpret_cast<float4*>(Ts)[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
    __syncthreads();
    if (tid < 64) {
        const int b = tid >> 3, j = tid & 7;          // diagonal block, column of the inverse
        const float* Lb = Ms + (8 * b) * kLDs + 8 * b;
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (i == j) ? 1.f : 0.f;
#pragma unroll
        for (int i = 1; i < 8; ++i) {
            float s = 0.f;
#pragma unroll
            for (int t = 0; t < i; ++t) s += Lb[i * kLDs + t] * x[t];
            x[i] = (i > j) ? -s : x[i];
        }
        float* Tb = Ts + (8 * b) * kLDs + 8 * b;
#pragma unroll
        for (int i = 0; i < 8; ++i) Tb[i * kLDs + j] = x[i];
    }
    __syncthreads();
    // merges: tmp_p = C_p Ai_p ; T21_p = -Bi_p tmp_p
    tile_mm<8, 4>([&](int p) { return Ms + (16 * p + 8) * kLDs + 16 * p; }, [&](int p) { return Ts + (16 * p) * kLDs + 16 * p; },
                  [&](int p) { return tmp + p * 8 * kLDs; }, 1.f);
    __syncthreads();
    tile_mm<8, 4>([&](int p) { return Ts + (16 * p + 8) * kLDs + 16 * p + 8; }, [&](int p) { return tmp + p * 8 * kLDs; },
                  [&](int p) { return Ts + (16 * p + 8) * kLDs + 16 * p; }, -1.f);
    __syncthreads();
    warp_mm<16, 2>([&](int p) { return Ms + (32 * p + 16) * kLDs + 32 * p; }, [&](int p) { return Ts + (32 * p) * kLDs + 32 * p; },
                   [&](int p) { return tmp + p * 16 * kLDs; }, 1.f);
    __syncthreads();
    warp_mm<16, 2>([&](int p) { return Ts + (32 * p + 16) * kLDs + 32 * p + 16; }, [&](int p) { return tmp + p * 16 * kLDs; },
                   [&](int p) { return Ts + (32 * p + 16) * kLDs + 32 * p; }, -1.f);
    __syncthreads();
    warp_mm<32, 1>([&](int) { return Ms + 32 * kLDs; }, [&](int) { return Ts; }, [&](int) { return tmp; }, 1.f);
    __syncthreads();
    warp_mm<32, 1>([&](int) { return Ts + 32 * kLDs + 32; }, [&](int) { return tmp; }, [&](int) { return Ts + 32 * kLDs; }, -1.f);
    __syncthreads();
}

}  // namespace

struct IntraFwdArgs {
    const int* chunk_tok0;
    const int* chunk_len;
    const __nv_bfloat16 *q, *k;       // [tokens][H][128]
    const void* g;                    // [tokens][H][128], gate dtype
    const void* beta;                 // [tokens][H]
    int gbf16, l2norm, H;
    float scale;
    TcWs t;
    simt::Ws w;                       // per-row scalars (inverse norms, beta) kept for the backward
    const __nv_bfloat16* xv;          // CONV only: the v convolution's input (q, k above are the q, k convolutions' inputs)
    ConvPrep conv;
};

// shared-memory map (bytes from a 1024-aligned base)
constexpr int kFS = 0;             // 32 KB  source stack of the chain in flight: [2 target blocks][64 rows], 2 k-blocks of 16 KB
constexpr int kFX = 32768;         // 32 KB  target stacks, chain pr at pr * 16 KB: rows (blk & 1) * 32 + {q: r, k: 16 + r}
constexpr int kFV = 65536;         // 16 KB  v tile (TMA): MN-major A of U^T = v^T (T diag(beta))^T
constexpr int kFQ = 81920;         // 16 KB  Q = beta e^G k: MN-major A of W^T = Q^T T^T
constexpr int kFTab = 98304;       // floats: cref[4][128] eC[4][128] eEnd[4][128] fb[3][128] | gend[128] | bet[64]
constexpr int kTabFloats = 15 * 128 + 128 + 64;
// after the A / M~ chains the stacks are dead: Ms, Ts, tmp (fp32) and the two bf16 T operands live in [0, 64 KB)
constexpr int kFMs = 0, kFTs = 64 * kLDs * 4, kFTmp = 2 * 64 * kLDs * 4, kFTb = 49152, kFTbb = 57344;
static_assert(kFTmp + 32 * kLDs * 4 <= kFTb, "inverse scratch overlaps the T operands");
constexpr int kIntraFwdSmem = kFTab + kTabFloats * 4 + 1024;

// y = silu(sum_m w[m] x[t - 3 + m]) for this thread's 4 rows x 8 channels from the 7 input rows it needs, in the
// arithmetic of the stand-alone convolution kernel (float32 accumulation in tap order, hardware-tanh sigmoid, one
// rounding to bf16), so that the fused call reproduces "convolution, then forward" bit for bit.
__device__ __forceinline__ void conv4_silu_rows(const uint4 (&xr)[7], const void* wgt, size_t wbase, int wf32, uint4 (&out)[4]) {
    float w[8][4];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        if (wf32) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(wgt) + wbase + 4 * c));
            w[c][0] = __bfloat162float(__float2bfloat16(f.x)); w[c][1] = __bfloat162float(__float2bfloat16(f.y));
            w[c][2] = __bfloat162float(__float2bfloat16(f.z)); w[c][3] = __bfloat162float(__float2bfloat16(f.w));
        } else {
            const uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(wgt) + wbase + 4 * c));
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
            w[c][0] = a.x; w[c][1] = a.y; w[c][2] = b.x; w[c][3] = b.y;
        }
    }
    float x[7][8];
#pragma unroll
    for (int j = 0; j < 7; ++j) unpack_bf16x8(xr[j], x[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float y[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float z = 0.f;
#pragma unroll
            for (int m = 0; m < 4; ++m) z += w[c][m] * x[j + m][c];
            float th;
            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * z));
            y[c] = z * fmaf(0.5f, th, 0.5f);
        }
        out[j] = pack8(y);
    }
}

template <bool GBF16, bool CONV>
__global__ void __launch_bounds__(kNT, 2)
    tc_intra_fwd_kernel(const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mUT,
                        const __grid_constant__ CUtensorMap mWT, const __grid_constant__ CUtensorMap mAT,
                        const __grid_constant__ CUtensorMap mMt, const __grid_constant__ CUtensorMap mE,
                        const __grid_constant__ CUtensorMap mP, const __grid_constant__ CUtensorMap mRm,
                        const __grid_constant__ CUtensorMap mTp, IntraFwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
    uint8_t* Sst = sm + kFS;
    uint8_t* vs = sm + kFV;
    uint8_t* Qs = sm + kFQ;
    float* cref = reinterpret_cast<float*>(sm + kFTab);      // [4][128] G at the first row of each 16-row block
    float* eC = cref + 512;                                  // [4][128] exp(cref)
    float* eEnd = eC + 512;                                  // [4][128] exp(G_end - cref)
    float* fbk = eEnd + 512;                                 // [3][128] exp(cref[I+1] - cref[I])
    float* gends = fbk + 384;                                // [128]    G_end
    float* bet = gends + 128;                                // [64]
    float* wtot = reinterpret_cast<float*>(sm + kFS);        // [8][128] per-warp sums of g (dead before the stacks are written)
    float* Ms = reinterpret_cast<float*>(sm + kFMs);
    float* Ts = reinterpret_cast<float*>(sm + kFTs);
    float* tmp = reinterpret_cast<float*>(sm + kFTmp);
    uint8_t* Tb = sm + kFTb;                                 // [64 rows x 128 B] K-major B: T
    uint8_t* Tbb = sm + kFTbb;                               //                              T diag(beta)
    __shared__ uint64_t bar_in, bar_am[2], bar_uw, bar_tr;
    __shared__ uint32_t tmem_slot;

    const int slot = blockIdx.x, h = blockIdx.y, H = p.H;
    const int len = p.chunk_len[slot];
    if (len == 0) return;
    const int tok0 = p.chunk_tok0[slot];
    const size_t ch = (size_t)slot * H + h;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cg = lane & 15;                      // channels 8*cg .. 8*cg+7
    const int rq = 2 * warp + (lane >> 4);         // rows 4*rq .. 4*rq+3
    const int J = warp >> 1;                       // 16-row block of this thread's rows
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

    if (tid == 0) {
        mbar_init(&bar_in, 1);
        mbar_init(&bar_am[0], 1);
        mbar_init(&bar_am[1], 1);
        mbar_init(&bar_uw, 1);
        mbar_init(&bar_tr, 1);
        mbar_fence_init();
        if (!CONV) {
            mbar_expect_tx(&bar_in, 16384);
            for (int kb = 0; kb < 2; ++kb) tma_load_2d(vs + kb * 8192, &mv, &bar_in, h * 128 + kb * 64, tok0);
        }
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 256);

    // ---- loads: this thread's 4 rows x 8 channels of g, q, k (row index clamped into the chunk, values masked)
    const size_t rstride = (size_t)H * 128;
    const size_t base = ((size_t)tok0 * H + h) * 128 + 8 * cg;
    float G[4][8];
    uint4 qraw[4], kraw[4];
    float brow[4];
    if constexpr (CONV) {
        // the three convolutions, one after the other (7 input rows for 4 output rows; the rows before the chunk belong to
        // the previous chunk of the same sequence, or are the zero padding at a sequence start); v goes straight into the
        // operand tile that TMA would have filled
        const bool first = p.w.seq_chunk0[p.w.chunk_seq[slot]] == slot;
        const size_t wbase = ((size_t)h * 128 + 8 * cg) * 4;
        auto rows = [&](const __nv_bfloat16* x, uint4 (&xr)[7]) {
#pragma unroll
            for (int jj = 0; jj < 7; ++jj) {
                const int i = 4 * rq - 3 + jj;
                const long long ic = min(i, len - 1);      // rows past the tail feed masked outputs only
                xr[jj] = (i >= 0 || !first) ? __ldg(reinterpret_cast<const uint4*>(x + (long long)base + ic * (long long)rstride))
                                            : make_uint4(0, 0, 0, 0);
            }
        };
        uint4 xr[7];
        rows(p.q, xr);
        conv4_silu_rows(xr, p.conv.w[0], wbase, p.conv.wf32, qraw);
        rows(p.k, xr);
        conv4_silu_rows(xr, p.conv.w[1], wbase, p.conv.wf32, kraw);
        rows(p.xv, xr);
        uint4 vr[4];
        conv4_silu_rows(xr, p.conv.w[2], wbase, p.conv.wf32, vr);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * rq + j;
            *reinterpret_cast<uint4*>(vs + piece_off(i, cg, 8192)) = i < len ? vr[j] : make_uint4(0, 0, 0, 0);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = 4 * rq + j, ic = min(i, len - 1);
        ld8(p.g, base + (size_t)ic * rstride, GBF16, G[j]);
        if constexpr (!CONV) {
            qraw[j] = __ldg(reinterpret_cast<const uint4*>(p.q + base + (size_t)ic * rstride));
            kraw[j] = __ldg(reinterpret_cast<const uint4*>(p.k + base + (size_t)ic * rstride));
        }
        brow[j] = ld_io(p.beta, (size_t)(tok0 + ic) * H + h, GBF16);
        if (i >= len) {
#pragma unroll
            for (int c = 0; c < 8; ++c) G[j][c] = 0.f;
            qraw[j] = make_uint4(0, 0, 0, 0);
            kraw[j] = make_uint4(0, 0, 0, 0);
            brow[j] = 0.f;
        }
    }
    // ---- cumulative log-decay: within the thread, across the two half-warps, then across warps through shared memory
#pragma unroll
    for (int j = 1; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 8; ++c) G[j][c] += G[j - 1][c];
    float pre[8];      // sum of the rows of the other half-warp (added to the upper half's rows)
#pragma unroll
    for (int c = 0; c < 8; ++c) pre[c] = __shfl_xor_sync(0xffffffffu, G[3][c], 16);
    if (lane < 16) {
        float tot[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) tot[c] = G[3][c] + pre[c];
        sts8c(wtot + warp * 128 + 4 * cg, tot);
#pragma unroll
        for (int c = 0; c < 8; ++c) pre[c] = 0.f;
    }
    // ---- inverse norms of this thread's rows: 16 lanes hold one row
    float qi[4], ki[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float fq[8], fk[8];
        unpack_bf16x8(qraw[j], fq);
        unpack_bf16x8(kraw[j], fk);
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            sq += fq[c] * fq[c];
            sk += fk[c] * fk[c];
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            sk += __shfl_xor_sync(0xffffffffu, sk, o);
        }
        const bool valid = 4 * rq + j < len;
        qi[j] = valid ? (p.l2norm ? rsqrtf(fmaxf(sq, 1e-24f)) : 1.0f) : 0.f;      // 1 / max(|q|, 1e-12)
        ki[j] = valid ? (p.l2norm ? rsqrtf(fmaxf(sk, 1e-24f)) : 1.0f) : 0.f;
        if (cg == 0) {
            const int i = 4 * rq + j;
            bet[i] = brow[j];
            p.w.beta[ch * 64 + i] = brow[j];
            p.w.qinv[ch * 64 + i] = qi[j];
            p.w.kinv[ch * 64 + i] = ki[j];
        }
        qi[j] *= p.scale;
    }
    tc_fence_before();
    __syncthreads();                                   // (1) warp sums, TMEM slot
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    {
        float gend[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) gend[c] = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 8; ++w2) {
            float t[8];
            lds8c(wtot + w2 * 128 + 4 * cg, t);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                gend[c] += t[c];
                pre[c] += (w2 < warp) ? t[c] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) G[j][c] += pre[c];
        if ((rq & 3) == 0) sts8c(cref + J * 128 + 4 * cg, G[0]);      // first row of block J
        if (rq == 0) {
            sts8c(gends + 4 * cg, gend);
            float e[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) e[c] = __expf(gend[c]);
            float* de = p.t.decay_end + ch * 128 + 8 * cg;
            *reinterpret_cast<float4*>(de) = make_float4(e[0], e[1], e[2], e[3]);
            *reinterpret_cast<float4*>(de + 4) = make_float4(e[4], e[5], e[6], e[7]);
        }
    }
    __syncthreads();                                   // (2) block references; wtot is dead from here
    // per (block, channel) factors, 512 + 384 entries over 256 threads
    for (int e = tid; e < 512; e += kNT) {
        const int I = e >> 7, d = e & 127;
        const float c = cref[e];
        eC[e] = __expf(c);
        eEnd[e] = __expf(gends[d] - c);
        if (I < 3) fbk[e] = __expf(cref[e + 128] - c);
    }
    __syncthreads();                                   // (3) tables

    // ---- operand panels, one row at a time: 16-byte pieces of the swizzled layouts
    {
        float cJ[8];
        lds8c(cref + J * 128 + 4 * cg, cJ);
        uint8_t* X = sm + kFX + (J >> 1) * 16384;
        __nv_bfloat16* Eg = p.t.E + ch * 8192 + 8 * cg;
        uint32_t rt[8][2];                             // R^T: channel c, rows 4rq .. 4rq+3 as two bf16 pairs
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * rq + j, r16 = i & 15;
            float fq[8], fk[8], ec[8], ee[8], f0[8], o8[8];
            unpack_bf16x8(qraw[j], fq);
            unpack_bf16x8(kraw[j], fk);
            lds8c(eC + J * 128 + 4 * cg, ec);
            lds8c(eEnd + J * 128 + 4 * cg, ee);
            float tq[8], inv[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                tq[c] = __expf(G[j][c] - cJ[c]);       // e^{G - c_J} in (0, 1]
                inv[c] = fast_rcp(tq[c]);              // e^{c_J - G}
                fq[c] *= qi[j];
                fk[c] *= ki[j];
            }
            const int xr = (J & 1) * 32 + r16;
#pragma unroll
            for (int c = 0; c < 8; ++c) o8[c] = fq[c] * tq[c];
            *reinterpret_cast<uint4*>(X + piece_off(xr, cg, 8192)) = pack8(o8);
#pragma unroll
            for (int c = 0; c < 8; ++c) o8[c] = fk[c] * tq[c];
            *reinterpret_cast<uint4*>(X + piece_off(xr + 16, cg, 8192)) = pack8(o8);
#pragma unroll
            for (int c = 0; c < 8; ++c) f0[c] = fk[c] * inv[c];      // source row scaled to its own block
            if (J <= 1) {                              // chain 0: target blocks 0, 1
                if (J == 0) {
                    *reinterpret_cast<uint4*>(Sst + piece_off(i, cg, 16384)) = pack8(f0);
                    float fb[8];
                    lds8c(fbk + 4 * cg, fb);
#pragma unroll
                    for (int c = 0; c < 8; ++c) o8[c] = f0[c] * fb[c];
                    *reinterpret_cast<uint4*>(Sst + piece_off(64 + i, cg, 16384)) = pack8(o8);
                } else {
                    *reinterpret_cast<uint4*>(Sst + piece_off(64 + i, cg, 16384)) = pack8(f0);
                }
            }
            // E = k e^{G_end - G} (global, token-major), Q = beta e^G k, R = q e^G
#pragma unroll
            for (int c = 0; c < 8; ++c) o8[c] = f0[c] * ee[c];
            *reinterpret_cast<uint4*>(Eg + (size_t)i * 128) = pack8(o8);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float eg = tq[c] * ec[c];        // e^G
                o8[c] = brow[j] * eg * fk[c];
                const float r = fq[c] * eg;
                if (j & 1) rt[c][j >> 1] = pack2(__uint_as_float(rt[c][j >> 1]), r);
                else rt[c][j >> 1] = __float_as_uint(r);
            }
            *reinterpret_cast<uint4*>(Qs + piece_off(i, cg, 8192)) = pack8(o8);
        }
        __nv_bfloat16* Rg = p.t.RT + ch * 8192 + (size_t)(8 * cg) * 64 + 4 * rq;
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint2*>(Rg + c * 64) = make_uint2(rt[c][0], rt[c][1]);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();                                   // (4) chain-0 operands complete
    auto issue_am = [&](int pr) {
        tc_fence_after();
        const uint32_t idesc = umma_idesc_bf16(128, 64, kMajorK, kMajorK);
        const uint32_t a0 = smem_u32(Sst), b0 = smem_u32(sm + kFX + pr * 16384);
#pragma unroll
        for (int k16 = 0; k16 < 8; ++k16)
            umma_bf16_ss(tmem + pr * 64, umma_smem_desc_sw128(a0 + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                         umma_smem_desc_sw128(b0 + (k16 >> 2) * 8192 + (k16 & 3) * 32, 16, 1024), idesc, k16 > 0);
        umma_commit(&bar_am[pr]);
    };
    if (tid == 0) issue_am(0);
    // ---- chain 1 (target blocks 2, 3): its source rows go into the same buffer once chain 0 has read it
    bool ok = mbar_wait(&bar_am[0], 0, p.t.status, 31);
    {
        float c2[8];
        lds8c(cref + 2 * 128 + 4 * cg, c2);
        float fb2[8];
        lds8c(fbk + 2 * 128 + 4 * cg, fb2);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * rq + j;
            float fk[8], s2[8], s3[8];
            unpack_bf16x8(kraw[j], fk);
            if (J <= 2) {
                // e^{c_2 - G} for rows of blocks 0..2 (for block 2 this is the own-block factor)
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    s2[c] = fk[c] * ki[j] * __expf(c2[c] - G[j][c]);
                    s3[c] = s2[c] * fb2[c];
                }
                *reinterpret_cast<uint4*>(Sst + piece_off(i, cg, 16384)) = pack8(s2);
            } else {
                float c3[8];
                lds8c(cref + 3 * 128 + 4 * cg, c3);
#pragma unroll
                for (int c = 0; c < 8; ++c) s3[c] = fk[c] * ki[j] * __expf(c3[c] - G[j][c]);
            }
            *reinterpret_cast<uint4*>(Sst + piece_off(64 + i, cg, 16384)) = pack8(s3);
        }
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);                        // (5) chain-1 operands complete
    if (tid == 0 && ok) issue_am(1);
    ok = mbar_wait(&bar_am[1], 0, p.t.status, 31) && ok;
    ok = __syncthreads_and(ok);                        // (6) both accumulators complete, stacks dead
    tc_fence_after();
    if (ok) {
        // ---- A^T panel, M~ panel and beta*M~ (fp32) from the two accumulators.  Lane = source row within a 64-row half;
        // warps 0-3 read chain 0, warps 4-7 chain 1; 32 columns: 16 of A (q targets), 16 of M~ (k targets).
        {
            const int m = (warp & 3) * 32 + lane;
            const int half = m >> 6, s = m & 63, pr = warp >> 2;
            const int Ib = 2 * pr + half;              // target block held in these columns
            uint32_t t[32];
            tmem_ld32(tmem + lane_base + pr * 64 + 32 * half, t);
            tmem_ld_wait();
            uint32_t at[8];
#pragma unroll
            for (int c = 0; c < 16; c += 2) {
                const float a0 = (s <= 16 * Ib + c) ? __uint_as_float(t[c]) : 0.f;
                const float a1 = (s <= 16 * Ib + c + 1) ? __uint_as_float(t[c + 1]) : 0.f;
                at[c >> 1] = pack2(a0, a1);
            }
            // both panels leave through shared memory (the T operands' region is still free) as one TMA store each
            uint8_t* ATs = sm + kFTb;              // [64 s][64 i]  bf16, 128-byte swizzle
            uint8_t* Mts = sm + kFTb + 8192;       // [64 tt][64 s]
            *reinterpret_cast<uint4*>(ATs + sw128_off(s, 2 * Ib)) = make_uint4(at[0], at[1], at[2], at[3]);
            *reinterpret_cast<uint4*>(ATs + sw128_off(s, 2 * Ib + 1)) = make_uint4(at[4], at[5], at[6], at[7]);
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const int tt = 16 * Ib + c;
                const float mt = (s < tt) ? __uint_as_float(t[16 + c]) : 0.f;
                Ms[tt * kLDs + s] = bet[tt] * mt;
                *reinterpret_cast<__nv_bfloat16*>(Mts + sw128_off(tt, s >> 3) + (s & 7) * 2) = __float2bfloat16(mt);
            }
        }
        fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            tma_store_2d(&mAT, sm + kFTb, 0, (int)(ch * 64));
            if (!p.t.fwd_only) tma_store_2d(&mMt, sm + kFTb + 8192, 0, (int)(ch * 64));
            tma_store_commit();
        }
        unit_lower_inverse(Ms, Ts, tmp);
        if (tid == 0) tma_store_wait_read();       // the staging region becomes the T operands below
        __syncthreads();
        // ---- T: bf16 K-major B operands (plain and column-scaled by beta); 32 bytes of a row each, lanes on
        // consecutive rows (272 bytes apart: every 16-byte access of a quarter-warp lands in its own banks).  The plain
        // operand tile is the T panel as TMA lays it out, so the panel is stored from it below.
        {
            const int i = tid & 63, seg = tid >> 6;
            const float* src = Ts + i * kLDs + 16 * seg;
            const float* bb = bet + 16 * seg;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float x[8], b8[8];
                lds8(src + 8 * hh, x);
                lds8(bb + 8 * hh, b8);
                const uint4 u = pack8(x);
                *reinterpret_cast<uint4*>(Tb + sw128_off(i, 2 * seg + hh)) = u;
#pragma unroll
                for (int c = 0; c < 8; ++c) x[c] *= b8[c];
                *reinterpret_cast<uint4*>(Tbb + sw128_off(i, 2 * seg + hh)) = pack8(x);
            }
        }
        // the value tile: wait for it, blank the rows past a ragged tail (they hold other tokens)
        if (!CONV) ok = mbar_wait(&bar_in, 0, p.t.status, 30);
        if (!CONV && len < 64 && ok) {
            for (int idx = tid; idx < (64 - len) * 16; idx += kNT) {
                const int r = len + (idx >> 4), c = idx & 15;
                *reinterpret_cast<uint4*>(vs + (c >> 3) * 8192 + sw128_off(r, c & 7)) = make_uint4(0, 0, 0, 0);
            }
        }
        fence_async_smem();
        // the E rows this block wrote with plain stores long ago come back by a bulk load below: order them for it
        __threadfence();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        tc_fence_before();
        ok = __syncthreads_and(ok);
        if (tid == 0 && ok) {
            if (!p.t.fwd_only) {                   // kept for the backward only
                tma_store_2d(&mTp, Tb, 0, (int)(ch * 64));
                tma_store_commit();
            }
            tc_fence_after();
            const uint32_t idesc = umma_idesc_bf16(128, 64, kMajorMN, kMajorK);
            const uint32_t b0 = smem_u32(Tb), b1 = smem_u32(Tbb);
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16)     // U^T = v^T (T diag(beta))^T
                umma_bf16_ss(tmem + 128, umma_smem_desc_sw128(smem_u32(vs) + k16 * 2048, 8192, 1024),
                             umma_smem_desc_sw128(b1 + k16 * 32, 16, 1024), idesc, k16 > 0);
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16)     // W^T = Q^T T^T
                umma_bf16_ss(tmem + 192, umma_smem_desc_sw128(smem_u32(Qs) + k16 * 2048, 8192, 1024),
                             umma_smem_desc_sw128(b0 + k16 * 32, 16, 1024), idesc, k16 > 0);
            umma_commit(&bar_uw);
        }
        if (ok) ok = mbar_wait(&bar_uw, 0, p.t.status, 32);
        tc_fence_after();
        // ---- chunk transition, fused: Pn = W^T E and Rm^T = R^T - W^T A^T need W^T (about to be staged below), E and
        // A^T.  The value and Q tiles are dead now: E and A^T come back into them by TMA while the panels are read out.
        const int kt = (warp & 3) * 32 + lane, gt = warp >> 2;      // transition read-out: key row, column half
        uint4 rtv[4];
        if (tid == 0 && ok) {
            tma_store_wait_all();                  // the A^T panel stored above is complete in global memory
            mbar_expect_tx(&bar_tr, 16384 + (p.t.fwd_only ? 0 : 8192));
            for (int nb = 0; nb < 2; ++nb) tma_load_2d(vs + nb * 8192, &mE, &bar_tr, nb * 64, (int)(ch * 64));
            if (!p.t.fwd_only) tma_load_2d(Qs, &mAT, &bar_tr, 0, (int)(ch * 64));
        }
        if (ok && !p.t.fwd_only) {
            const uint4* src = reinterpret_cast<const uint4*>(p.t.RT + ch * 8192 + (size_t)kt * 64 + 32 * gt);
#pragma unroll
            for (int j = 0; j < 4; ++j) rtv[j] = src[j];
        }
        if (ok) {
            // lane = value channel (U^T, warps 0-3) / key channel (W^T, warps 4-7): one 128-byte panel row per thread,
            // staged in the swizzled layout (the inverse's scratch is dead) and stored by TMA, 16 KB per panel
            const int which = warp >> 2;
            const int d = (warp & 3) * 32 + lane;
            uint8_t* stg = sm + which * 16384;
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + 128 + which * 64 + hb * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(stg + sw128_off(d, 4 * hb + c)) =
                        make_uint4(pack2(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                                   pack2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                                   pack2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                                   pack2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
            }
        }
        fence_async_smem();
        tc_fence_before();
        ok = __syncthreads_and(ok);
        if (tid == 0 && ok) {
            tma_store_2d(&mUT, sm, 0, (int)(ch * 128));
            tma_store_2d(&mWT, sm + 16384, 0, (int)(ch * 128));
            tma_store_commit();
            ok = mbar_wait(&bar_tr, 0, p.t.status, 33);
            if (ok) {
                tc_fence_after();
                // every accumulator column has been read out: Pn takes columns 0..127, (A W)^T columns 128..191
                const uint32_t a0 = smem_u32(sm + 16384), bE = smem_u32(vs), bA = smem_u32(Qs);
                const uint32_t id128 = umma_idesc_bf16(128, 128, kMajorK, kMajorMN);
                const uint32_t id64 = umma_idesc_bf16(128, 64, kMajorK, kMajorMN);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16)     // Pn = W^T E
                    umma_bf16_ss(tmem, umma_smem_desc_sw128(a0 + k16 * 32, 16, 1024),
                                 umma_smem_desc_sw128(bE + k16 * 2048, 8192, 1024), id128, k16 > 0);
                if (!p.t.fwd_only) {
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)     // (A W)^T = W^T A^T
                        umma_bf16_ss(tmem + 128, umma_smem_desc_sw128(a0 + k16 * 32, 16, 1024),
                                     umma_smem_desc_sw128(bA + k16 * 2048, 8192, 1024), id64, k16 > 0);
                }
                umma_commit(&bar_uw);
            }
        }
        if (ok) ok = mbar_wait(&bar_uw, 1, p.t.status, 34);      // no block-wide barrier: the staging below overwrites only what
        tc_fence_after();                                         // the completed products were the last to read
        if (ok) {
            // both results leave through shared memory in the swizzled layout (Pn over the dead T operands and inverse
            // scratch, Rm^T over the E tile the products have finished reading) and are stored by TMA
            uint8_t* Pst = sm + 32768 + gt * 16384;          // [128 key rows][64 columns of half gt]
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + 64 * gt + 32 * b, r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(Pst + sw128_off(kt, 4 * b + c)) =
                        make_uint4(pack2(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                                   pack2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                                   pack2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                                   pack2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
            }
            if (!p.t.fwd_only) {     // the adjoint scan's operand is not needed in a forward-only call
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + 128 + 32 * gt, r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float f[8];
                    unpack_bf16x8(rtv[c], f);
                    *reinterpret_cast<uint4*>(vs + sw128_off(kt, 4 * gt + c)) =
                        make_uint4(pack2(f[0] - __uint_as_float(r[8 * c]), f[1] - __uint_as_float(r[8 * c + 1])),
                                   pack2(f[2] - __uint_as_float(r[8 * c + 2]), f[3] - __uint_as_float(r[8 * c + 3])),
                                   pack2(f[4] - __uint_as_float(r[8 * c + 4]), f[5] - __uint_as_float(r[8 * c + 5])),
                                   pack2(f[6] - __uint_as_float(r[8 * c + 6]), f[7] - __uint_as_float(r[8 * c + 7])));
                }
            }
        }
        fence_async_smem();
        ok = __syncthreads_and(ok);
        if (tid == 0 && ok) {
            for (int nb = 0; nb < 2; ++nb) tma_store_2d(&mP, sm + 32768 + nb * 16384, nb * 64, (int)(ch * 128));
            if (!p.t.fwd_only) tma_store_2d(&mRm, vs, 0, (int)(ch * 128));
            tma_store_commit();
        }
        if (tid == 0) tma_store_wait_read();           // shared memory must outlive the reads of the bulk stores
    } else {
        // unwinding: the value tile must have landed before the block may exit
        if (!CONV) mbar_wait(&bar_in, 0, nullptr, 0);
        if (tid == 0) tma_store_wait_read();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 256);
}

}  // namespace tc

int tc_intra_forward(const simt::Ws& w, const tc::TcWs& t, const void* q, const void* k, const void* v, const void* g,
                     const void* beta, int gbf16, int l2norm, float scale, int tokens, const tc::ConvPrep* conv, cudaStream_t st) {
    using namespace tc;
    IntraFwdArgs a;
    a.chunk_tok0 = w.chunk_tok0; a.chunk_len = w.chunk_len;
    a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k);
    a.g = g; a.beta = beta; a.gbf16 = gbf16; a.l2norm = l2norm; a.H = w.H; a.scale = scale; a.t = t; a.w = w;
    a.xv = static_cast<const __nv_bfloat16*>(v);
    a.conv = conv != nullptr ? *conv : tc::ConvPrep{{nullptr, nullptr, nullptr}, 0};
    if (conv != nullptr && !t.fwd_only) return KDA_ERR_UNSUPPORTED;      // a backward would need q, k, v in memory
    const uint64_t nch = (uint64_t)w.nslots * w.H;
    CUtensorMap mv, mUT, mWT, mAT, mMt, mE, mP, mRm, mTp;
    int rc = make_map_bf16(&mv, v, (uint64_t)tokens, (uint64_t)w.H * 128, 64, 64);
    rc |= make_map_bf16(&mUT, t.UT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mWT, t.WT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mAT, t.AT, nch * 64, 64, 64, 64);
    rc |= make_map_bf16(&mMt, t.fwd_only ? t.AT : t.Mt, nch * 64, 64, 64, 64);      // not stored in a forward-only call
    rc |= make_map_bf16(&mE, t.E, nch * 64, 128, 64, 64);
    rc |= make_map_bf16(&mTp, t.fwd_only ? t.AT : t.Tp, nch * 64, 64, 64, 64);      // not stored in a forward-only call
    rc |= make_map_bf16(&mP, t.Pn, nch * 128, 128, 64, 128);
    rc |= make_map_bf16(&mRm, t.fwd_only ? t.WT : t.RmT, nch * 128, 64, 64, 128);      // not stored in a forward-only call
    if (rc) return KDA_ERR_CUDA;
    auto kern = conv != nullptr ? (gbf16 ? tc_intra_fwd_kernel<true, true> : tc_intra_fwd_kernel<false, true>)
                                : (gbf16 ? tc_intra_fwd_kernel<true, false> : tc_intra_fwd_kernel<false, false>);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kIntraFwdSmem) != cudaSuccess) return KDA_ERR_CUDA;
    KDA_LAUNCH("tc_intra_fwd_kernel", st, kern<<<dim3(w.nslots, w.H), kNT, kIntraFwdSmem, st>>>(mv, mUT, mWT, mAT, mMt, mE, mP, mRm, mTp, a));
    return launch_status();
}

}  // namespace kda
