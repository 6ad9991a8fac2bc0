// Tensor-core lane, chunk-parallel part of the forward: one CTA per (chunk, head) builds every operand panel
// the scans consume.  K = V = 128, chunk = 64 tokens, bf16 UMMA operands, fp32 accumulation.
//
//   norms, cumulative log-decay G (fp32)                                       CUDA cores, thread = channel
//   A[t][s], M~[t][s] = sum_d (q|k)[t,d] e^{G_t-c} * k[s,d] e^{c-G_s}         tcgen05, M=128 N=64 K=128, two chains
//       c = G at the first row of the 16-row target block, so both factors stay in range for any g in [-5, 0]
//       (restates the per-tile decay centre of reference chunk_wy_forward.cu:312-376, 447-450)
//   T = (I + beta M~)^-1                                                       fp32, block forward substitution
//   U^T = P^T T^T,  W^T = Q^T T^T   (P = beta v, Q = beta e^G k)                tcgen05, M=128 N=64 K=64, MN-major A
//   R^T = (q e^G)^T, E = k e^{G_end-G}, e^{G_end}, A^T, T                       panels for the scans / backward
// Restates reference chunk_wy_forward.cu:125-405 and 761-858.

#include <cstdio>

#include "common.cuh"
#include "simt_ws.cuh"
#include "tc_common.cuh"
#include "tc_ws.cuh"

namespace kda {
namespace tc {

#ifdef KDA_PHASE_TIMING
#define KDA_TICK(n) do { if (threadIdx.x == 0 && blockIdx.y == 0 && (blockIdx.x == 0 || blockIdx.x == 100)) tick[n] = clock64(); } while (0)
#else
#define KDA_TICK(n) do { } while (0)
#endif

int make_map_bf16(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows);

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void st_bf16(uint8_t* base, uint32_t off, float x) {
    *reinterpret_cast<__nv_bfloat16*>(base + off) = __float2bfloat16(x);
}
// byte offset of element (row r, column d) of a K-major / MN-major swizzled panel whose 64-column blocks are
// `blk_bytes` apart
__device__ __forceinline__ uint32_t el_off(int r, int d, uint32_t blk_bytes) {
    return (uint32_t)(d >> 6) * blk_bytes + sw128_off(r, (d & 63) >> 3) + (uint32_t)(d & 7) * 2;
}

constexpr int kLDs = 68;

constexpr int kNT = 512;   // threads per CTA: thread (I, d) = 16-token row block I (warp >> 2), channel d (tid & 127)

// dst[S x S] = alpha * A[S x S] * B[S x S] (row-major fp32, leading dimension kLDs, 16-byte aligned columns) for NB
// independent problems addressed through the callers' pointer functions.  Each of the first S*S*NB/8 threads owns a
// 2 x 4 tile of one product, so a step of the contraction costs a warp three shared-memory wavefronts (two broadcast
// words of A, one 16-byte row piece of B) for eight multiply-adds per thread.
template <int S, int NB, class PA, class PB, class PD>
__device__ __forceinline__ void block_mm(PA pa, PB pb, PD pd, float alpha) {
    constexpr int TPP = S * S / 8;                // threads per problem
    const int tid = threadIdx.x;
    if (tid >= TPP * NB) return;
    const int prob = tid / TPP, rem = tid - prob * TPP;
    const int i0 = (rem / (S / 4)) * 2, j0 = (rem % (S / 4)) * 4;
    const float* A0 = pa(prob) + i0 * kLDs;
    const float* B = pb(prob) + j0;
    float acc[2][4];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
#pragma unroll
    for (int t = 0; t < S; ++t) {
        const float a0 = A0[t], a1 = A0[kLDs + t];
        const float4 bv = *reinterpret_cast<const float4*>(B + t * kLDs);
        acc[0][0] += a0 * bv.x; acc[0][1] += a0 * bv.y; acc[0][2] += a0 * bv.z; acc[0][3] += a0 * bv.w;
        acc[1][0] += a1 * bv.x; acc[1][1] += a1 * bv.y; acc[1][2] += a1 * bv.z; acc[1][3] += a1 * bv.w;
    }
    float* D = pd(prob) + i0 * kLDs + j0;
#pragma unroll
    for (int r = 0; r < 2; ++r)
        *reinterpret_cast<float4*>(D + r * kLDs) = make_float4(alpha * acc[r][0], alpha * acc[r][1], alpha * acc[r][2], alpha * acc[r][3]);
}

// Ts = (I + Ms)^-1 for strictly lower-triangular Ms (64x64): 8x8 diagonal solves (a short dependent chain per thread),
// then merges to 16, 32 and 64 with   inv([[A,0],[C,B]]) = [[Ai,0],[-Bi C Ai, Bi]].
__device__ void unit_lower_inverse(const float* Ms, float* Ts, float* tmp) {
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
    // 16x16 merges, four independent pairs of 8x8 blocks: tmp_p = C_p Ai_p ; T21_p = -Bi_p tmp_p
    {
        const int p = tid >> 6, i = (tid >> 3) & 7, j = tid & 7;
        if (tid < 256) {
            const float* C = Ms + (16 * p + 8 + i) * kLDs + 16 * p;
            const float* Ai = Ts + (16 * p) * kLDs + 16 * p + j;
            float a = 0.f;
#pragma unroll
            for (int t = 0; t < 8; ++t) a += C[t] * Ai[t * kLDs];
            tmp[(p * 8 + i) * kLDs + j] = a;
        }
        __syncthreads();
            if (tid < 256) {
            const float* Bi = Ts + (16 * p + 8 + i) * kLDs + 16 * p + 8;
            const float* Tm = tmp + (p * 8) * kLDs + j;
            float a = 0.f;
#pragma unroll
            for (int t = 0; t < 8; ++t) a += Bi[t] * Tm[t * kLDs];
            Ts[(16 * p + 8 + i) * kLDs + 16 * p + j] = -a;
        }
        __syncthreads();
        }
    // 32x32 merges, two independent pairs: tmp_p = C_p Ai_p ; T21_p = -Bi_p tmp_p
    block_mm<16, 2>([&](int p) { return Ms + (32 * p + 16) * kLDs + 32 * p; },
                    [&](int p) { return Ts + (32 * p) * kLDs + 32 * p; },
                    [&](int p) { return tmp + p * 16 * kLDs; }, 1.f);
    __syncthreads();
    block_mm<16, 2>([&](int p) { return Ts + (32 * p + 16) * kLDs + 32 * p + 16; },
                    [&](int p) { return tmp + p * 16 * kLDs; },
                    [&](int p) { return Ts + (32 * p + 16) * kLDs + 32 * p; }, -1.f);
    __syncthreads();
    // 64x64 merge
    block_mm<32, 1>([&](int) { return Ms + 32 * kLDs; }, [&](int) { return Ts; }, [&](int) { return tmp; }, 1.f);
    __syncthreads();
    block_mm<32, 1>([&](int) { return Ts + 32 * kLDs + 32; }, [&](int) { return tmp; },
                    [&](int) { return Ts + 32 * kLDs; }, -1.f);
    __syncthreads();
}

struct IntraFwdArgs {
    const int* chunk_tok0;
    const int* chunk_len;
    const __nv_bfloat16 *q, *k, *v;   // [tokens][H][128]
    const void* g;                    // [tokens][H][128], gate dtype
    const void* beta;                 // [tokens][H]
    int gbf16, l2norm, H;
    float scale;
    TcWs t;
    simt::Ws w;                       // per-row scalars (inverse norms, beta) kept for the backward
};

// shared-memory map (bytes from a 1024-aligned base)
constexpr int kFS0 = 0;          // 32 KB  source stack, target blocks 0|1   -> later Ms, Ts, tmp (fp32)
constexpr int kFX0 = 32768;      // 16 KB  target stack, blocks 0|1
constexpr int kFS1 = 49152;      // 32 KB  source stack, target blocks 2|3
constexpr int kFX1 = 81920;      // 16 KB  target stack, blocks 2|3          -> later T and T diag(beta) (bf16)
constexpr int kFQ = 98304;       // 16 KB  Q = beta e^G k (MN-major A)
constexpr int kFIn = 114688;     // 48 KB  q | k | v tiles (TMA)
constexpr int kFSmall = 163840;  // floats: gsum[4][128] cref[4][128] qinv[64] kinv[64] beta[64]
constexpr int kIntraFwdSmem = kFSmall + (2 * 512 + 3 * 64) * 4 + 1024;

__device__ __forceinline__ void tmem_ld16f(uint32_t taddr, float (&f)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(r[j]);
}

__global__ void __launch_bounds__(kNT, 1)
    tc_intra_fwd_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                        const __grid_constant__ CUtensorMap mv, IntraFwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* S0 = sm + kFS0;
    uint8_t* X0 = sm + kFX0;
    uint8_t* S1 = sm + kFS1;
    uint8_t* X1 = sm + kFX1;
    float* Ms = reinterpret_cast<float*>(sm);      // phase-2 view of the source/target stacks
    float* Ts = Ms + 64 * kLDs;
    float* tmp = Ts + 64 * kLDs;
    uint8_t* Tb = sm + kFX1;                       // [64 rows x 128 B] K-major B: T
    uint8_t* Tbb = sm + kFX1 + 8192;               //                              T diag(beta)
    uint8_t* Qs = sm + kFQ;
    uint8_t* qs = sm + kFIn;
    uint8_t* ks = qs + 16384;
    uint8_t* vs = ks + 16384;                      // doubles as the MN-major A operand of U^T = v^T (T diag(beta))^T
    float* gsum = reinterpret_cast<float*>(sm + kFSmall);
    float* cref = gsum + 512;
    float* qinv = cref + 512;
    float* kinv = qinv + 64;
    float* bet = kinv + 64;
    __shared__ uint64_t bar_am, bar_uw, bar_in;
    __shared__ uint32_t tmem_slot;
#ifdef KDA_PHASE_TIMING
    long long tick[12];
#endif
    const int slot = blockIdx.x, h = blockIdx.y, H = p.H;
    const int len = p.chunk_len[slot];
    if (len == 0) return;
    const int tok0 = p.chunk_tok0[slot];
    const size_t ch = (size_t)slot * H + h;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int I = warp >> 2, d = tid & 127;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    KDA_TICK(0);

    if (tid == 0) {
        mbar_init(&bar_am, 1);
        mbar_init(&bar_uw, 1);
        mbar_init(&bar_in, 1);
        mbar_fence_init();
        mbar_expect_tx(&bar_in, 49152);
        for (int kb = 0; kb < 2; ++kb) {
            tma_load_2d(qs + kb * 8192, &mq, &bar_in, h * 128 + kb * 64, tok0);
            tma_load_2d(ks + kb * 8192, &mk, &bar_in, h * 128 + kb * 64, tok0);
            tma_load_2d(vs + kb * 8192, &mv, &bar_in, h * 128 + kb * 64, tok0);
        }
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 256);

    // ---- cumulative log-decay of this thread's 16 rows (loads unconditional, row index clamped into the chunk)
    const size_t rstride = (size_t)H * 128;
    const size_t col = ((size_t)tok0 * H + h) * 128 + d;
    float G[16];
    {
#pragma unroll
        for (int r = 0; r < 16; ++r) G[r] = ld_io(p.g, col + (size_t)min(16 * I + r, len - 1) * rstride, p.gbf16);
        float run = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            run += (16 * I + r < len) ? G[r] : 0.f;
            G[r] = run;
        }
        gsum[I * 128 + d] = run;
    }
    if (tid < 64) {
        const float b = tid < len ? ld_io(p.beta, (size_t)(tok0 + tid) * H + h, p.gbf16) : 0.f;
        bet[tid] = b;
        p.w.beta[ch * 64 + tid] = b;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool ok = mbar_wait(&bar_in, 0, p.t.status, 30);
    KDA_TICK(1);
    // ---- inverse norms: one thread per row (q rows on threads 0..63, k rows on 64..127)
    if (tid < 128) {
        const int r = tid & 63;
        const uint8_t* tile = tid < 64 ? qs : ks;
        float ss = 0.f;
        if (r < len) {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                uint4 u = *reinterpret_cast<const uint4*>(tile + (c >> 3) * 8192 + sw128_off(r, c & 7));
                const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 f = __bfloat1622float2(hh[j]);
                    ss += f.x * f.x + f.y * f.y;
                }
            }
        } else if (tid < 64) {
            // rows past a ragged tail hold other tokens: blank the value rows that feed the U product
#pragma unroll
            for (int c = 0; c < 16; ++c)
                *reinterpret_cast<uint4*>(vs + (c >> 3) * 8192 + sw128_off(r, c & 7)) = make_uint4(0, 0, 0, 0);
        }
        float inv = 0.f;
        if (r < len) inv = p.l2norm ? 1.0f / fmaxf(sqrtf(ss), 1e-12f) : 1.0f;
        if (tid < 64) {
            qinv[r] = inv;
            p.w.qinv[ch * 64 + r] = inv;
        } else {
            kinv[r] = inv;
            p.w.kinv[ch * 64 + r] = inv;
        }
    }
    float gend;
    {
        const float s0 = gsum[d], s1 = gsum[128 + d], s2 = gsum[256 + d], s3 = gsum[384 + d];
        const float pre = I == 0 ? 0.f : (I == 1 ? s0 : (I == 2 ? s0 + s1 : s0 + s1 + s2));
        gend = s0 + s1 + s2 + s3;
#pragma unroll
        for (int r = 0; r < 16; ++r) G[r] += pre;
        cref[I * 128 + d] = G[0];
        if (I == 0) p.t.decay_end[ch * 128 + d] = __expf(gend);
    }
    __syncthreads();
    KDA_TICK(2);

    // ---- operand panels for this thread's 16 rows of channel d
    {
        const float c0 = cref[d], c1 = cref[128 + d], c2 = cref[256 + d], c3 = cref[384 + d];
        const float cI = I == 0 ? c0 : (I == 1 ? c1 : (I == 2 ? c2 : c3));
        const float fb0 = __expf(c1 - c0), fb1 = __expf(c2 - c1), fb2 = __expf(c3 - c2);
        uint8_t* X = (I < 2) ? X0 : X1;
        uint32_t rt[8];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int i = 16 * I + r;
            float qv = 0.f, kv = 0.f;
            if (i < len) {
                qv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(qs + el_off(i, d, 8192)));
                kv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(ks + el_off(i, d, 8192)));
            }
            const float qn = qv * qinv[i] * p.scale, kn = kv * kinv[i];
            const float gi = G[r];
            const float eG = __expf(gi);
            const float r_ = qn * eG;
            if (r & 1) rt[r >> 1] = pack2(__uint_as_float(rt[r >> 1]), r_);
            else rt[r >> 1] = __float_as_uint(r_);
            p.t.E[ch * 8192 + i * 128 + d] = __float2bfloat16(kn * __expf(gend - gi));
            st_bf16(Qs, el_off(i, d, 8192), bet[i] * eG * kn);
            // decay-masked product operands: targets relative to their own 16-row block, sources to every later block
            const float tq = __expf(gi - cI);
            const int xr = (I & 1) * 32 + r;
            st_bf16(X, el_off(xr, d, 8192), qn * tq);
            st_bf16(X, el_off(xr + 16, d, 8192), kn * tq);
            float f = kn * __expf(cI - gi);      // source row i scaled to its own block
            float s0v = 0.f, s1v = 0.f, s2v = 0.f, s3v = 0.f;
            if (I == 0) { s0v = f; f *= fb0; }
            if (I <= 1) { s1v = f; f *= fb1; }
            if (I <= 2) { s2v = f; f *= fb2; }
            s3v = f;
            st_bf16(S0, el_off(i, d, 16384), s0v);
            st_bf16(S0, el_off(64 + i, d, 16384), s1v);
            st_bf16(S1, el_off(i, d, 16384), s2v);
            st_bf16(S1, el_off(64 + i, d, 16384), s3v);
        }
        uint4* dst = reinterpret_cast<uint4*>(p.t.RT + ch * 8192 + (size_t)d * 64 + 16 * I);
        dst[0] = make_uint4(rt[0], rt[1], rt[2], rt[3]);
        dst[1] = make_uint4(rt[4], rt[5], rt[6], rt[7]);
    }
    KDA_TICK(3);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after();
        const uint32_t idesc = umma_idesc_bf16(128, 64, kMajorK, kMajorK);
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
            const uint32_t a0 = smem_u32(pr ? S1 : S0), b0 = smem_u32(pr ? X1 : X0);
#pragma unroll
            for (int k16 = 0; k16 < 8; ++k16)
                umma_bf16_ss(tmem + pr * 64, umma_smem_desc_sw128(a0 + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                             umma_smem_desc_sw128(b0 + (k16 >> 2) * 8192 + (k16 & 3) * 32, 16, 1024), idesc, k16 > 0);
        }
        umma_commit(&bar_am);
    }
    ok = mbar_wait(&bar_am, 0, p.t.status, 31) && ok;
    ok = __syncthreads_and(ok);
    tc_fence_after();
    KDA_TICK(4);
    if (ok) {
        // ---- A^T panel, M~ panel and beta*M~ (fp32) from the two accumulators.  Lane = source row (two 64-row
        // halves per chain); the four warp groups split chain x {A columns, M~ columns}.
        {
            const int m = (warp & 3) * 32 + lane;          // accumulator row
            const int half = m >> 6, s = m & 63;
            const int pr = I >> 1, sub = I & 1;            // chain, 0: A columns / 1: M~ columns
            const int Ib = 2 * pr + half;                  // target block held in these columns
            float t[16];
            tmem_ld16f(tmem + lane_base + pr * 64 + 32 * half + 16 * sub, t);
            if (sub == 0) {
                uint32_t at[8];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float a = (s <= 16 * Ib + c) ? t[c] : 0.f;
                    if (c & 1) at[c >> 1] = pack2(__uint_as_float(at[c >> 1]), a);
                    else at[c >> 1] = __float_as_uint(a);
                }
                uint4* dst = reinterpret_cast<uint4*>(p.t.AT + ch * 4096 + s * 64 + 16 * Ib);
                dst[0] = make_uint4(at[0], at[1], at[2], at[3]);
                dst[1] = make_uint4(at[4], at[5], at[6], at[7]);
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int tt = 16 * Ib + c;
                    const float mt = (s < tt) ? t[c] : 0.f;
                    Ms[tt * kLDs + s] = bet[tt] * mt;
                    if (!p.t.fwd_only) p.t.Mt[ch * 4096 + tt * 64 + s] = __float2bfloat16(mt);
                }
            }
        }
        __syncthreads();
        KDA_TICK(5);
        unit_lower_inverse(Ms, Ts, tmp);
        KDA_TICK(6);
        // ---- T: bf16 K-major B operands (plain and column-scaled by beta) and the bf16 panel; one 16-byte chunk each
        {
            const int i = tid >> 3, c16 = tid & 7;
            const float* src = Ts + i * kLDs + 8 * c16;
            const float* bb = bet + 8 * c16;
            uint4 u = make_uint4(pack2(src[0], src[1]), pack2(src[2], src[3]), pack2(src[4], src[5]), pack2(src[6], src[7]));
            *reinterpret_cast<uint4*>(Tb + sw128_off(i, c16)) = u;
            if (!p.t.fwd_only) *reinterpret_cast<uint4*>(p.t.Tp + ch * 4096 + i * 64 + 8 * c16) = u;
            *reinterpret_cast<uint4*>(Tbb + sw128_off(i, c16)) =
                make_uint4(pack2(src[0] * bb[0], src[1] * bb[1]), pack2(src[2] * bb[2], src[3] * bb[3]),
                           pack2(src[4] * bb[4], src[5] * bb[5]), pack2(src[6] * bb[6], src[7] * bb[7]));
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
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
        KDA_TICK(7);
        ok = mbar_wait(&bar_uw, 0, p.t.status, 32);
        ok = __syncthreads_and(ok);
        tc_fence_after();
        KDA_TICK(8);
        if (ok) {
            // lane = value channel (U^T) / key channel (W^T); warp groups split {U, W} x {tokens 0..31, 32..63}
            const int which = I >> 1, hb = I & 1;
            __nv_bfloat16* base = (which ? p.t.WT : p.t.UT) + ch * 8192 + (size_t)d * 64 + hb * 32;
            uint32_t r[32];
            tmem_ld32(tmem + lane_base + 128 + which * 64 + hb * 32, r);
            tmem_ld_wait();
            uint4* dst = reinterpret_cast<uint4*>(base);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                dst[c] = make_uint4(pack2(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                                    pack2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                                    pack2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                                    pack2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
        }
    }
    KDA_TICK(9);
#ifdef KDA_PHASE_TIMING
    if (threadIdx.x == 0 && blockIdx.y == 0 && (blockIdx.x == 0 || blockIdx.x == 100))
        printf("intra_fwd blk %d: g+tma %lld | norms %lld | panels %lld | mma_am %lld | readout %lld | inverse %lld | T+issue %lld | mma_uw %lld | epilogue %lld | total %lld\n",
               blockIdx.x, tick[1] - tick[0], tick[2] - tick[1], tick[3] - tick[2], tick[4] - tick[3], tick[5] - tick[4],
               tick[6] - tick[5], tick[7] - tick[6], tick[8] - tick[7], tick[9] - tick[8], tick[9] - tick[0]);
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 256);
}

}  // namespace tc

int tc_intra_forward(const simt::Ws& w, const tc::TcWs& t, const void* q, const void* k, const void* v, const void* g,
                     const void* beta, int gbf16, int l2norm, float scale, int tokens, cudaStream_t st) {
    using namespace tc;
    IntraFwdArgs a;
    a.chunk_tok0 = w.chunk_tok0; a.chunk_len = w.chunk_len;
    a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k);
    a.v = static_cast<const __nv_bfloat16*>(v);
    a.g = g; a.beta = beta; a.gbf16 = gbf16; a.l2norm = l2norm; a.H = w.H; a.scale = scale; a.t = t; a.w = w;
    CUtensorMap mq, mk, mv;
    if (make_map_bf16(&mq, q, (uint64_t)tokens, (uint64_t)w.H * 128, 64, 64) ||
        make_map_bf16(&mk, k, (uint64_t)tokens, (uint64_t)w.H * 128, 64, 64) ||
        make_map_bf16(&mv, v, (uint64_t)tokens, (uint64_t)w.H * 128, 64, 64))
        return KDA_ERR_CUDA;
    if (cudaFuncSetAttribute(tc_intra_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kIntraFwdSmem) != cudaSuccess)
        return KDA_ERR_CUDA;
    KDA_LAUNCH("tc_intra_fwd_kernel", st,
               tc_intra_fwd_kernel<<<dim3(w.nslots, w.H), kNT, kIntraFwdSmem, st>>>(mq, mk, mv, a));
    return launch_status();
}

}  // namespace kda
