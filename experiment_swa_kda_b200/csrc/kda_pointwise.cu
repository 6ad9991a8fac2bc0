// Bandwidth-bound KDA kernels: gate activations, recurrent decode step, short causal
// depthwise convolution (+SiLU) and gated RMSNorm, forward and backward.  All are
// HBM-bound: wide coalesced loads, warp-shuffle reductions, deterministic two-stage
// reductions for the weight gradients (no floating-point atomics).

#include <algorithm>

#include <type_traits>

#include "common.cuh"

namespace kda {
namespace pw {

// sigmoid for the bf16 I/O paths: one hardware tanh (relative error 2^-11, far inside bf16 rounding) instead of an
// exponential and a reciprocal - these kernels are bound by instruction issue, not by DRAM; float32 I/O keeps expf and a
// true divide
template <bool FAST>
__device__ __forceinline__ float sigmoid_t(float x) {
    if (FAST) {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
        return fmaf(0.5f, t, 0.5f);
    }
    return 1.0f / (1.0f + expf(-x));
}

// =============================================================================================
// gate / beta activations
// =============================================================================================
__global__ void gate_fwd_kernel(size_t n_gate, size_t n_beta, int H, int K, int bf16, const void* __restrict__ raw,
                                const void* __restrict__ bl, const float* __restrict__ A_log,
                                const float* __restrict__ dt_bias, float lb, float* __restrict__ g,
                                float* __restrict__ beta) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_gate; i += stride) {
        const int kk = (int)(i % K), h = (int)((i / K) % H);
        const float z = expf(A_log[h]) * (ld_io(raw, i, bf16) + dt_bias[h * K + kk]);
        g[i] = lb * sigmoidf_(z);
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_beta; i += stride)
        beta[i] = sigmoidf_(ld_io(bl, i, bf16));
}

constexpr int kGateRows = 32;  // tokens per first-stage reduction block

// stage 1: d_raw, d_beta_logits and per-block column partials of ddt_bias / dA_log
__global__ void gate_bwd_kernel(int tokens, int H, int K, int bf16, const void* __restrict__ raw,
                                const void* __restrict__ bl, const float* __restrict__ A_log,
                                const float* __restrict__ dt_bias, float lb, const float* __restrict__ dg,
                                const float* __restrict__ dbeta, void* __restrict__ d_raw, void* __restrict__ d_bl,
                                float* __restrict__ part_b, float* __restrict__ part_a) {
    const int HK = H * K;
    const int t0 = blockIdx.x * kGateRows, t1 = min(tokens, t0 + kGateRows);
    for (int c = threadIdx.x; c < HK; c += blockDim.x) {
        const int h = c / K;
        const float ea = expf(A_log[h]), bias = dt_bias[c];
        float sb = 0.f, sa = 0.f;
        for (int t = t0; t < t1; ++t) {
            const size_t i = (size_t)t * HK + c;
            const float x = ld_io(raw, i, bf16) + bias;
            const float sg = sigmoidf_(ea * x);
            const float dr = dg[i] * lb * sg * (1.f - sg) * ea;
            st_io(d_raw, i, bf16, dr);
            sb += dr;
            sa += dr * x;
        }
        part_b[(size_t)blockIdx.x * HK + c] = sb;
        part_a[(size_t)blockIdx.x * HK + c] = sa;
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        for (int t = t0; t < t1; ++t) {
            const size_t i = (size_t)t * H + c;
            const float b = sigmoidf_(ld_io(bl, i, bf16));
            st_io(d_bl, i, bf16, dbeta[i] * b * (1.f - b));
        }
    }
}

// stage 2: one block per head, 1024 threads = 8 row segments x 128 columns (wider heads loop over column groups);
// fixed summation order
__global__ void __launch_bounds__(1024) gate_bwd_reduce_kernel(int nblk, int H, int K, const float* __restrict__ part_b,
                                                               const float* __restrict__ part_a, float* __restrict__ ddt_bias,
                                                               float* __restrict__ dA_log) {
    __shared__ float redb[8][128], reda[8][128];
    __shared__ float wsum[4];
    const int h = blockIdx.x, HK = H * K;
    const int col = threadIdx.x & 127, seg = threadIdx.x >> 7;
    float accA = 0.f;                      // segment 0 only: this column's share of sum_k (dr * x), over all column groups
    for (int k0 = 0; k0 < K; k0 += 128) {
        const int kk = k0 + col, c = h * K + kk;
        float sb = 0.f, sa = 0.f;
        if (kk < K)
            for (int b = seg; b < nblk; b += 8) {
                sb += part_b[(size_t)b * HK + c];
                sa += part_a[(size_t)b * HK + c];
            }
        redb[seg][col] = sb;
        reda[seg][col] = sa;
        __syncthreads();
        if (seg == 0 && kk < K) {
            float tb = 0.f, ta = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                tb += redb[r][col];
                ta += reda[r][col];
            }
            ddt_bias[c] = tb;
            accA += ta;
        }
        __syncthreads();
    }
    if (seg == 0) {                        // 4 warps hold the head's column sums: warp totals, then one thread
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) accA += __shfl_xor_sync(0xffffffffu, accA, o);
        if ((col & 31) == 0) wsum[col >> 5] = accA;
    }
    __syncthreads();
    if (threadIdx.x == 0) dA_log[h] = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
}

// =============================================================================================
// recurrent decode step
//   S' = S * exp(g);  r = v - k^T S';  S'' = S' + beta k r^T;  o = q^T S''
// The state is V-first [n_seq,H,V,K]: a row (fixed value index) is K contiguous floats.  One
// warp owns a row at a time: a single coalesced read and a single coalesced write per row, two
// shuffle reductions, and o_v = q.S'_v + beta r_v (q.k) so the row is never re-read.
// =============================================================================================
// NV4 > 0: K % 4 == 0, lane owns NV4 float4 of a row (keys 128*j + 4*lane + 0..3); NV4 == 0: scalar layout,
// lane owns keys lane + 32*e.  R rows are kept in flight per warp; every load is issued unconditionally
// (addresses clamped, values masked) so the loads of a row group overlap.
// When raw.A_log is set, g and beta hold the raw gate logits and beta logits instead and are activated here
// (g = lb * sigmoid(exp(A_log[h]) * (raw + dt_bias[h,k])), beta = sigmoid(logit)): one launch less per token and layer.
struct RawGate {
    const float* A_log;      // [H], or nullptr: g and beta are already activated
    const float* dt_bias;    // [H*K]
    float lb;
};

template <int NV4, int R>
__global__ void __launch_bounds__(256) decode_kernel(int H, int K, int V, int bf16, int gbf16, int l2norm, float scale,
                                                     const void* __restrict__ q, const void* __restrict__ k,
                                                     const void* __restrict__ v, const void* __restrict__ g,
                                                     const void* __restrict__ beta, const float* s_in, float* s_out,
                                                     void* __restrict__ o, int rows_per_cta, RawGate raw) {
    constexpr int NE = NV4 > 0 ? 4 * NV4 : 8;     // state elements per lane per row
    const int bh = blockIdx.x;                    // sequence * H + head
    const int v_base = blockIdx.y * rows_per_cta;
    const int v_end = min(V, v_base + rows_per_cta);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto key_of = [&](int e) { return NV4 > 0 ? (128 * (e >> 2) + 4 * lane + (e & 3)) : (lane + 32 * e); };
    auto load_rows = [&](int r0, float (&s)[R][NE], float (&vv)[R]) {
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int row = min(r0 + j, v_end - 1);
            const float* src = s_in + ((size_t)bh * V + row) * K;
            if (NV4 > 0) {
#pragma unroll
                for (int e4 = 0; e4 < NV4; ++e4) {
                    const int kk = min(128 * e4 + 4 * lane, K - 4);
                    const float4 x = __ldcs(reinterpret_cast<const float4*>(src + kk));
                    s[j][4 * e4 + 0] = x.x; s[j][4 * e4 + 1] = x.y; s[j][4 * e4 + 2] = x.z; s[j][4 * e4 + 3] = x.w;
                }
            } else {
#pragma unroll
                for (int e = 0; e < NE; ++e) s[j][e] = src[min(lane + 32 * e, K - 1)];
            }
            vv[j] = ld_io(v, (size_t)bh * V + row, bf16);
        }
    };
    // first row group goes out before the per-(sequence, head) scalars are needed
    float s[R][NE], vv[R];
    int r0 = v_base + warp * R;
    if (r0 < v_end) load_rows(r0, s, vv);

    float qe[NE], ke[NE], dec[NE];
#pragma unroll
    for (int e = 0; e < NE; ++e) {
        const size_t i = (size_t)bh * K + min(key_of(e), K - 1);
        qe[e] = ld_io(q, i, bf16);
        ke[e] = ld_io(k, i, bf16);
        dec[e] = ld_io(g, i, gbf16);
    }
    float bt = ld_io(beta, bh, gbf16);
    if (raw.A_log != nullptr) {
        const int hh = bh % H;
        const float ea = expf(raw.A_log[hh]);
        bt = sigmoidf_(bt);
#pragma unroll
        for (int e = 0; e < NE; ++e)
            dec[e] = raw.lb * sigmoidf_(ea * (dec[e] + raw.dt_bias[hh * K + min(key_of(e), K - 1)]));
    }
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int e = 0; e < NE; ++e) {
        const bool in = key_of(e) < K;
        qe[e] = in ? qe[e] : 0.f;
        ke[e] = in ? ke[e] : 0.f;
        dec[e] = in ? expf(dec[e]) : 0.f;
        sq += qe[e] * qe[e];
        sk += ke[e] * ke[e];
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float qi = (l2norm ? 1.f / fmaxf(sqrtf(sq), 1e-12f) : 1.f) * scale;
    const float ki = l2norm ? 1.f / fmaxf(sqrtf(sk), 1e-12f) : 1.f;
    float qk = 0.f;
#pragma unroll
    for (int e = 0; e < NE; ++e) {
        qe[e] *= qi;
        ke[e] *= ki;
        qk += qe[e] * ke[e];
    }
    qk = warp_sum(qk);

    for (; r0 < v_end; r0 += 8 * R) {
        float a[R], b[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            a[j] = 0.f;
            b[j] = 0.f;
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                s[j][e] *= dec[e];
                a[j] += ke[e] * s[j][e];
                b[j] += qe[e] * s[j][e];
            }
        }
        // R independent reductions interleaved
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int j = 0; j < R; ++j) {
                a[j] += __shfl_xor_sync(0xffffffffu, a[j], off);
                b[j] += __shfl_xor_sync(0xffffffffu, b[j], off);
            }
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int row = r0 + j;
            if (row < v_end) {
                const float br = bt * (vv[j] - a[j]);
                float* dst = s_out + ((size_t)bh * V + row) * K;
                if (NV4 > 0) {
#pragma unroll
                    for (int e4 = 0; e4 < NV4; ++e4) {
                        const int kk = 128 * e4 + 4 * lane;
                        if (kk < K)
                            __stcs(reinterpret_cast<float4*>(dst + kk),
                                   make_float4(s[j][4 * e4 + 0] + br * ke[4 * e4 + 0], s[j][4 * e4 + 1] + br * ke[4 * e4 + 1],
                                               s[j][4 * e4 + 2] + br * ke[4 * e4 + 2], s[j][4 * e4 + 3] + br * ke[4 * e4 + 3]));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < NE; ++e) {
                        const int kk = lane + 32 * e;
                        if (kk < K) dst[kk] = s[j][e] + br * ke[e];
                    }
                }
                if (lane == 0) st_io(o, (size_t)bh * V + row, bf16, b[j] + br * qk);
            }
        }
        if (r0 + 8 * R < v_end) load_rows(r0 + 8 * R, s, vv);
    }
}

// =============================================================================================
// short causal depthwise convolution (+ SiLU)
//   xx = [cache[..., :], x] along time (cache slot p <-> time p - W);  y[t] = act(sum_j w[c][j] xx[t + 1 + j])
// One thread: VEC adjacent channels x kConvTT consecutive tokens, sliding window in registers.
// =============================================================================================
constexpr int kConvTT = 4;

template <int VEC, bool BF16>
__device__ __forceinline__ void ld_vec(float (&dst)[VEC], const void* p, size_t i) {
    if (BF16) {
        if (VEC == 8) {
            uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __bfloat1622float2(h[j]);
                dst[2 * j] = f.x;
                dst[2 * j + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst[j] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i + j]);
        }
    } else {
        if (VEC == 4) {
            float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
            dst[0] = f.x; dst[1] = f.y; dst[2] = f.z; dst[3] = f.w;
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst[j] = reinterpret_cast<const float*>(p)[i + j];
        }
    }
}

template <int VEC, bool BF16>
__device__ __forceinline__ void st_vec(void* p, size_t i, const float (&src)[VEC]) {
    if (BF16) {
        if (VEC == 8) {
            uint4 u;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(src[2 * j], src[2 * j + 1]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = u;
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) reinterpret_cast<__nv_bfloat16*>(p)[i + j] = __float2bfloat16(src[j]);
        }
    } else {
        if (VEC == 4) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = make_float4(src[0], src[1], src[2], src[3]);
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) reinterpret_cast<float*>(p)[i + j] = src[j];
        }
    }
}


// one weight; float32 weights next to bf16 activations are rounded to bf16 first, which is what a cast of the
// weight tensor to the activation dtype would have produced
__device__ __forceinline__ float ld_w(const void* w, size_t i, bool bf16, int wf32) {
    if (wf32) {
        const float f = reinterpret_cast<const float*>(w)[i];
        return bf16 ? __bfloat162float(__float2bfloat16(f)) : f;
    }
    return ld_io(w, i, bf16);
}

// weights of VEC adjacent channels: W*VEC contiguous elements starting at c0*W
template <int W, int VEC, bool BF16>
__device__ __forceinline__ void ld_weights(float (&wv)[W][VEC], const void* wgt, int c0, int wf32) {
    float flat[W * VEC];
    constexpr int N = W * VEC;
    const size_t base = (size_t)c0 * W;
    if (wf32) {
#pragma unroll
        for (int j = 0; j < N; ++j) flat[j] = ld_w(wgt, base + j, BF16, 1);
    } else if (BF16 && N % 8 == 0 && (base % 8) == 0) {
#pragma unroll
        for (int j = 0; j < N / 8; ++j) {
            float t[8];
            ld_vec<8, true>(t, wgt, base + 8 * j);
#pragma unroll
            for (int e = 0; e < 8; ++e) flat[8 * j + e] = t[e];
        }
    } else if (!BF16 && N % 4 == 0 && (base % 4) == 0) {
#pragma unroll
        for (int j = 0; j < N / 4; ++j) {
            float t[4];
            ld_vec<4, false>(t, wgt, base + 4 * j);
#pragma unroll
            for (int e = 0; e < 4; ++e) flat[4 * j + e] = t[e];
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) flat[j] = ld_io(wgt, base + j, BF16);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
#pragma unroll
        for (int j = 0; j < W; ++j) wv[j][e] = flat[e * W + j];
}

// xx at time tau (tau < 0 reaches into the cache: slot W + tau), for VEC channels starting at c0
template <int VEC, bool BF16>
__device__ __forceinline__ void ld_xx(float (&dst)[VEC], const void* x, const void* cache, int b, int tau, int c0, int T,
                                      int C, int W) {
    if (tau >= 0) {
        ld_vec<VEC, BF16>(dst, x, ((size_t)b * T + tau) * C + c0);
    } else if (cache != nullptr && W + tau >= 0) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) dst[j] = ld_io(cache, ((size_t)b * C + c0 + j) * W + (W + tau), BF16);
    } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) dst[j] = 0.f;
    }
}

template <int W, int VEC, bool BF16>
__global__ void __launch_bounds__(256) conv_fwd_kernel(int B, int T, int C, int silu, int wf32, const void* __restrict__ x,
                                                       const void* __restrict__ wgt, const void* __restrict__ cache,
                                                       void* __restrict__ y, void* __restrict__ fin) {
    const int ncg = C / VEC, ntile = (T + kConvTT - 1) / kConvTT;
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (size_t)B * ntile * ncg) return;
    const int cg = (int)(gid % ncg), tile = (int)((gid / ncg) % ntile), b = (int)(gid / ((size_t)ncg * ntile));
    const int c0 = cg * VEC, t0 = tile * kConvTT, t1 = min(T, t0 + kConvTT);
    float wv[W][VEC];
    ld_weights<W, VEC, BF16>(wv, wgt, c0, wf32);
    // inputs at times t0-(W-1) .. t0+kConvTT-1.  Interior tiles issue every load unconditionally (so they
    // overlap); only the first and last tile of a sequence take the guarded path.
    float xin[kConvTT + W - 1][VEC];
    if (t0 >= W - 1 && t0 + kConvTT <= T) {
#pragma unroll
        for (int j = 0; j < kConvTT + W - 1; ++j)
            ld_vec<VEC, BF16>(xin[j], x, ((size_t)b * T + (t0 - (W - 1) + j)) * C + c0);
    } else {
#pragma unroll
        for (int j = 0; j < kConvTT + W - 1; ++j) {
            const int tau = t0 - (W - 1) + j;
            if (tau < T) ld_xx<VEC, BF16>(xin[j], x, cache, b, tau, c0, T, C, W);
            else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) xin[j][e] = 0.f;
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < kConvTT; ++tt) {
        const int t = t0 + tt;
        if (t < t1) {
            float out[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float z = 0.f;
#pragma unroll
                for (int j = 0; j < W; ++j) z += wv[j][e] * xin[tt + j][e];
                out[e] = silu ? z * sigmoid_t<BF16>(z) : z;
            }
            st_vec<VEC, BF16>(y, ((size_t)b * T + t) * C + c0, out);
        }
    }
    if (fin != nullptr && t1 == T) {
        // cache slot j holds xx at time T - W + j
        for (int j = 0; j < W; ++j) {
            float tmp[VEC];
            ld_xx<VEC, BF16>(tmp, x, cache, b, T - W + j, c0, T, C, W);
#pragma unroll
            for (int e = 0; e < VEC; ++e) st_io(fin, ((size_t)b * C + c0 + e) * W + j, BF16, tmp[e]);
        }
    }
}

// One decode token through n same-shaped convolutions (the q, k and v branches of a layer) in ONE launch: every cache
// row [W] is shifted by one, the new input appended, y = act(w . row) - the cache is updated IN PLACE.  Same arithmetic
// order as conv_fwd_kernel, so the result equals the non-mutating call bit for bit.
struct ConvStepItems {
    const void* x[4];
    const void* w[4];
    void* cache[4];
    void* y[4];
};

template <int W, bool BF16>
__global__ void __launch_bounds__(256) conv_step_kernel(int B, int C, int silu, int wf32, ConvStepItems items) {
    const int item = blockIdx.y;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // b * C + c
    if (idx >= (size_t)B * C) return;
    const int c = (int)(idx % C);
    void* cache = items.cache[item];
    float xx[W];
#pragma unroll
    for (int j = 0; j + 1 < W; ++j) xx[j] = ld_io(cache, idx * W + j + 1, BF16);
    xx[W - 1] = ld_io(items.x[item], idx, BF16);
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) z += ld_w(items.w[item], (size_t)c * W + j, BF16, wf32) * xx[j];
    st_io(items.y[item], idx, BF16, silu ? z * sigmoid_t<BF16>(z) : z);
#pragma unroll
    for (int j = 0; j < W; ++j) st_io(cache, idx * W + j, BF16, xx[j]);
}

// Forward without a carried-in window and without a final-state output (the training path).  Lane = channel pair, so
// every global access of a warp is one contiguous 128-byte (bf16) row segment; each thread slides the window over 8
// consecutive tokens with all of its loads issued up front.
template <bool BF16>
__device__ __forceinline__ float2 ld_pair(const void* p, size_t i) {
    // read-only path: the inputs are never written by the kernel that reads them
    if (BF16) {
        const unsigned u = __ldg(reinterpret_cast<const unsigned*>(reinterpret_cast<const __nv_bfloat16*>(p) + i));
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
    }
    return __ldg(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(p) + i));
}
template <bool BF16>
__device__ __forceinline__ void st_pair(void* p, size_t i, float a, float b) {
    if (BF16) *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = __floats2bfloat162_rn(a, b);
    else *reinterpret_cast<float2*>(reinterpret_cast<float*>(p) + i) = make_float2(a, b);
}

// N consecutive weights starting at element `base` (the W taps of N / W adjacent channels), with 16-byte loads when the
// run is 16-byte aligned: a warp then reads one contiguous span instead of 32 scattered words per tap.
template <int N, bool BF16>
__device__ __forceinline__ void ld_wrun(float (&flat)[N], const void* wgt, size_t base, int wf32) {
    const bool f32 = wf32 || !BF16;
    if (f32 && N % 4 == 0 && base % 4 == 0) {
#pragma unroll
        for (int j = 0; j < N / 4; ++j) {
            const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(wgt) + base + 4 * j);
            flat[4 * j] = f.x; flat[4 * j + 1] = f.y; flat[4 * j + 2] = f.z; flat[4 * j + 3] = f.w;
        }
        if (BF16) {
#pragma unroll
            for (int j = 0; j < N; ++j) flat[j] = __bfloat162float(__float2bfloat16(flat[j]));
        }
    } else if (!f32 && N % 8 == 0 && base % 8 == 0) {
#pragma unroll
        for (int j = 0; j < N / 8; ++j) {
            float t[8];
            ld_vec<8, true>(t, wgt, base + 8 * j);
#pragma unroll
            for (int e = 0; e < 8; ++e) flat[8 * j + e] = t[e];
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) flat[j] = ld_w(wgt, base + j, BF16, wf32);
    }
}

constexpr int kConvPairT = 8;    // tokens per thread

// VEC adjacent channels (2 or 4) as floats
template <int VEC, bool BF16>
__device__ __forceinline__ void ld_cvec(float (&d)[VEC], const void* p, size_t i) {
    if (VEC == 2) {
        const float2 v = ld_pair<BF16>(p, i);
        d[0] = v.x; d[1] = v.y;
    } else if (BF16) {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i));
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        d[0] = a.x; d[1] = a.y; d[2] = b.x; d[3] = b.y;
    } else {
        const float4 f = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i));
        d[0] = f.x; d[1] = f.y; d[2] = f.z; d[3] = f.w;
    }
}
template <int VEC, bool BF16>
__device__ __forceinline__ void st_cvec(void* p, size_t i, const float (&s)[VEC]) {
    if (VEC == 2) {
        st_pair<BF16>(p, i, s[0], s[1]);
    } else if (BF16) {
        uint2 u;
        *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(s[0], s[1]);
        *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(s[2], s[3]);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = u;
    } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = make_float4(s[0], s[1], s[2], s[3]);
    }
}

// Gate activations, K % 4 == 0: a thread owns 4 adjacent channels (one head), so raw gate, bias, g and their gradients
// move as 8- / 16-byte accesses and the head's exp(A_log) is computed once per 4 elements.
template <bool BF16>
__global__ void __launch_bounds__(256) gate_fwd4_kernel(unsigned n4, unsigned n_beta, int H, int K, const void* __restrict__ raw,
                                                        const void* __restrict__ bl, const float* __restrict__ A_log,
                                                        const float* __restrict__ dt_bias, float lb, float* __restrict__ g,
                                                        float* __restrict__ beta) {
    const unsigned hk4 = (unsigned)(H * K) >> 2;
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned i4 = blockIdx.x * blockDim.x + threadIdx.x; i4 < n4; i4 += stride) {
        const unsigned c = (i4 % hk4) * 4;
        const float ea = expf(A_log[c / (unsigned)K]);
        const float4 bias = *reinterpret_cast<const float4*>(dt_bias + c);
        float r[4];
        ld_cvec<4, BF16>(r, raw, (size_t)i4 * 4);
        float4 o;
        o.x = lb * sigmoidf_(ea * (r[0] + bias.x));
        o.y = lb * sigmoidf_(ea * (r[1] + bias.y));
        o.z = lb * sigmoidf_(ea * (r[2] + bias.z));
        o.w = lb * sigmoidf_(ea * (r[3] + bias.w));
        *reinterpret_cast<float4*>(g + (size_t)i4 * 4) = o;
    }
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n_beta; i += stride) beta[i] = sigmoidf_(ld_io(bl, i, BF16));
}

// grid: x = blocks of 128 columns (lane = 4 channels), y = blocks of kGateRows tokens; warp w takes rows w, w + 8, ...
template <bool BF16>
__global__ void __launch_bounds__(256) gate_bwd4_kernel(int tokens, int H, int K, const void* __restrict__ raw,
                                                        const void* __restrict__ bl, const float* __restrict__ A_log,
                                                        const float* __restrict__ dt_bias, float lb, const float* __restrict__ dg,
                                                        const float* __restrict__ dbeta, void* __restrict__ d_raw,
                                                        void* __restrict__ d_bl, float* __restrict__ part_b,
                                                        float* __restrict__ part_a) {
    constexpr int RPW = kGateRows / 8;
    __shared__ float red[2][8][128];
    const int HK = H * K;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = (blockIdx.x * 32 + lane) * 4;
    const int t0 = blockIdx.y * kGateRows;
    const bool cok = c < HK;
    const int cl = cok ? c : 0;
    const float ea = expf(A_log[cl / K]);
    const float4 bias = *reinterpret_cast<const float4*>(dt_bias + cl);
    const float bz[4] = {bias.x, bias.y, bias.z, bias.w};
    float rv[RPW][4];
    float4 gv[RPW];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {          // every load of the thread in flight at once
        const int t = min(t0 + w + 8 * j, tokens - 1);
        ld_cvec<4, BF16>(rv[j], raw, (size_t)t * HK + cl);
        gv[j] = __ldg(reinterpret_cast<const float4*>(dg + (size_t)t * HK + cl));
    }
    float sb[4] = {0.f, 0.f, 0.f, 0.f}, sa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
        const int t = t0 + w + 8 * j;
        if (t < tokens && cok) {
            const float gg[4] = {gv[j].x, gv[j].y, gv[j].z, gv[j].w};
            float dr[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x = rv[j][e] + bz[e];
                const float sg = sigmoidf_(ea * x);
                dr[e] = gg[e] * lb * sg * (1.f - sg) * ea;
                sb[e] += dr[e];
                sa[e] += dr[e] * x;
            }
            st_cvec<4, BF16>(d_raw, (size_t)t * HK + c, dr);
        }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        red[0][w][4 * lane + e] = sb[e];
        red[1][w][4 * lane + e] = sa[e];
    }
    __syncthreads();
    if (threadIdx.x < 128 && blockIdx.x * 128 + threadIdx.x < HK) {
        float tb = 0.f, ta = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            tb += red[0][r][threadIdx.x];
            ta += red[1][r][threadIdx.x];
        }
        const size_t o = (size_t)blockIdx.y * HK + blockIdx.x * 128 + threadIdx.x;
        part_b[o] = tb;
        part_a[o] = ta;
    }
    if (blockIdx.x == 0) {                  // beta logits of this block's rows
        const int nb = min(kGateRows, tokens - t0) * H;
        for (int i = threadIdx.x; i < nb; i += 256) {
            const size_t o = (size_t)t0 * H + i;
            const float b = sigmoidf_(ld_io(bl, o, BF16));
            st_io(d_bl, o, BF16, dbeta[o] * b * (1.f - b));
        }
    }
}

// Up to kConvItems same-shaped convolutions (the q, k and v branches of a layer) share one launch: blockIdx.z runs over
// item x batch.
constexpr int kConvItems = 4;
struct ConvFwdItems {
    const void* x[kConvItems];
    const void* w[kConvItems];
    void* y[kConvItems];
};
struct ConvBwdItems {
    const void* x[kConvItems];
    const void* w[kConvItems];
    const void* dy[kConvItems];
    void* dx[kConvItems];
};
struct ColumnSumItems {
    float* out[kConvItems];
};
// Entry i of a kernel-parameter array by compile-time indices only: a run-time subscript would make every thread copy the
// whole array to local memory first.
template <class T>
__device__ __forceinline__ T pick_item(T const (&a)[kConvItems], int i) {
    T r = a[0];
    if (i == 1) r = a[1];
    if (i == 2) r = a[2];
    if (i == 3) r = a[3];
    return r;
}

// grid: x = channel blocks of 32*VEC, y = blocks of 8 time groups x kConvPairT tokens, z = item * B + batch
template <int W, int VEC, bool BF16>
__global__ void __launch_bounds__(256) conv_fwd_pair_kernel(int B, int T, int C, int silu, int wf32, ConvFwdItems items) {
    const int p = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int c = (blockIdx.x * 32 + p) * VEC;
    const int item = blockIdx.z / B;
    const int t0 = (blockIdx.y * 8 + g) * kConvPairT, b = blockIdx.z - item * B;
    if (t0 >= T) return;
    const void* __restrict__ x = pick_item(items.x, item);
    const void* __restrict__ wgt = pick_item(items.w, item);
    void* __restrict__ y = pick_item(items.y, item);
    const bool cok = c < C;
    const int cl = cok ? c : 0;
    float wv[W][VEC];
    {
        float flat[W * VEC];
        ld_wrun<W * VEC, BF16>(flat, wgt, (size_t)cl * W, wf32);
#pragma unroll
        for (int e = 0; e < VEC; ++e)
#pragma unroll
            for (int m = 0; m < W; ++m) wv[m][e] = flat[e * W + m];
    }
    const size_t rowbase = (size_t)b * T;
    float xin[kConvPairT + W - 1][VEC];
    if (t0 >= W - 1 && t0 + kConvPairT <= T) {
        // interior: plain address arithmetic, every load independent
        const size_t base = (rowbase + t0 - (W - 1)) * C + cl;
#pragma unroll
        for (int j = 0; j < kConvPairT + W - 1; ++j) ld_cvec<VEC, BF16>(xin[j], x, base + (size_t)j * C);
    } else {
#pragma unroll
        for (int j = 0; j < kConvPairT + W - 1; ++j) {
            const int t = t0 - (W - 1) + j;
            const int tc = min(max(t, 0), T - 1);
            ld_cvec<VEC, BF16>(xin[j], x, (rowbase + tc) * C + cl);
            if (t < 0 || t >= T) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) xin[j][e] = 0.f;
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < kConvPairT; ++tt) {
        float out[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float z = 0.f;
#pragma unroll
            for (int m = 0; m < W; ++m) z += wv[m][e] * xin[tt + m][e];
            out[e] = silu ? z * sigmoid_t<BF16>(z) : z;
        }
        if (t0 + tt < T && cok) st_cvec<VEC, BF16>(y, (rowbase + t0 + tt) * C + c, out);
    }
}

// Backward.  blockDim = (16 channel groups, 16 time tiles).  Each thread recomputes the
// pre-activations of its tile plus W-1 following tokens, emits dx for its tile and a
// register partial of dweight; the 8 tiles of a block are summed in shared memory and
// written as one partial per block, reduced in fixed order by column_sum_kernel.
constexpr int kConvBT = 4;   // tokens per thread in the backward

template <int W, int VEC, bool BF16>
__global__ void __launch_bounds__(256) conv_bwd_kernel(int B, int T, int C, int silu, int wf32, const void* __restrict__ x,
                                                       const void* __restrict__ wgt, const void* __restrict__ cache,
                                                       const void* __restrict__ dy, const void* __restrict__ dfin,
                                                       void* __restrict__ dx, void* __restrict__ dcache,
                                                       float* __restrict__ dw_part) {
    __shared__ float red[16][16][W * VEC];
    const int ncg = C / VEC, ntile = (T + kConvBT - 1) / kConvBT;
    const int cg = blockIdx.x * 16 + threadIdx.x;
    const int tile = blockIdx.y * 16 + threadIdx.y;
    const int b = blockIdx.z;
    const bool active = cg < ncg && tile < ntile;
    float dwv[W][VEC];
#pragma unroll
    for (int j = 0; j < W; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) dwv[j][e] = 0.f;
    if (active) {
        const int c0 = cg * VEC, t0 = tile * kConvBT, t1 = min(T, t0 + kConvBT);
        float wv[W][VEC];
        ld_weights<W, VEC, BF16>(wv, wgt, c0, wf32);
        if (t0 >= W - 1 && t0 + kConvBT + W <= T) {
            // interior tile: every load is unconditional and independent, then pure register arithmetic
            float xin[kConvBT + 2 * (W - 1)][VEC];   // x at t0-(W-1) .. t0+kConvBT+W-2
            float gy[kConvBT + W - 1][VEC];          // dy, then dz, at t0 .. t0+kConvBT+W-2
#pragma unroll
            for (int j = 0; j < kConvBT + 2 * (W - 1); ++j)
                ld_vec<VEC, BF16>(xin[j], x, ((size_t)b * T + (t0 - (W - 1) + j)) * C + c0);
#pragma unroll
            for (int j = 0; j < kConvBT + W - 1; ++j) ld_vec<VEC, BF16>(gy[j], dy, ((size_t)b * T + t0 + j) * C + c0);
#pragma unroll
            for (int j = 0; j < kConvBT + W - 1; ++j)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float z = 0.f;
#pragma unroll
                    for (int m = 0; m < W; ++m) z += wv[m][e] * xin[j + m][e];
                    if (silu) {
                        const float sg = sigmoid_t<BF16>(z);
                        gy[j][e] *= sg * (1.f + z * (1.f - sg));
                    }
                }
#pragma unroll
            for (int j = 0; j < kConvBT; ++j) {
                float out[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int m = 0; m < W; ++m) {
                        a += wv[m][e] * gy[j + W - 1 - m][e];
                        dwv[m][e] += gy[j][e] * xin[j + m][e];
                    }
                    out[e] = a;
                }
                st_vec<VEC, BF16>(dx, ((size_t)b * T + t0 + j) * C + c0, out);
            }
        } else {
        float win[W][VEC];   // xx window ending at the token whose dz is being produced
        float dzw[W][VEC];   // dzw[m] = dz at token (cur - (W-1) + m)
#pragma unroll
        for (int j = 0; j < W; ++j)
#pragma unroll
            for (int e = 0; e < VEC; ++e) dzw[j][e] = 0.f;
#pragma unroll
        for (int j = 0; j < W - 1; ++j) ld_xx<VEC, BF16>(win[j + 1], x, cache, b, t0 - (W - 1) + j, c0, T, C, W);
        // walk cur over [t0, t1 + W - 1): produce dz[cur]; once W-1 tokens ahead, emit dx[cur - (W-1)]
#pragma unroll
        for (int step = 0; step < kConvBT + W - 1; ++step) {
            const int cur = t0 + step;
            if (cur >= t1 + W - 1) break;
#pragma unroll
            for (int j = 0; j < W - 1; ++j)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    win[j][e] = win[j + 1][e];
                    dzw[j][e] = dzw[j + 1][e];
                }
            if (cur < T) {
                ld_vec<VEC, BF16>(win[W - 1], x, ((size_t)b * T + cur) * C + c0);
                float g[VEC];
                ld_vec<VEC, BF16>(g, dy, ((size_t)b * T + cur) * C + c0);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float z = 0.f;
#pragma unroll
                    for (int j = 0; j < W; ++j) z += wv[j][e] * win[j][e];
                    if (silu) {
                        const float sg = sigmoid_t<BF16>(z);
                        g[e] *= sg * (1.f + z * (1.f - sg));
                    }
                    dzw[W - 1][e] = g[e];
                    if (cur < t1) {
#pragma unroll
                        for (int j = 0; j < W; ++j) dwv[j][e] += g[e] * win[j][e];
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) { dzw[W - 1][e] = 0.f; win[W - 1][e] = 0.f; }
            }
            const int t = cur - (W - 1);     // dx[t] = sum_j w[j] dz[t + W-1-j] = sum_j w[j] dzw[W-1-j]
            if (t >= t0 && t < t1) {
                float out[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int j = 0; j < W; ++j) a += wv[j][e] * dzw[W - 1 - j][e];
                    if (dfin != nullptr && t >= T - W) a += ld_io(dfin, ((size_t)b * C + c0 + e) * W + (W + t - T), BF16);
                    out[e] = a;
                }
                st_vec<VEC, BF16>(dx, ((size_t)b * T + t) * C + c0, out);
            }
        }
        }   // guarded (boundary) path
        if (dcache != nullptr && tile == 0) {
            // cache slot p is time p - W (< 0): d = sum_j w[j] dz[p - W + W-1-j] = sum_j w[j] dz[p-1-j], plus the
            // final-state cotangent when the sequence is shorter than the window.  Needs dz[0 .. W-2]: recompute.
            float dz0[W][VEC];
#pragma unroll
            for (int m = 0; m < W; ++m)
#pragma unroll
                for (int e = 0; e < VEC; ++e) dz0[m][e] = 0.f;
            float w2[W][VEC];
#pragma unroll
            for (int j = 0; j < W - 1; ++j) ld_xx<VEC, BF16>(w2[j + 1], x, cache, b, -(W - 1) + j, c0, T, C, W);
            for (int t = 0; t < W - 1 && t < T; ++t) {
#pragma unroll
                for (int j = 0; j < W - 1; ++j)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) w2[j][e] = w2[j + 1][e];
                ld_vec<VEC, BF16>(w2[W - 1], x, ((size_t)b * T + t) * C + c0);
                float g[VEC];
                ld_vec<VEC, BF16>(g, dy, ((size_t)b * T + t) * C + c0);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float z = 0.f;
#pragma unroll
                    for (int j = 0; j < W; ++j) z += wv[j][e] * w2[j][e];
                    if (silu) {
                        const float sg = sigmoid_t<BF16>(z);
                        g[e] *= sg * (1.f + z * (1.f - sg));
                    }
#pragma unroll
                    for (int m = 0; m < W; ++m)
                        if (m == t) dz0[m][e] = g[e];
                }
            }
#pragma unroll
            for (int p = 0; p < W; ++p)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int j = 0; j < W; ++j) {
                        const int m = p - 1 - j;
                        if (m >= 0 && m < W) a += wv[j][e] * dz0[m][e];
                    }
                    if (dfin != nullptr && p - T >= 0) a += ld_io(dfin, ((size_t)b * C + c0 + e) * W + (p - T), BF16);
                    st_io(dcache, ((size_t)b * C + c0 + e) * W + p, BF16, a);
                }
        }
    }
#pragma unroll
    for (int j = 0; j < W; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) red[threadIdx.y][threadIdx.x][j * VEC + e] = dwv[j][e];
    __syncthreads();
    if (threadIdx.y == 0 && cg < ncg) {
        const size_t pblk = (size_t)blockIdx.z * gridDim.y + blockIdx.y;
#pragma unroll
        for (int j = 0; j < W; ++j)
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float a = 0.f;
#pragma unroll
                for (int r = 0; r < 16; ++r) a += red[r][threadIdx.x][j * VEC + e];
                dw_part[(pblk * C + cg * VEC + e) * W + j] = a;
            }
    }
}

// Backward without a carried-in window (no initial state, no final-state cotangent: the training path).  One block
// owns 64 tokens x 64 channels.  It stages x (with a W-1 halo on both sides) and dy (W-1 halo after) in shared memory
// as float pairs, turns dy into dz in place (each pre-activation is recomputed once, not once per window position),
// then forms dx from the dz window and the block's dweight partial.  Lane = channel pair, so every global access of a
// warp is one contiguous row segment; warp = row group.
constexpr int kConvTileT = 64, kConvTileC = 64;

template <int W, bool BF16>
__global__ void __launch_bounds__(256) conv_bwd_tile_kernel(int B, int T, int C, int silu, int wf32, ConvBwdItems items,
                                                            float* __restrict__ dw_part) {
    constexpr int XR = kConvTileT + 2 * (W - 1);   // x rows  t0-(W-1) .. t0+63+(W-1)
    constexpr int GR = kConvTileT + W - 1;         // dy rows t0 .. t0+63+(W-1)
    constexpr int RPW = kConvTileT / 8;            // consecutive rows per warp
    // x stays in its storage type (a bf16 pair is one 32-bit word); dy is widened because dz replaces it in place
    typedef typename std::conditional<BF16, __nv_bfloat162, float2>::type xpair_t;
    __shared__ __align__(16) xpair_t xs[XR][32];
    __shared__ __align__(16) float2 gs[GR][32];
    __shared__ float red[8][W][kConvTileC];
    const int p = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int cb = blockIdx.x * kConvTileC;
    const int c = cb + 2 * p;
    const int item = blockIdx.z / B;
    const int t0 = blockIdx.y * kConvTileT, b = blockIdx.z - item * B;
    const void* __restrict__ x = pick_item(items.x, item);
    const void* __restrict__ wgt = pick_item(items.w, item);
    const void* __restrict__ dy = pick_item(items.dy, item);
    void* __restrict__ dx = pick_item(items.dx, item);
    const bool cok = c < C;
    const int cl = cok ? c : 0;                    // loads stay unconditional: out-of-range lanes read column 0 and are masked
    float w0[W], w1[W];
    {
        float flat[2 * W];
        ld_wrun<2 * W, BF16>(flat, wgt, (size_t)cl * W, wf32);
#pragma unroll
        for (int m = 0; m < W; ++m) {
            w0[m] = flat[m];
            w1[m] = flat[W + m];
        }
    }
    const size_t rowbase = (size_t)b * T;
    auto xload = [&](int tc) -> xpair_t {
        if constexpr (BF16) {
            const unsigned u = __ldg(reinterpret_cast<const unsigned*>(reinterpret_cast<const __nv_bfloat16*>(x) + (rowbase + tc) * C + cl));
            return *reinterpret_cast<const __nv_bfloat162*>(&u);
        } else {
            return __ldg(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(x) + (rowbase + tc) * C + cl));
        }
    };
    auto xwide = [](const xpair_t& v) -> float2 {
        if constexpr (BF16) return __bfloat1622float2(v);
        else return v;
    };
    if (t0 >= W - 1 && t0 + GR <= T && cb + kConvTileC <= C && (C & 3) == 0) {
        // interior tile: no clamping, four channels per thread (sixteen threads cover a 64-channel row, a warp two rows),
        // addresses advance by a constant stride
        const int q = threadIdx.x & 15, rg = threadIdx.x >> 4;
        const size_t e0 = (rowbase + t0 - (W - 1) + rg) * C + cb + 4 * q;       // x row rg of the tile, this thread's channels
        const size_t step = (size_t)16 * C;
#pragma unroll
        for (int it = 0; it < (XR + 15) / 16; ++it) {
            const int r = rg + 16 * it;
            if (r < XR) {
                if constexpr (BF16) {
                    const uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(x) + e0 + it * step));
                    *reinterpret_cast<uint2*>(&xs[r][2 * q]) = u;
                } else {
                    const float4 f = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + e0 + it * step));
                    *reinterpret_cast<float4*>(&xs[r][2 * q]) = f;
                }
            }
        }
        const size_t g0 = (rowbase + t0 + rg) * C + cb + 4 * q;
#pragma unroll
        for (int it = 0; it < (GR + 15) / 16; ++it) {
            const int r = rg + 16 * it;
            if (r < GR) {
                float4 f;
                if constexpr (BF16) {
                    const uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(dy) + g0 + it * step));
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
                    const float2 b2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
                    f = make_float4(a.x, a.y, b2.x, b2.y);
                } else {
                    f = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(dy) + g0 + it * step));
                }
                *reinterpret_cast<float4*>(&gs[r][2 * q]) = f;
            }
        }
    } else {
#pragma unroll
        for (int r = g; r < XR; r += 8) {
            const int t = t0 - (W - 1) + r;
            xpair_t v = xload(min(max(t, 0), T - 1));
            if (t < 0 || t >= T || !cok) v = xpair_t();
            xs[r][p] = v;
        }
#pragma unroll
        for (int r = g; r < GR; r += 8) {
            const int t = t0 + r;
            float2 v = ld_pair<BF16>(dy, (rowbase + min(t, T - 1)) * C + cl);
            if (t >= T || !cok) v = make_float2(0.f, 0.f);
            gs[r][p] = v;
        }
    }
    __syncthreads();
    float dw0[W], dw1[W];
#pragma unroll
    for (int m = 0; m < W; ++m) dw0[m] = dw1[m] = 0.f;
    // dz for rows r0 .. r0+n-1, walking down with the x window in registers; dweight only from the tile's own rows
    auto dz_rows = [&](int r0, int n, bool own) {
        float2 xw[W];
#pragma unroll
        for (int m = 0; m < W - 1; ++m) xw[m] = xwide(xs[r0 + m][p]);
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            if (i < n) {
                const int r = r0 + i;
                xw[W - 1] = xwide(xs[r + W - 1][p]);
                float2 gy = gs[r][p];
                float z0 = 0.f, z1 = 0.f;
#pragma unroll
                for (int m = 0; m < W; ++m) {
                    z0 += w0[m] * xw[m].x;
                    z1 += w1[m] * xw[m].y;
                }
                if (silu) {
                    const float s0 = sigmoid_t<BF16>(z0), s1 = sigmoid_t<BF16>(z1);
                    gy.x *= s0 * (1.f + z0 * (1.f - s0));
                    gy.y *= s1 * (1.f + z1 * (1.f - s1));
                }
                gs[r][p] = gy;                     // dz; element (r, p) is touched by this thread only
                if (own) {
#pragma unroll
                    for (int m = 0; m < W; ++m) {
                        dw0[m] += gy.x * xw[m].x;
                        dw1[m] += gy.y * xw[m].y;
                    }
                }
#pragma unroll
                for (int m = 0; m < W - 1; ++m) xw[m] = xw[m + 1];
            }
        }
    };
    dz_rows(g * RPW, RPW, true);
    if (g < W - 1) dz_rows(kConvTileT + g, 1, false);   // halo rows: their dweight belongs to the next block
#pragma unroll
    for (int m = 0; m < W; ++m) {
        red[g][m][2 * p] = dw0[m];
        red[g][m][2 * p + 1] = dw1[m];
    }
    __syncthreads();
    // dx[t] = sum_m w[m] dz[t + W-1-m], again with a register window over this warp's consecutive rows
    {
        const int r0 = g * RPW;
        float2 dw_[W];
#pragma unroll
        for (int m = 0; m < W - 1; ++m) dw_[m] = gs[r0 + m][p];
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = r0 + i, t = t0 + r;
            dw_[W - 1] = gs[r + W - 1][p];
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int m = 0; m < W; ++m) {
                a0 += w0[m] * dw_[W - 1 - m].x;
                a1 += w1[m] * dw_[W - 1 - m].y;
            }
            if (t < T && cok) st_pair<BF16>(dx, (rowbase + t) * C + c, a0, a1);
#pragma unroll
            for (int m = 0; m < W - 1; ++m) dw_[m] = dw_[m + 1];
        }
    }
    if (threadIdx.x < kConvTileC && cb + threadIdx.x < C) {
        const size_t pblk = (size_t)blockIdx.z * gridDim.y + blockIdx.y;
#pragma unroll
        for (int m = 0; m < W; ++m) {
            float a = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) a += red[r][m][threadIdx.x];
            dw_part[(pblk * C + cb + threadIdx.x) * W + m] = a;
        }
    }
}

// Backward, training path, bf16 with C % 128 == 0.  A thread owns 4 adjacent channels and a run of consecutive tokens
// and streams down its rows once: x and dy rows arrive through a thread-private ring in shared memory filled by
// asynchronous 8-byte copies kConvRingDepth rows ahead (no registers held for data in flight, no block-wide barrier in
// the loop), the x window and the dz window live in registers as circular buffers with compile-time indices, and every
// pre-activation, SiLU derivative, dweight and dx multiply-add is done exactly once per element.  Only the W-1 rows
// either side of a run are touched twice.  Block = 8 warps = 8 runs x 128 channels; one dweight partial per block.
constexpr int kConvRingDepth = 16;

template <int W>
__global__ void __launch_bounds__(256, 3) conv_bwd_ring_kernel(int B, int T, int C, int run, int silu, int wf32, ConvBwdItems items,
                                                               float* __restrict__ dw_part) {
    constexpr int D = kConvRingDepth;
    extern __shared__ __align__(16) uint8_t ring_raw[];
    uint2* ring = reinterpret_cast<uint2*>(ring_raw);          // [D][2: x | dy][256 threads]
    float (*red)[W][128] = reinterpret_cast<float (*)[W][128]>(ring_raw);      // [8][W][128], once the ring is drained
    const int p = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int c = (blockIdx.x * 32 + p) * 4;                   // C % 128 == 0: in range
    const int item = blockIdx.z / B, b = blockIdx.z - item * B;
    const int t0 = (blockIdx.y * 8 + g) * run;
    const __nv_bfloat16* __restrict__ x = static_cast<const __nv_bfloat16*>(pick_item(items.x, item));
    const void* __restrict__ wgt = pick_item(items.w, item);
    const __nv_bfloat16* __restrict__ dy = static_cast<const __nv_bfloat16*>(pick_item(items.dy, item));
    __nv_bfloat16* __restrict__ dx = static_cast<__nv_bfloat16*>(pick_item(items.dx, item));
    float wv[W][4];
    {
        float flat[W * 4];
        ld_wrun<W * 4, true>(flat, wgt, (size_t)c * W, wf32);
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int m = 0; m < W; ++m) wv[m][e] = flat[e * W + m];
    }
    float dwv[W][4];
#pragma unroll
    for (int m = 0; m < W; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) dwv[m][e] = 0.f;
    auto widen = [](const uint2& u, float (&f)[4]) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        f[0] = a.x; f[1] = a.y; f[2] = b2.x; f[3] = b2.y;
    };
    if (t0 < T) {
        // stream step j handles token tx = t0 - (W-1) + j: x[tx] enters the window; from tx >= t0 on dz[tx] is formed;
        // from tx >= t0 + W-1 on dx[tx - (W-1)] leaves.  Steps run to a multiple of W so the circular indices are static.
        const int nr = ((run + 2 * (W - 1) + W - 1) / W) * W;
        const size_t rowbase = (size_t)b * T;
        const uint32_t slot0 = (uint32_t)__cvta_generic_to_shared(ring + threadIdx.x);
        auto issue = [&](int j) {
            if (j < nr) {
                const int tx = min(max(t0 - (W - 1) + j, 0), T - 1);
                const size_t off = (rowbase + tx) * C + c;
                const uint32_t dst = slot0 + (uint32_t)((j % D) * 2) * 256u * 8u;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(x + off) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 256u * 8u), "l"(dy + off) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
#pragma unroll 1
        for (int j = 0; j < D - 1; ++j) issue(j);
        float xc[W][4], dzc[W][4];
#pragma unroll
        for (int m = 0; m < W; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) xc[m][e] = dzc[m][e] = 0.f;
#pragma unroll 1
        for (int jj = 0; jj < nr; jj += W) {
#pragma unroll
            for (int u = 0; u < W; ++u) {
                const int j = jj + u;
                issue(j + D - 1);                  // refills the slot whose row was consumed one step ago
                asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
                const int tx = t0 - (W - 1) + j;
                const uint2 xr = ring[((j % D) * 2) * 256 + threadIdx.x];
                const uint2 gr = ring[((j % D) * 2 + 1) * 256 + threadIdx.x];
                widen(xr, xc[u]);
                if (tx < 0 || tx >= T) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) xc[u][e] = 0.f;
                }
                float gy[4];
                widen(gr, gy);
                const bool live = tx >= t0 && tx < T;             // dz[tx] exists and belongs to this run's window
                const bool own = live && tx < t0 + run;           // ... and its dweight is this run's
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float z = 0.f;
#pragma unroll
                    for (int m = 0; m < W; ++m) z += wv[m][e] * xc[(u + 1 + m) % W][e];      // x[tx - (W-1) + m]
                    float dzv = gy[e];
                    if (silu) {
                        const float sg = sigmoid_t<true>(z);
                        dzv *= sg * (1.f + z * (1.f - sg));
                    }
                    dzv = live ? dzv : 0.f;
                    dzc[u][e] = dzv;
                    if (own) {
#pragma unroll
                        for (int m = 0; m < W; ++m) dwv[m][e] += dzv * xc[(u + 1 + m) % W][e];
                    }
                }
                const int td = tx - (W - 1);
                if (td >= t0 && td < t0 + run && td < T) {
                    float a[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        a[e] = 0.f;
#pragma unroll
                        for (int m = 0; m < W; ++m) a[e] += wv[m][e] * dzc[(u - m + W) % W][e];  // dz[tx - m]
                    }
                    st_cvec<4, true>(dx, (rowbase + td) * C + c, a);
                }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();                               // every warp has drained its ring: the memory becomes the partials
#pragma unroll
    for (int m = 0; m < W; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[g][m][4 * p + e] = dwv[m][e];
    __syncthreads();
    if (threadIdx.x < 128) {
        const size_t pblk = (size_t)blockIdx.z * gridDim.y + blockIdx.y;
#pragma unroll
        for (int m = 0; m < W; ++m) {
            float a = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) a += red[r][m][threadIdx.x];
            dw_part[(pblk * C + blockIdx.x * 128 + threadIdx.x) * W + m] = a;
        }
    }
}

// =============================================================================================
// gated RMSNorm:  y = x * inv * w * sigmoid(gate),  inv = rsqrt(mean(x^2) + eps).  One warp per row.
// =============================================================================================
template <bool BF16>
__device__ __forceinline__ void ld4(float (&d)[4], const void* p, size_t i) {
    if (BF16) {
        uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
        float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        d[0] = a.x; d[1] = a.y; d[2] = b.x; d[3] = b.y;
    } else {
        float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
        d[0] = f.x; d[1] = f.y; d[2] = f.z; d[3] = f.w;
    }
}
template <bool BF16>
__device__ __forceinline__ void st4(void* p, size_t i, const float (&s)[4]) {
    if (BF16) {
        uint2 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
        h[0] = __floats2bfloat162_rn(s[0], s[1]);
        h[1] = __floats2bfloat162_rn(s[2], s[3]);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = u;
    } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = make_float4(s[0], s[1], s[2], s[3]);
    }
}

// VEC4: dim % 128 == 0, lane owns 4 contiguous elements per 128-wide segment; else scalar stride-32.
template <bool BF16, bool VEC4>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(long long rows, int D, float eps, const void* __restrict__ x,
                                                          const void* __restrict__ gate, const float* __restrict__ w,
                                                          void* __restrict__ y, float* __restrict__ inv_rms) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long nwarp = (long long)gridDim.x * 8;
    for (long long row = warp0; row < rows; row += nwarp) {
        const size_t base = (size_t)row * D;
        float ss = 0.f;
        if (VEC4) {
            for (int d = 4 * lane; d < D; d += 128) {
                float a[4];
                ld4<BF16>(a, x, base + d);
                ss += a[0] * a[0] + a[1] * a[1] + a[2] * a[2] + a[3] * a[3];
            }
        } else {
            for (int d = lane; d < D; d += 32) {
                float a = ld_io(x, base + d, BF16);
                ss += a * a;
            }
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
        if (lane == 0) inv_rms[row] = inv;
        if (VEC4) {
            for (int d = 4 * lane; d < D; d += 128) {
                float a[4], gt[4], out[4];
                ld4<BF16>(a, x, base + d);
                ld4<BF16>(gt, gate, base + d);
                const float4 ww = *reinterpret_cast<const float4*>(w + d);
                const float wa[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) out[e] = a[e] * inv * wa[e] * sigmoid_t<BF16>(gt[e]);
                st4<BF16>(y, base + d, out);
            }
        } else {
            for (int d = lane; d < D; d += 32)
                st_io(y, base + d, BF16, ld_io(x, base + d, BF16) * inv * w[d] * sigmoid_t<BF16>(ld_io(gate, base + d, BF16)));
        }
    }
}

// Backward: u = n*w, y = u*s;  dgate = dy*u*s*(1-s);  du = dy*s;  dw += du*n;  dn = du*w;
//           dx = inv * (dn - n * mean(dn*n)).
// dweight: every warp accumulates its rows into its own shared-memory row, the block sums the
// eight rows in fixed order and writes one partial per block.
template <bool BF16, bool VEC4>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(long long rows, int D, const void* __restrict__ x,
                                                          const void* __restrict__ gate, const float* __restrict__ w,
                                                          const float* __restrict__ inv_rms, const void* __restrict__ dy,
                                                          void* __restrict__ dx, void* __restrict__ dgate,
                                                          float* __restrict__ dw_part) {
    extern __shared__ float dws[];   // [8][D]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    float* mine = dws + (size_t)wid * D;
    for (int d = lane; d < D; d += 32) mine[d] = 0.f;
    const long long warp0 = (long long)blockIdx.x * 8 + wid;
    const long long nwarp = (long long)gridDim.x * 8;
    for (long long row = warp0; row < rows; row += nwarp) {
        const size_t base = (size_t)row * D;
        const float inv = inv_rms[row];
        float dot = 0.f;
        if (VEC4) {
            for (int d = 4 * lane; d < D; d += 128) {
                float a[4], gt[4], gy[4];
                ld4<BF16>(a, x, base + d);
                ld4<BF16>(gt, gate, base + d);
                ld4<BF16>(gy, dy, base + d);
                const float4 ww = *reinterpret_cast<const float4*>(w + d);
                const float wa[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) dot += gy[e] * sigmoid_t<BF16>(gt[e]) * wa[e] * a[e] * inv;
            }
        } else {
            for (int d = lane; d < D; d += 32)
                dot += ld_io(dy, base + d, BF16) * sigmoid_t<BF16>(ld_io(gate, base + d, BF16)) * w[d] * ld_io(x, base + d, BF16) * inv;
        }
        dot = warp_sum(dot) / (float)D;
        if (VEC4) {
            for (int d = 4 * lane; d < D; d += 128) {
                float a[4], gt[4], gy[4], ox[4], og[4];
                ld4<BF16>(a, x, base + d);
                ld4<BF16>(gt, gate, base + d);
                ld4<BF16>(gy, dy, base + d);
                const float4 ww = *reinterpret_cast<const float4*>(w + d);
                const float wa[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float n = a[e] * inv, s = sigmoid_t<BF16>(gt[e]);
                    const float du = gy[e] * s;
                    og[e] = gy[e] * n * wa[e] * s * (1.f - s);
                    ox[e] = inv * (du * wa[e] - n * dot);
                    mine[d + e] += du * n;
                }
                st4<BF16>(dx, base + d, ox);
                st4<BF16>(dgate, base + d, og);
            }
        } else {
            for (int d = lane; d < D; d += 32) {
                const float n = ld_io(x, base + d, BF16) * inv, s = sigmoid_t<BF16>(ld_io(gate, base + d, BF16));
                const float gyv = ld_io(dy, base + d, BF16);
                const float du = gyv * s;
                st_io(dgate, base + d, BF16, gyv * n * w[d] * s * (1.f - s));
                st_io(dx, base + d, BF16, inv * (du * w[d] - n * dot));
                mine[d] += du * n;
            }
        }
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += 256) {
        float a = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) a += dws[(size_t)r * D + d];
        dw_part[(size_t)blockIdx.x * D + d] = a;
    }
}

// Rows of exactly 128 elements (the head width of the tensor-core lane): the row lives in registers, and a warp works on
// four rows at a time with all of their loads issued before the first reduction, so that a thread has 8-12 independent
// 8-byte (bf16) loads in flight instead of one row's worth.
constexpr int kRmsRows = 4;

template <bool BF16>
__global__ void __launch_bounds__(256) rmsnorm_fwd128_kernel(long long rows, float eps, const void* __restrict__ x,
                                                             const void* __restrict__ gate, const float* __restrict__ w,
                                                             void* __restrict__ y, float* __restrict__ inv_rms) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long nwarp = (long long)gridDim.x * 8;
    const float4 ww = *reinterpret_cast<const float4*>(w + 4 * lane);
    const float wa[4] = {ww.x, ww.y, ww.z, ww.w};
    for (long long row0 = warp0 * kRmsRows; row0 < rows; row0 += nwarp * kRmsRows) {
        float a[kRmsRows][4], gt[kRmsRows][4], ss[kRmsRows];
#pragma unroll
        for (int r = 0; r < kRmsRows; ++r) {
            const size_t base = (size_t)min(row0 + r, rows - 1) * 128 + 4 * lane;
            ld4<BF16>(a[r], x, base);
            ld4<BF16>(gt[r], gate, base);
        }
#pragma unroll
        for (int r = 0; r < kRmsRows; ++r) ss[r] = a[r][0] * a[r][0] + a[r][1] * a[r][1] + a[r][2] * a[r][2] + a[r][3] * a[r][3];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < kRmsRows; ++r) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], o);
#pragma unroll
        for (int r = 0; r < kRmsRows; ++r) {
            if (row0 + r < rows) {
                const float inv = rsqrtf(ss[r] * (1.0f / 128.0f) + eps);
                if (lane == 0) inv_rms[row0 + r] = inv;
                float out[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) out[e] = a[r][e] * inv * wa[e] * sigmoid_t<BF16>(gt[r][e]);
                st4<BF16>(y, (size_t)(row0 + r) * 128 + 4 * lane, out);
            }
        }
    }
}

template <bool BF16>
__global__ void __launch_bounds__(256) rmsnorm_bwd128_kernel(long long rows, const void* __restrict__ x,
                                                             const void* __restrict__ gate, const float* __restrict__ w,
                                                             const float* __restrict__ inv_rms, const void* __restrict__ dy,
                                                             void* __restrict__ dx, void* __restrict__ dgate,
                                                             float* __restrict__ dw_part) {
    __shared__ float dws[8][128];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long warp0 = (long long)blockIdx.x * 8 + wid;
    const long long nwarp = (long long)gridDim.x * 8;
    const float4 ww = *reinterpret_cast<const float4*>(w + 4 * lane);
    const float wa[4] = {ww.x, ww.y, ww.z, ww.w};
    float dwa[4] = {0.f, 0.f, 0.f, 0.f};
    for (long long row0 = warp0 * kRmsRows; row0 < rows; row0 += nwarp * kRmsRows) {
        float a[kRmsRows][4], gt[kRmsRows][4], gy[kRmsRows][4], inv[kRmsRows], dot[kRmsRows];
#pragma unroll
        for (int r = 0; r < kRmsRows; ++r) {
            const long long rr = min(row0 + r, rows - 1);
            const size_t base = (size_t)rr * 128 + 4 * lane;
            ld4<BF16>(a[r], x, base);
            ld4<BF16>(gt[r], gate, base);
            ld4<BF16>(gy[r], dy, base);
            inv[r] = inv_rms[rr];
        }
#pragma unroll
        for (int r = 0; r < kRmsRows; ++r) {
            dot[r] = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                gt[r][e] = sigmoid_t<BF16>(gt[r][e]);          // s
                a[r][e] *= inv[r];                             // n
                dot[r] += gy[r][e] * gt[r][e] * wa[e] * a[r][e];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < kRmsRows; ++r) dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], o);
#pragma unroll
        for (int r = 0; r < kRmsRows; ++r) {
            if (row0 + r < rows) {
                const float mean = dot[r] * (1.0f / 128.0f);
                float ox[4], og[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float n = a[r][e], sg = gt[r][e];
                    const float du = gy[r][e] * sg;
                    og[e] = gy[r][e] * n * wa[e] * sg * (1.f - sg);
                    ox[e] = inv[r] * (du * wa[e] - n * mean);
                    dwa[e] += du * n;
                }
                const size_t base = (size_t)(row0 + r) * 128 + 4 * lane;
                st4<BF16>(dx, base, ox);
                st4<BF16>(dgate, base, og);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) dws[wid][4 * lane + e] = dwa[e];
    __syncthreads();
    if (threadIdx.x < 128) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) t += dws[r][threadIdx.x];
        dw_part[(size_t)blockIdx.x * 128 + threadIdx.x] = t;
    }
}

// out[i] = sum over b of part[b][i]: 32 columns per block, 32 row segments summed in a fixed order
__global__ void __launch_bounds__(1024) column_sum_kernel(int nblk, int N, const float* __restrict__ part_all,
                                                          ColumnSumItems outs) {
    __shared__ float red[32][33];
    const float* __restrict__ part = part_all + (size_t)blockIdx.y * nblk * N;     // blockIdx.y = item
    float* __restrict__ out = pick_item(outs.out, (int)blockIdx.y);
    const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + lane;
    float a = 0.f;
    if (i < N)
        for (int b = seg; b < nblk; b += 32) a += part[(size_t)b * N + i];
    red[seg][lane] = a;
    __syncthreads();
    if (seg == 0 && i < N) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) t += red[r][lane];
        out[i] = t;
    }
}


}  // namespace pw
}  // namespace kda

// =============================================================================================
// C ABI
// =============================================================================================
using namespace kda;

extern "C" int kda_gate_fwd(int32_t tokens, int32_t heads, int32_t key_dim, int32_t io_dtype, const void* raw_gate,
                            const void* beta_logits, const float* A_log, const float* dt_bias, float lower_bound,
                            float* g_out, float* beta_out, void* stream) {
    if (tokens < 0 || heads <= 0 || key_dim <= 0) return KDA_ERR_BAD_SHAPE;
    if (tokens == 0) return KDA_OK;
    if (!raw_gate || !beta_logits || !A_log || !dt_bias || !g_out || !beta_out) return KDA_ERR_NULL;
    const size_t n = (size_t)tokens * heads * key_dim;
    cudaStream_t fst = (cudaStream_t)stream;
    const bool al = ((reinterpret_cast<uintptr_t>(raw_gate) | reinterpret_cast<uintptr_t>(dt_bias) | reinterpret_cast<uintptr_t>(g_out)) % 16) == 0;
    if (key_dim % 4 == 0 && al && n / 4 < (1ull << 31) && (size_t)tokens * heads < (1ull << 31)) {
        const unsigned n4 = (unsigned)(n / 4), nb = (unsigned)((size_t)tokens * heads);
        const int blocks4 = (int)std::min<size_t>(((size_t)n4 + 255) / 256, 148 * 16);
        if (io_dtype == KDA_DTYPE_BF16)
            KDA_LAUNCH("gate_fwd_kernel", fst, pw::gate_fwd4_kernel<true><<<blocks4, 256, 0, fst>>>(n4, nb, heads, key_dim, raw_gate, beta_logits, A_log, dt_bias, lower_bound, g_out, beta_out));
        else
            KDA_LAUNCH("gate_fwd_kernel", fst, pw::gate_fwd4_kernel<false><<<blocks4, 256, 0, fst>>>(n4, nb, heads, key_dim, raw_gate, beta_logits, A_log, dt_bias, lower_bound, g_out, beta_out));
        return launch_status();
    }
    const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 16);
    KDA_LAUNCH("gate_fwd_kernel", (cudaStream_t)stream, pw::gate_fwd_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(n, (size_t)tokens * heads, heads, key_dim,
                                                                   io_dtype == KDA_DTYPE_BF16, raw_gate, beta_logits,
                                                                   A_log, dt_bias, lower_bound, g_out, beta_out));
    return launch_status();
}

extern "C" size_t kda_gate_bwd_scratch_bytes(int32_t tokens, int32_t heads, int32_t key_dim) {
    const size_t nblk = (size_t)ceil_div(tokens > 0 ? tokens : 1, pw::kGateRows);
    return align_up(2 * nblk * heads * key_dim * sizeof(float), 256);
}

extern "C" int kda_gate_bwd(int32_t tokens, int32_t heads, int32_t key_dim, int32_t io_dtype, const void* raw_gate,
                            const void* beta_logits, const float* A_log, const float* dt_bias, float lower_bound,
                            const float* dg, const float* dbeta, void* d_raw_gate, void* d_beta_logits, float* dA_log,
                            float* ddt_bias, void* scratch, size_t scratch_bytes, void* stream) {
    if (tokens < 0 || heads <= 0 || key_dim <= 0) return KDA_ERR_BAD_SHAPE;
    if (!A_log || !dt_bias || !dA_log || !ddt_bias) return KDA_ERR_NULL;
    if (tokens > 0 && (!raw_gate || !beta_logits || !dg || !dbeta || !d_raw_gate || !d_beta_logits)) return KDA_ERR_NULL;
    if (!scratch || scratch_bytes < kda_gate_bwd_scratch_bytes(tokens, heads, key_dim)) return KDA_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int nblk = tokens > 0 ? ceil_div(tokens, pw::kGateRows) : 0;
    float* part_b = static_cast<float*>(scratch);
    float* part_a = part_b + (size_t)(nblk > 0 ? nblk : 1) * heads * key_dim;
    const bool al = ((reinterpret_cast<uintptr_t>(raw_gate) | reinterpret_cast<uintptr_t>(dt_bias) | reinterpret_cast<uintptr_t>(dg) |
                      reinterpret_cast<uintptr_t>(d_raw_gate)) % 16) == 0;
    if (nblk > 0 && key_dim % 4 == 0 && al) {
        const dim3 grid(ceil_div(heads * key_dim, 128), nblk);
        if (io_dtype == KDA_DTYPE_BF16)
            KDA_LAUNCH("gate_bwd_kernel", st, pw::gate_bwd4_kernel<true><<<grid, 256, 0, st>>>(tokens, heads, key_dim, raw_gate, beta_logits, A_log, dt_bias, lower_bound, dg, dbeta, d_raw_gate, d_beta_logits, part_b, part_a));
        else
            KDA_LAUNCH("gate_bwd_kernel", st, pw::gate_bwd4_kernel<false><<<grid, 256, 0, st>>>(tokens, heads, key_dim, raw_gate, beta_logits, A_log, dt_bias, lower_bound, dg, dbeta, d_raw_gate, d_beta_logits, part_b, part_a));
    } else if (nblk > 0)
        KDA_LAUNCH("gate_bwd_kernel", st, pw::gate_bwd_kernel<<<nblk, 256, 0, st>>>(tokens, heads, key_dim, io_dtype == KDA_DTYPE_BF16, raw_gate,
                                                  beta_logits, A_log, dt_bias, lower_bound, dg, dbeta, d_raw_gate,
                                                  d_beta_logits, part_b, part_a));
    KDA_LAUNCH("gate_bwd_reduce_kernel", st, pw::gate_bwd_reduce_kernel<<<heads, 1024, 0, st>>>(nblk, heads, key_dim, part_b, part_a, ddt_bias, dA_log));
    return launch_status();
}

static int decode_launch(int n_seq, int heads, int key_dim, int value_dim, int bf16, int gbf16, int l2norm, float scale, const void* q,
                         const void* k, const void* v, const void* g, const void* beta, const float* state_in, float* state_out,
                         void* o, cudaStream_t st, pw::RawGate raw = pw::RawGate{nullptr, nullptr, 0.f}) {
    // four rows in flight per warp: at ~70 registers three to four CTAs share an SM, so one CTA's prologue (norms, decay) hides
    // under the others' streaming; eight rows per warp measured 20 % slower
    // one CTA per (sequence, head) once there are enough of them to fill the GPU; otherwise split the value rows
    const int rows_per_cta = (n_seq * heads >= 148 * 4) ? value_dim : 32;
    dim3 grid(n_seq * heads, ceil_div(value_dim, rows_per_cta));
    const bool vec = (key_dim % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(state_in) | reinterpret_cast<uintptr_t>(state_out)) % 16 == 0);
    if (vec && key_dim <= 128)
        KDA_LAUNCH("decode_kernel", st, pw::decode_kernel<1, 4><<<grid, 256, 0, st>>>(heads, key_dim, value_dim, bf16, gbf16, l2norm, scale, q, k, v, g, beta, state_in, state_out, o, rows_per_cta, raw));
    else if (vec)
        KDA_LAUNCH("decode_kernel", st, pw::decode_kernel<2, 4><<<grid, 256, 0, st>>>(heads, key_dim, value_dim, bf16, gbf16, l2norm, scale, q, k, v, g, beta, state_in, state_out, o, rows_per_cta, raw));
    else
        KDA_LAUNCH("decode_kernel", st, pw::decode_kernel<0, 4><<<grid, 256, 0, st>>>(heads, key_dim, value_dim, bf16, gbf16, l2norm, scale, q, k, v, g, beta, state_in, state_out, o, rows_per_cta, raw));
    return launch_status();
}

extern "C" int kda_decode_step_raw(int32_t n_seq, int32_t heads, int32_t key_dim, int32_t value_dim, int32_t io_dtype, float scale,
                                   const void* q, const void* k, const void* v, const void* raw_gate, const void* beta_logits,
                                   const float* A_log, const float* dt_bias, float lower_bound, const float* state_in,
                                   float* state_out, void* o, void* stream) {
    if (n_seq < 0 || heads <= 0 || key_dim <= 0 || value_dim <= 0 || key_dim > KDA_MAX_DIM || value_dim > KDA_MAX_DIM)
        return KDA_ERR_BAD_SHAPE;
    if (n_seq == 0) return KDA_OK;
    if (!q || !k || !v || !raw_gate || !beta_logits || !A_log || !dt_bias || !state_in || !state_out || !o) return KDA_ERR_NULL;
    const int bf16 = io_dtype == KDA_DTYPE_BF16;
    return decode_launch(n_seq, heads, key_dim, value_dim, bf16, bf16, 1, scale, q, k, v, raw_gate, beta_logits, state_in, state_out, o,
                         (cudaStream_t)stream, pw::RawGate{A_log, dt_bias, lower_bound});
}

extern "C" int kda_decode_step(int32_t n_seq, int32_t heads, int32_t key_dim, int32_t value_dim, int32_t io_dtype,
                               int32_t gate_dtype, int32_t l2norm, float scale, const void* q, const void* k, const void* v, const void* g,
                               const void* beta, const float* state_in, float* state_out, void* o, void* stream) {
    if (n_seq < 0 || heads <= 0 || key_dim <= 0 || value_dim <= 0 || key_dim > KDA_MAX_DIM || value_dim > KDA_MAX_DIM)
        return KDA_ERR_BAD_SHAPE;
    if (n_seq == 0) return KDA_OK;
    if (!q || !k || !v || !g || !beta || !state_in || !state_out || !o) return KDA_ERR_NULL;
    return decode_launch(n_seq, heads, key_dim, value_dim, io_dtype == KDA_DTYPE_BF16, gate_dtype == KDA_DTYPE_BF16, l2norm, scale, q, k,
                         v, g, beta, state_in, state_out, o, (cudaStream_t)stream);
}

extern "C" int kda_decode_steps(int32_t n_steps, int32_t n_seq, int32_t heads, int32_t key_dim, int32_t value_dim, int32_t io_dtype,
                                int32_t gate_dtype, int32_t l2norm, float scale, const void* q, const void* k, const void* v,
                                const void* g, const void* beta, float* state, void* o, void* stream) {
    if (n_steps < 0 || n_seq < 0 || heads <= 0 || key_dim <= 0 || value_dim <= 0 || key_dim > KDA_MAX_DIM || value_dim > KDA_MAX_DIM)
        return KDA_ERR_BAD_SHAPE;
    if (n_seq == 0 || n_steps == 0) return KDA_OK;
    if (!q || !k || !v || !g || !beta || !state || !o) return KDA_ERR_NULL;
    const int bf16 = io_dtype == KDA_DTYPE_BF16, gbf16 = gate_dtype == KDA_DTYPE_BF16;
    const size_t io_b = bf16 ? 2 : 4, g_b = gbf16 ? 2 : 4;
    const size_t nk = (size_t)n_seq * heads * key_dim, nv = (size_t)n_seq * heads * value_dim, nb = (size_t)n_seq * heads;
    auto at = [](const void* p, size_t bytes) { return static_cast<const void*>(static_cast<const char*>(p) + bytes); };
    for (int i = 0; i < n_steps; ++i) {
        // the state is updated in place: a warp reads a whole row before it writes it, and no row is shared between warps
        int rc = decode_launch(n_seq, heads, key_dim, value_dim, bf16, gbf16, l2norm, scale, at(q, i * nk * io_b), at(k, i * nk * io_b),
                               at(v, i * nv * io_b), at(g, i * nk * g_b), at(beta, i * nb * g_b), state, state,
                               static_cast<char*>(o) + i * nv * io_b, (cudaStream_t)stream);
        if (rc) return rc;
    }
    return KDA_OK;
}

namespace {

// training path (no carried-in window, no final state) for n same-shaped convolutions in one launch
template <int W>
int conv_fwd_fast(int n, int B, int T, int C, int bf16, int wf32, int silu, const pw::ConvFwdItems& it, cudaStream_t st) {
    const int vec = C % 128 == 0 ? 4 : 2;         // channels per thread
    const dim3 grid(ceil_div(C, 32 * vec), ceil_div(T, 8 * pw::kConvPairT), B * n);
    if (vec == 4) {
        if (bf16) KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_pair_kernel<W, 4, true><<<grid, 256, 0, st>>>(B, T, C, silu, wf32, it));
        else KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_pair_kernel<W, 4, false><<<grid, 256, 0, st>>>(B, T, C, silu, wf32, it));
    } else {
        if (bf16) KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_pair_kernel<W, 2, true><<<grid, 256, 0, st>>>(B, T, C, silu, wf32, it));
        else KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_pair_kernel<W, 2, false><<<grid, 256, 0, st>>>(B, T, C, silu, wf32, it));
    }
    return launch_status();
}

template <int W>
int conv_bwd_fast(int n, int B, int T, int C, int bf16, int wf32, int silu, const pw::ConvBwdItems& it, float* const* dwgt,
                  float* part, cudaStream_t st) {
    dim3 grid(ceil_div(C, pw::kConvTileC), ceil_div(T, pw::kConvTileT), B * n);
    // tokens per thread run of the streaming kernel: long runs amortise the W-1 halo rows; below ~12 warps per SM at
    // 32-token runs the tile kernel (64 tokens x 64 channels per block, more and smaller blocks) is the faster one
    const long long warps64 = (long long)(C / 128) * ceil_div(T, 64) * B * n;
    if (bf16 && C % 128 == 0 && warps64 >= 148LL * 12) {
        const int run = warps64 >= 148LL * 48 ? 64 : 32;
        grid = dim3(C / 128, ceil_div(T, 8 * run), B * n);                  // never more partial rows than the tile kernel's
        const size_t ring_bytes = (size_t)pw::kConvRingDepth * 2 * 256 * 8;
        if (cudaFuncSetAttribute(pw::conv_bwd_ring_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring_bytes) != cudaSuccess)
            return KDA_ERR_CUDA;
        KDA_LAUNCH("conv_bwd_kernel", st, pw::conv_bwd_ring_kernel<W><<<grid, 256, ring_bytes, st>>>(B, T, C, run, silu, wf32, it, part));
    } else if (bf16) KDA_LAUNCH("conv_bwd_kernel", st, pw::conv_bwd_tile_kernel<W, true><<<grid, 256, 0, st>>>(B, T, C, silu, wf32, it, part));
    else KDA_LAUNCH("conv_bwd_kernel", st, pw::conv_bwd_tile_kernel<W, false><<<grid, 256, 0, st>>>(B, T, C, silu, wf32, it, part));
    const int nblk = grid.y * B;                  // partial rows per item
    pw::ColumnSumItems outs = {};
    for (int i = 0; i < n; ++i) outs.out[i] = dwgt[i];
    KDA_LAUNCH("conv_dw_reduce_kernel", st, pw::column_sum_kernel<<<dim3(ceil_div(C * W, 32), n), 1024, 0, st>>>(nblk, C * W, part, outs));
    return launch_status();
}

template <int W>
int conv_fwd_w(int B, int T, int C, int bf16, int wf32, int silu, const void* x, const void* w, const void* cache, void* y,
               void* fin, cudaStream_t st) {
    const int ntile = ceil_div(T, pw::kConvTT);
    auto blocks = [&](int vec) { return (unsigned)(((size_t)B * ntile * (C / vec) + 255) / 256); };
    const bool al16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16) == 0;
    if (!cache && !fin && C % 2 == 0 && al16) {
        pw::ConvFwdItems it = {};
        it.x[0] = x; it.w[0] = w; it.y[0] = y;
        return conv_fwd_fast<W>(1, B, T, C, bf16, wf32, silu, it, st);
    }
    if (bf16) {
        if (C % 8 == 0 && al16) KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_kernel<W, 8, true><<<blocks(8), 256, 0, st>>>(B, T, C, silu, wf32, x, w, cache, y, fin));
        else KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_kernel<W, 1, true><<<blocks(1), 256, 0, st>>>(B, T, C, silu, wf32, x, w, cache, y, fin));
    } else {
        if (C % 4 == 0 && al16) KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_kernel<W, 4, false><<<blocks(4), 256, 0, st>>>(B, T, C, silu, wf32, x, w, cache, y, fin));
        else KDA_LAUNCH("conv_fwd_kernel", st, pw::conv_fwd_kernel<W, 1, false><<<blocks(1), 256, 0, st>>>(B, T, C, silu, wf32, x, w, cache, y, fin));
    }
    return launch_status();
}

inline void conv_bwd_grid(int B, int T, int C, int vec, dim3& grid) {
    grid = dim3(ceil_div(C / vec, 16), ceil_div(ceil_div(T, pw::kConvBT), 16), B);
}

template <int W>
int conv_bwd_w(int B, int T, int C, int bf16, int wf32, int silu, const void* x, const void* w, const void* cache, const void* dy,
               const void* dfin, void* dx, void* dcache, float* dwgt, float* part, cudaStream_t st) {
    const bool al16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) % 16) == 0;
    dim3 grid, block(16, 16);
    if constexpr (W <= 4) {
        // no carried-in window and no final-state cotangent: the tiled kernel (same partial layout: one row of
        // partials per 64-token tile and batch entry)
        if (!cache && !dfin && !dcache && C % 2 == 0 && al16) {
            pw::ConvBwdItems it = {};
            it.x[0] = x; it.w[0] = w; it.dy[0] = dy; it.dx[0] = dx;
            return conv_bwd_fast<W>(1, B, T, C, bf16, wf32, silu, it, &dwgt, part, st);
        }
    }
    // the vector path keeps W*VEC partials per thread in shared memory; wide windows use the scalar path
    constexpr bool kVecOk = W <= 4;
    if (bf16) {
        if constexpr (kVecOk) {
            if (C % 8 == 0 && al16) {
                conv_bwd_grid(B, T, C, 8, grid);
                KDA_LAUNCH("conv_bwd_kernel", st, pw::conv_bwd_kernel<W, 8, true><<<grid, block, 0, st>>>(B, T, C, silu, wf32, x, w, cache, dy, dfin, dx, dcache, part));
            }
        }
        if (!(kVecOk && C % 8 == 0 && al16)) {
            conv_bwd_grid(B, T, C, 1, grid);
            KDA_LAUNCH("conv_bwd_kernel", st, pw::conv_bwd_kernel<W, 1, true><<<grid, block, 0, st>>>(B, T, C, silu, wf32, x, w, cache, dy, dfin, dx, dcache, part));
        }
    } else {
        if constexpr (kVecOk) {
            if (C % 4 == 0 && al16) {
                conv_bwd_grid(B, T, C, 4, grid);
                KDA_LAUNCH("conv_bwd_kernel", st, pw::conv_bwd_kernel<W, 4, false><<<grid, block, 0, st>>>(B, T, C, silu, wf32, x, w, cache, dy, dfin, dx, dcache, part));
            }
        }
        if (!(kVecOk && C % 4 == 0 && al16)) {
            conv_bwd_grid(B, T, C, 1, grid);
            KDA_LAUNCH("conv_bwd_kernel", st, pw::conv_bwd_kernel<W, 1, false><<<grid, block, 0, st>>>(B, T, C, silu, wf32, x, w, cache, dy, dfin, dx, dcache, part));
        }
    }
    const int nblk = grid.y * grid.z;
    pw::ColumnSumItems outs = {};
    outs.out[0] = dwgt;
    KDA_LAUNCH("conv_dw_reduce_kernel", st, pw::column_sum_kernel<<<ceil_div(C * W, 32), 1024, 0, st>>>(nblk, C * W, part, outs));
    return launch_status();
}

}  // namespace

#define KDA_CONV_SWITCH(CALL)            \
    switch (width) {                     \
        case 1: return CALL(1);          \
        case 2: return CALL(2);          \
        case 3: return CALL(3);          \
        case 4: return CALL(4);          \
        case 5: return CALL(5);          \
        case 6: return CALL(6);          \
        case 7: return CALL(7);          \
        case 8: return CALL(8);          \
        default: return KDA_ERR_UNSUPPORTED; \
    }

extern "C" int kda_conv_fwd(int32_t batch, int32_t seq_len, int32_t channels, int32_t width, int32_t io_dtype,
                            int32_t silu, const void* x, const void* weight, const void* initial_state, void* y,
                            void* final_state, void* stream) {
    if (batch <= 0 || seq_len <= 0 || channels <= 0 || width <= 0) return KDA_ERR_BAD_SHAPE;
    if (!x || !weight || !y) return KDA_ERR_NULL;
    const int wf32 = (io_dtype & KDA_WEIGHT_F32) != 0;
    const int bf16 = (io_dtype & 0xff) == KDA_DTYPE_BF16;
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(WW) conv_fwd_w<WW>(batch, seq_len, channels, bf16, wf32, silu, x, weight, initial_state, y, final_state, st)
    KDA_CONV_SWITCH(CALL)
#undef CALL
}

extern "C" size_t kda_conv_bwd_scratch_bytes(int32_t batch, int32_t seq_len, int32_t channels, int32_t width) {
    const size_t nblk = (size_t)ceil_div(ceil_div(seq_len > 0 ? seq_len : 1, pw::kConvBT), 16) * (batch > 0 ? batch : 1);
    return align_up(nblk * channels * width * sizeof(float), 256);
}

extern "C" int kda_conv_bwd(int32_t batch, int32_t seq_len, int32_t channels, int32_t width, int32_t io_dtype,
                            int32_t silu, const void* x, const void* weight, const void* initial_state, const void* d_y,
                            const void* d_final_state, void* dx, float* dweight, void* d_initial_state, void* scratch,
                            size_t scratch_bytes, void* stream) {
    if (batch <= 0 || seq_len <= 0 || channels <= 0 || width <= 0) return KDA_ERR_BAD_SHAPE;
    if (!x || !weight || !d_y || !dx || !dweight) return KDA_ERR_NULL;
    if (!scratch || scratch_bytes < kda_conv_bwd_scratch_bytes(batch, seq_len, channels, width)) return KDA_ERR_WORKSPACE;
    const int wf32 = (io_dtype & KDA_WEIGHT_F32) != 0;
    const int bf16 = (io_dtype & 0xff) == KDA_DTYPE_BF16;
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(WW)                                                                                                  \
    conv_bwd_w<WW>(batch, seq_len, channels, bf16, wf32, silu, x, weight, initial_state, d_y, d_final_state, dx,  \
                   d_initial_state, dweight, static_cast<float*>(scratch), st)
    KDA_CONV_SWITCH(CALL)
#undef CALL
}

// n same-shaped convolutions (the q, k and v branches of a layer) in one launch each way: training path only (no
// carried-in window, no final state), width <= 4, even channel count, 16-byte aligned tensors; anything else returns
// KDA_ERR_UNSUPPORTED and the caller issues the per-tensor calls.
namespace {
bool conv_multi_ok(int n, int channels, int width, const void* const* a, const void* const* b, const void* const* c) {
    if (n < 1 || n > pw::kConvItems || width > 4 || channels % 2 != 0) return false;
    for (int i = 0; i < n; ++i) {
        if (!a[i] || !b[i] || (c && !c[i])) return false;
        if ((reinterpret_cast<uintptr_t>(a[i]) | reinterpret_cast<uintptr_t>(b[i]) | (c ? reinterpret_cast<uintptr_t>(c[i]) : 0)) % 16) return false;
    }
    return true;
}
}  // namespace

extern "C" int kda_conv_fwd_multi(int32_t n_items, int32_t batch, int32_t seq_len, int32_t channels, int32_t width,
                                  int32_t io_dtype, int32_t silu, const void* const* x, const void* const* weight,
                                  void* const* y, void* stream) {
    if (batch <= 0 || seq_len <= 0 || channels <= 0 || width <= 0) return KDA_ERR_BAD_SHAPE;
    if (!x || !weight || !y) return KDA_ERR_NULL;
    if (!conv_multi_ok(n_items, channels, width, x, const_cast<const void* const*>(y), nullptr)) return KDA_ERR_UNSUPPORTED;
    const int wf32 = (io_dtype & KDA_WEIGHT_F32) != 0;
    const int bf16 = (io_dtype & 0xff) == KDA_DTYPE_BF16;
    pw::ConvFwdItems it = {};
    for (int i = 0; i < n_items; ++i) {
        if (!weight[i]) return KDA_ERR_NULL;
        it.x[i] = x[i]; it.w[i] = weight[i]; it.y[i] = y[i];
    }
    cudaStream_t st = (cudaStream_t)stream;
    switch (width) {
        case 1: return conv_fwd_fast<1>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, st);
        case 2: return conv_fwd_fast<2>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, st);
        case 3: return conv_fwd_fast<3>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, st);
        default: return conv_fwd_fast<4>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, st);
    }
}

extern "C" int kda_conv_step_multi(int32_t n_items, int32_t batch, int32_t channels, int32_t width, int32_t io_dtype, int32_t silu,
                                   const void* const* x, const void* const* weight, void* const* cache, void* const* y, void* stream) {
    if (n_items < 1 || n_items > 4 || batch <= 0 || channels <= 0) return KDA_ERR_BAD_SHAPE;
    if (width < 1 || width > 4) return KDA_ERR_UNSUPPORTED;
    if (!x || !weight || !cache || !y) return KDA_ERR_NULL;
    const int wf32 = (io_dtype & KDA_WEIGHT_F32) != 0;
    const int bf16 = (io_dtype & 0xff) == KDA_DTYPE_BF16;
    pw::ConvStepItems it = {};
    for (int i = 0; i < n_items; ++i) {
        if (!x[i] || !weight[i] || !cache[i] || !y[i]) return KDA_ERR_NULL;
        it.x[i] = x[i]; it.w[i] = weight[i]; it.cache[i] = cache[i]; it.y[i] = y[i];
    }
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(ceil_div(batch * channels, 256), n_items);
#define KDA_CONV_STEP(WW)                                                                                                          \
    do {                                                                                                                           \
        if (bf16) KDA_LAUNCH("conv_step_kernel", st, pw::conv_step_kernel<WW, true><<<grid, 256, 0, st>>>(batch, channels, silu, wf32, it)); \
        else KDA_LAUNCH("conv_step_kernel", st, pw::conv_step_kernel<WW, false><<<grid, 256, 0, st>>>(batch, channels, silu, wf32, it));     \
    } while (0)
    switch (width) {
        case 1: KDA_CONV_STEP(1); break;
        case 2: KDA_CONV_STEP(2); break;
        case 3: KDA_CONV_STEP(3); break;
        default: KDA_CONV_STEP(4); break;
    }
#undef KDA_CONV_STEP
    return launch_status();
}

extern "C" size_t kda_conv_bwd_multi_scratch_bytes(int32_t n_items, int32_t batch, int32_t seq_len, int32_t channels, int32_t width) {
    return (size_t)(n_items > 0 ? n_items : 1) * kda_conv_bwd_scratch_bytes(batch, seq_len, channels, width);
}

extern "C" int kda_conv_bwd_multi(int32_t n_items, int32_t batch, int32_t seq_len, int32_t channels, int32_t width,
                                  int32_t io_dtype, int32_t silu, const void* const* x, const void* const* weight,
                                  const void* const* d_y, void* const* dx, float* const* dweight, void* scratch,
                                  size_t scratch_bytes, void* stream) {
    if (batch <= 0 || seq_len <= 0 || channels <= 0 || width <= 0) return KDA_ERR_BAD_SHAPE;
    if (!x || !weight || !d_y || !dx || !dweight) return KDA_ERR_NULL;
    if (!conv_multi_ok(n_items, channels, width, x, d_y, const_cast<const void* const*>(dx))) return KDA_ERR_UNSUPPORTED;
    if (!scratch || scratch_bytes < kda_conv_bwd_multi_scratch_bytes(n_items, batch, seq_len, channels, width)) return KDA_ERR_WORKSPACE;
    const int wf32 = (io_dtype & KDA_WEIGHT_F32) != 0;
    const int bf16 = (io_dtype & 0xff) == KDA_DTYPE_BF16;
    pw::ConvBwdItems it = {};
    for (int i = 0; i < n_items; ++i) {
        if (!weight[i] || !dweight[i]) return KDA_ERR_NULL;
        it.x[i] = x[i]; it.w[i] = weight[i]; it.dy[i] = d_y[i]; it.dx[i] = dx[i];
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* part = static_cast<float*>(scratch);
    switch (width) {
        case 1: return conv_bwd_fast<1>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, dweight, part, st);
        case 2: return conv_bwd_fast<2>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, dweight, part, st);
        case 3: return conv_bwd_fast<3>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, dweight, part, st);
        default: return conv_bwd_fast<4>(n_items, batch, seq_len, channels, bf16, wf32, silu, it, dweight, part, st);
    }
}

namespace {
inline int rms_blocks(long long rows) { return (int)std::min<long long>((rows + 7) / 8, 148LL * 4); }
}  // namespace

extern "C" int kda_rmsnorm_gate_fwd(int64_t rows, int32_t dim, int32_t io_dtype, float eps, const void* x,
                                    const void* gate, const float* weight, void* y, float* inv_rms, void* stream) {
    if (rows < 0 || dim <= 0 || dim > 1024) return KDA_ERR_BAD_SHAPE;
    if (rows == 0) return KDA_OK;
    if (!x || !gate || !weight || !y || !inv_rms) return KDA_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    const int nb = rms_blocks(rows);
    const bool vec = dim % 128 == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(y) |
                       reinterpret_cast<uintptr_t>(weight)) % 16) == 0;
    if (vec && dim == 128) {
        const int nb4 = (int)std::min<long long>((rows + 8 * pw::kRmsRows - 1) / (8 * pw::kRmsRows), 148LL * 8);
        if (io_dtype == KDA_DTYPE_BF16) KDA_LAUNCH("rmsnorm_fwd_kernel", st, pw::rmsnorm_fwd128_kernel<true><<<nb4, 256, 0, st>>>(rows, eps, x, gate, weight, y, inv_rms));
        else KDA_LAUNCH("rmsnorm_fwd_kernel", st, pw::rmsnorm_fwd128_kernel<false><<<nb4, 256, 0, st>>>(rows, eps, x, gate, weight, y, inv_rms));
        return launch_status();
    }
    if (io_dtype == KDA_DTYPE_BF16) {
        if (vec) KDA_LAUNCH("rmsnorm_fwd_kernel", st, pw::rmsnorm_fwd_kernel<true, true><<<nb, 256, 0, st>>>(rows, dim, eps, x, gate, weight, y, inv_rms));
        else KDA_LAUNCH("rmsnorm_fwd_kernel", st, pw::rmsnorm_fwd_kernel<true, false><<<nb, 256, 0, st>>>(rows, dim, eps, x, gate, weight, y, inv_rms));
    } else {
        if (vec) KDA_LAUNCH("rmsnorm_fwd_kernel", st, pw::rmsnorm_fwd_kernel<false, true><<<nb, 256, 0, st>>>(rows, dim, eps, x, gate, weight, y, inv_rms));
        else KDA_LAUNCH("rmsnorm_fwd_kernel", st, pw::rmsnorm_fwd_kernel<false, false><<<nb, 256, 0, st>>>(rows, dim, eps, x, gate, weight, y, inv_rms));
    }
    return launch_status();
}

extern "C" size_t kda_rmsnorm_gate_bwd_scratch_bytes(int64_t rows, int32_t dim) {
    return align_up((size_t)rms_blocks(rows > 0 ? rows : 1) * dim * sizeof(float), 256);
}

extern "C" int kda_rmsnorm_gate_bwd(int64_t rows, int32_t dim, int32_t io_dtype, const void* x, const void* gate,
                                    const float* weight, const float* inv_rms, const void* d_y, void* dx, void* dgate,
                                    float* dweight, void* scratch, size_t scratch_bytes, void* stream) {
    if (rows < 0 || dim <= 0 || dim > 1024) return KDA_ERR_BAD_SHAPE;
    if (!weight || !dweight) return KDA_ERR_NULL;
    if (rows > 0 && (!x || !gate || !inv_rms || !d_y || !dx || !dgate)) return KDA_ERR_NULL;
    if (!scratch || scratch_bytes < kda_rmsnorm_gate_bwd_scratch_bytes(rows, dim)) return KDA_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int nb = rows > 0 ? rms_blocks(rows) : 0;
    float* part = static_cast<float*>(scratch);
    const size_t smem = (size_t)8 * dim * sizeof(float);
    const bool vec = dim % 128 == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(d_y) |
                       reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dgate) | reinterpret_cast<uintptr_t>(weight)) % 16) == 0;
    if (nb > 0 && vec && dim == 128) {
        if (io_dtype == KDA_DTYPE_BF16) KDA_LAUNCH("rmsnorm_bwd_kernel", st, pw::rmsnorm_bwd128_kernel<true><<<nb, 256, 0, st>>>(rows, x, gate, weight, inv_rms, d_y, dx, dgate, part));
        else KDA_LAUNCH("rmsnorm_bwd_kernel", st, pw::rmsnorm_bwd128_kernel<false><<<nb, 256, 0, st>>>(rows, x, gate, weight, inv_rms, d_y, dx, dgate, part));
    } else if (nb > 0) {
        if (io_dtype == KDA_DTYPE_BF16) {
            if (vec) KDA_LAUNCH("rmsnorm_bwd_kernel", st, pw::rmsnorm_bwd_kernel<true, true><<<nb, 256, smem, st>>>(rows, dim, x, gate, weight, inv_rms, d_y, dx, dgate, part));
            else KDA_LAUNCH("rmsnorm_bwd_kernel", st, pw::rmsnorm_bwd_kernel<true, false><<<nb, 256, smem, st>>>(rows, dim, x, gate, weight, inv_rms, d_y, dx, dgate, part));
        } else {
            if (vec) KDA_LAUNCH("rmsnorm_bwd_kernel", st, pw::rmsnorm_bwd_kernel<false, true><<<nb, 256, smem, st>>>(rows, dim, x, gate, weight, inv_rms, d_y, dx, dgate, part));
            else KDA_LAUNCH("rmsnorm_bwd_kernel", st, pw::rmsnorm_bwd_kernel<false, false><<<nb, 256, smem, st>>>(rows, dim, x, gate, weight, inv_rms, d_y, dx, dgate, part));
        }
    }
    pw::ColumnSumItems outs = {};
    outs.out[0] = dweight;
    KDA_LAUNCH("rmsnorm_dw_reduce_kernel", st, pw::column_sum_kernel<<<ceil_div(dim, 32), 1024, 0, st>>>(nb, dim, part, outs));
    return launch_status();
}

// =============================================================================================
// Allocation-free variant of the gated-RMSNorm backward
// =============================================================================================
// The regular backward needs a caller-provided scratch buffer for the per-block partial sums of the
// weight gradient.  Some callers have nowhere to get one: code running against a frozen memory plan
// (a serving engine that sized all of its device memory at start-up), a plugin that is handed tensors
// but no allocator, or anything that must not call cudaMalloc because that call synchronises the
// device.  For them the partials live in a fixed array inside the library image.
namespace {
constexpr int kStaticMaxDim = 256;                 // widest row the static variant accepts
constexpr int kStaticMaxBlocks = 148 * 8;          // the backward never launches more blocks than this
constexpr int kMaxDevices = 64;
static __device__ __align__(256) float g_rms_static_scratch[(size_t)kStaticMaxBlocks * kStaticMaxDim];   // 1.2 MB per GPU
float* g_rms_static_ptr[kMaxDevices] = {nullptr};  // device address of the array, per device ordinal
}  // namespace

extern "C" int kda_rmsnorm_gate_bwd_static(int64_t rows, int32_t dim, int32_t io_dtype, const void* x, const void* gate,
                                           const float* weight, const float* inv_rms, const void* d_y, void* dx,
                                           void* dgate, float* dweight, void* stream) {
    if (rows < 0 || dim <= 0) return KDA_ERR_BAD_SHAPE;
    if (dim > kStaticMaxDim) return KDA_ERR_UNSUPPORTED;   // beyond the built-in scratch: use kda_rmsnorm_gate_bwd
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return KDA_ERR_CUDA;
    if (g_rms_static_ptr[device] == nullptr) {
        // In host code the array's name is only a handle; the kernels need its address on the current device.
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_rms_static_scratch) != cudaSuccess || p == nullptr) return KDA_ERR_CUDA;
        g_rms_static_ptr[device] = static_cast<float*>(p);
    }
    const size_t bytes = (size_t)kStaticMaxBlocks * kStaticMaxDim * sizeof(float);
    return kda_rmsnorm_gate_bwd(rows, dim, io_dtype, x, gate, weight, inv_rms, d_y, dx, dgate, dweight,
                                g_rms_static_ptr[device], bytes, stream);
}

