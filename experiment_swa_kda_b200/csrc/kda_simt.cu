// Chunked KDA forward and backward in float32 on the CUDA cores ("fp32 lane").
//
// General shapes: any K, V <= 256, any sequence length, packed sequences,
// initial / final state.  Every matrix of the chunked WY algebra is handled as
// 64x64 float32 tiles staged in shared memory; rows beyond a ragged chunk tail
// and columns beyond K / V are zero, which makes them inert in every product
// (zero q, k, v, beta and log-decay rows leave A, M, T, U, W, Z and all adjoints
// unchanged for the valid rows).
//
// Per chunk (64 tokens of one sequence and head), H = incoming state [K,V]:
//   G = cumsum(g);  A = tril(sum_d qn kn rho);  M = beta * stril(sum_d kn kn rho), rho = exp(G_i - G_s)
//   T = (I + M)^-1;  U = T (beta v);  W = T (beta exp(G) kn);  Z = U - W H
//   O = (qn exp(G)) H + A Z;  H' = exp(G_end) H + (kn exp(G_end - G))^T Z
// The equations restate reference chunk_wy_forward.cu:125-405, 761-858, 940-1275, 1498-1588
// and, for the adjoints, chunk_wy_backward.cu:2445-2562, 2818-3331, 3337-3552, 3787-3894.

#include <cstdlib>

#include "common.cuh"
#include "simt_ws.cuh"
#include "tc_ws.cuh"

namespace kda {
namespace simt {

// ---------------------------------------------------------------------------------------------
// tile helpers (256 threads)
// ---------------------------------------------------------------------------------------------

// 64x64 tile from a padded float32 array (row stride ld_src floats, 16-byte aligned).
template <bool TR>
__device__ __forceinline__ void ld_tile(float* dst, const float* __restrict__ src, size_t ld_src) {
    for (int idx = threadIdx.x; idx < 1024; idx += 256) {
        int r = idx >> 4, c4 = (idx & 15) << 2;
        float4 x = *reinterpret_cast<const float4*>(src + (size_t)r * ld_src + c4);
        if (!TR) {
            *reinterpret_cast<float4*>(dst + r * kLD + c4) = x;
        } else {
            dst[(c4 + 0) * kLD + r] = x.x;
            dst[(c4 + 1) * kLD + r] = x.y;
            dst[(c4 + 2) * kLD + r] = x.z;
            dst[(c4 + 3) * kLD + r] = x.w;
        }
    }
}

// 64x64 tile from a caller tensor in its I/O dtype; element (r,c) at base[r*stride + c]; zero outside nr x nc.
template <bool TR>
__device__ __forceinline__ void ld_tile_io(float* dst, const void* base, int bf16, size_t off, size_t stride, int nr,
                                           int nc) {
    for (int idx = threadIdx.x; idx < 4096; idx += 256) {
        int r = idx >> 6, c = idx & 63;
        float x = (r < nr && c < nc) ? ld_io(base, off + (size_t)r * stride + c, bf16) : 0.0f;
        if (!TR) dst[r * kLD + c] = x;
        else dst[c * kLD + r] = x;
    }
}

__device__ __forceinline__ void zero_acc(float (&acc)[4][4]) {
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0.0f;
}

// acc[r][c] += sum_kk At[kk][4*ty + r] * Bs[kk][4*tx + c]   (At holds the left operand transposed)
__device__ __forceinline__ void mm64(float (&acc)[4][4], const float* __restrict__ At, const float* __restrict__ Bs,
                                     int kk0 = 0, int kk1 = 64) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const float* ap = At + 4 * ty;
    const float* bp = Bs + 4 * tx;
#pragma unroll 4
    for (int kk = kk0; kk < kk1; ++kk) {
        float4 a = *reinterpret_cast<const float4*>(ap + kk * kLD);
        float4 b = *reinterpret_cast<const float4*>(bp + kk * kLD);
        acc[0][0] += a.x * b.x; acc[0][1] += a.x * b.y; acc[0][2] += a.x * b.z; acc[0][3] += a.x * b.w;
        acc[1][0] += a.y * b.x; acc[1][1] += a.y * b.y; acc[1][2] += a.y * b.z; acc[1][3] += a.y * b.w;
        acc[2][0] += a.z * b.x; acc[2][1] += a.z * b.y; acc[2][2] += a.z * b.z; acc[2][3] += a.z * b.w;
        acc[3][0] += a.w * b.x; acc[3][1] += a.w * b.y; acc[3][2] += a.w * b.z; acc[3][3] += a.w * b.w;
    }
}

// registers -> shared tile, row-major or transposed
template <bool TR>
__device__ __forceinline__ void st_acc(float* dst, const float (&acc)[4][4], float alpha = 1.0f) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (!TR) dst[(4 * ty + r) * kLD + 4 * tx + c] = alpha * acc[r][c];
            else dst[(4 * tx + c) * kLD + 4 * ty + r] = alpha * acc[r][c];
        }
}

// registers -> padded float32 global tile
__device__ __forceinline__ void st_acc_g(float* dst, size_t ld, const float (&acc)[4][4]) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
    for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float4*>(dst + (size_t)(4 * ty + r) * ld + 4 * tx) =
            make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
}

// ---------------------------------------------------------------------------------------------
// chunk table: which tokens each 64-token chunk slot covers
// ---------------------------------------------------------------------------------------------
// A packed batch is described by cu_seqlens, which the caller controls: every segment is checked against the token
// count and the slot budget before it enters the tables, so that no later kernel can be steered outside the tensors.
// A segment that starts before the previous one ends, has a negative length or reaches past `tokens` is treated as
// empty; chunks beyond the slot budget are dropped; either raises the status word (kStatusBadCuSeqlens), as does a
// table that does not start at 0 or does not end at `tokens`.
constexpr int kStatusBadCuSeqlens = 10;
constexpr int kScanOrderMax = 512;      // batches up to this many sequences get a longest-first scan order

__global__ void chunk_table_kernel(Ws w, const int32_t* __restrict__ cu, int n_seq, int seq_len, int tokens, int* status) {
    __shared__ int total;
    if (threadIdx.x == 0) {
        int flag = 0;
        int acc = 0, prev_end = 0;
        for (int s = 0; s < n_seq; ++s) {
            w.seq_chunk0[s] = acc;
            int len = seq_len;
            if (cu) {
                const int t0 = cu[s], t1 = cu[s + 1];
                len = t1 - t0;
                if (t0 < prev_end || len < 0 || t1 > tokens) { len = 0; flag = 1; }
                else prev_end = t1;
            }
            int nc = (len + kChunk - 1) / kChunk;
            if (acc + nc > w.nslots) { nc = w.nslots - acc; flag = 1; }
            acc += nc;
        }
        if (cu && (cu[0] != 0 || prev_end != tokens)) flag = 1;
        w.seq_chunk0[n_seq] = acc;
        total = acc;
        *status = flag ? kStatusBadCuSeqlens : 0;      // every forward starts with a clean status word
    }
    __syncthreads();
    for (int s = threadIdx.x; s < n_seq; s += blockDim.x) {
        const int c0 = w.seq_chunk0[s], nc = w.seq_chunk0[s + 1] - c0;
        const int t0 = cu ? cu[s] : s * seq_len;
        const int len = cu ? (cu[s + 1] - cu[s]) : seq_len;
        for (int j = 0; j < nc; ++j) {
            w.chunk_seq[c0 + j] = s;
            w.chunk_tok0[c0 + j] = t0 + j * kChunk;
            w.chunk_len[c0 + j] = min(kChunk, len - j * kChunk);
        }
    }
    // Scan order: the scans run one CTA per (sequence, head) with one CTA per SM, so starting the longest chains first
    // keeps the tail of the launch short (longest-processing-time-first).  Rank by counting; identity for large batches,
    // which balance by themselves.
    for (int s = threadIdx.x; s < n_seq; s += blockDim.x) {
        int rank = s;
        if (n_seq <= kScanOrderMax) {
            const int nc = w.seq_chunk0[s + 1] - w.seq_chunk0[s];
            rank = 0;
            for (int j = 0; j < n_seq; ++j) {
                const int ncj = w.seq_chunk0[j + 1] - w.seq_chunk0[j];
                rank += (ncj > nc || (ncj == nc && j < s)) ? 1 : 0;
            }
        }
        w.seq_order[rank] = s;
    }
    for (int c = total + threadIdx.x; c < w.nslots; c += blockDim.x) {
        w.chunk_seq[c] = -1;
        w.chunk_tok0[c] = 0;
        w.chunk_len[c] = 0;
    }
}

// ---------------------------------------------------------------------------------------------
// K1  prep: normalise q, k; cumulative log-decay; padded float32 copies
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prep_kernel(Ws w, const void* __restrict__ q, const void* __restrict__ k,
                                                   const void* __restrict__ g, const void* __restrict__ beta, int bf16,
                                                   int gbf16, int l2norm, float scale) {
    const int slot = blockIdx.x, h = blockIdx.y;
    const int len = w.chunk_len[slot];
    if (len == 0) return;
    const int tok0 = w.chunk_tok0[slot];
    const int K = w.K, Kp = w.Kp, H = w.H;
    const size_t ch = (size_t)slot * H + h;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int i = warp; i < kChunk; i += 8) {
        float* qo = w.qn + (ch * kChunk + i) * Kp;
        float* ko = w.kn + (ch * kChunk + i) * Kp;
        if (i < len) {
            size_t off = ((size_t)(tok0 + i) * H + h) * K;
            float sq = 0.f, sk = 0.f;
            for (int d = lane; d < K; d += 32) {
                float a = ld_io(q, off + d, bf16), b = ld_io(k, off + d, bf16);
                sq += a * a;
                sk += b * b;
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            float qi = l2norm ? 1.0f / fmaxf(sqrtf(sq), 1e-12f) : 1.0f;
            float ki = l2norm ? 1.0f / fmaxf(sqrtf(sk), 1e-12f) : 1.0f;
            for (int d = lane; d < Kp; d += 32) {
                qo[d] = d < K ? ld_io(q, off + d, bf16) * qi * scale : 0.f;
                ko[d] = d < K ? ld_io(k, off + d, bf16) * ki : 0.f;
            }
            if (lane == 0) {
                w.qinv[ch * kChunk + i] = qi;
                w.kinv[ch * kChunk + i] = ki;
                w.beta[ch * kChunk + i] = ld_io(beta, (size_t)(tok0 + i) * H + h, gbf16);
            }
        } else {
            for (int d = lane; d < Kp; d += 32) { qo[d] = 0.f; ko[d] = 0.f; }
            if (lane == 0) {
                w.qinv[ch * kChunk + i] = 0.f;
                w.kinv[ch * kChunk + i] = 0.f;
                w.beta[ch * kChunk + i] = 0.f;
            }
        }
    }
    for (int d = threadIdx.x; d < Kp; d += 256) {
        float run = 0.f;
        float* Go = w.G + ch * kChunk * Kp + d;
        for (int i = 0; i < kChunk; ++i) {
            if (i < len && d < K) run += ld_io(g, ((size_t)(tok0 + i) * H + h) * K + d, gbf16);
            Go[(size_t)i * Kp] = run;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// K2  A, M under the decay mask and T = (I + M)^-1
// ---------------------------------------------------------------------------------------------

// dst[m x n] (+)= alpha * A[m x kd] * B[kd x n]; all row-major with leading dimension kLD
__device__ __forceinline__ void small_mm(float* dst, const float* A, const float* B, int m, int n, int kd, float alpha) {
    for (int idx = threadIdx.x; idx < m * n; idx += 256) {
        int i = idx / n, j = idx - i * n;
        float s = 0.f;
        for (int t = 0; t < kd; ++t) s += A[i * kLD + t] * B[t * kLD + j];
        dst[i * kLD + j] = alpha * s;
    }
}

// In-place inverse of the unit lower-triangular L = I + Ms (Ms strictly lower, 64x64) -> Ts.
// Block forward substitution: 16x16 diagonal blocks, then 32x32 and 64x64 merges
//   inv([[A,0],[C,B]]) = [[Ai,0],[-Bi C Ai, Bi]].
__device__ void unit_lower_inverse(const float* Ms, float* Ts, float* tmp) {
    const int tid = threadIdx.x;
    for (int idx = tid; idx < 64 * kLD; idx += 256) Ts[idx] = 0.f;
    __syncthreads();
    if (tid < 64) {
        const int b = tid >> 4, j = tid & 15;
        const float* Lb = Ms + (16 * b) * kLD + 16 * b;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = (i == j) ? 1.f : 0.f;
#pragma unroll
        for (int i = 1; i < 16; ++i) {
            float s = 0.f;
#pragma unroll
            for (int t = 0; t < i; ++t) s += Lb[i * kLD + t] * x[t];
            x[i] = (i > j) ? -s : x[i];
        }
        float* Tb = Ts + (16 * b) * kLD + 16 * b;
#pragma unroll
        for (int i = 0; i < 16; ++i) Tb[i * kLD + j] = x[i];
    }
    __syncthreads();
    // 32x32 merges (two independent pairs)
    for (int p = 0; p < 2; ++p) {
        const int o = 32 * p;
        small_mm(tmp + p * 16 * kLD, Ms + (o + 16) * kLD + o, Ts + o * kLD + o, 16, 16, 16, 1.f);  // C * Ai
    }
    __syncthreads();
    for (int p = 0; p < 2; ++p) {
        const int o = 32 * p;
        small_mm(Ts + (o + 16) * kLD + o, Ts + (o + 16) * kLD + o + 16, tmp + p * 16 * kLD, 16, 16, 16, -1.f);
    }
    __syncthreads();
    // 64x64 merge
    small_mm(tmp, Ms + 32 * kLD, Ts, 32, 32, 32, 1.f);
    __syncthreads();
    small_mm(Ts + 32 * kLD, Ts + 32 * kLD + 32, tmp, 32, 32, 32, -1.f);
    __syncthreads();
}

__global__ void __launch_bounds__(256) build_am_kernel(Ws w) {
    extern __shared__ __align__(16) float sm[];
    float* qT = sm;                  // [d][i]
    float* kT = qT + 64 * kLD;
    float* GT = kT + 64 * kLD;
    float* Ms = GT + 64 * kLD;
    float* Ts = Ms + 64 * kLD;
    float* tmp = Ts + 64 * kLD;      // 32 rows
    const int slot = blockIdx.x, h = blockIdx.y;
    if (w.chunk_len[slot] == 0) return;
    const size_t ch = (size_t)slot * w.H + h;
    const int Kp = w.Kp;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float accA[4][4], accM[4][4];
    zero_acc(accA);
    zero_acc(accM);
    for (int kt = 0; kt < Kp / 64; ++kt) {
        __syncthreads();
        ld_tile<true>(qT, w.qn + ch * kChunk * Kp + kt * 64, Kp);
        ld_tile<true>(kT, w.kn + ch * kChunk * Kp + kt * 64, Kp);
        ld_tile<true>(GT, w.G + ch * kChunk * Kp + kt * 64, Kp);
        __syncthreads();
        if (tx <= ty) {
            for (int d = 0; d < 64; ++d) {
                float4 qi = *reinterpret_cast<const float4*>(qT + d * kLD + 4 * ty);
                float4 ki = *reinterpret_cast<const float4*>(kT + d * kLD + 4 * ty);
                float4 gi = *reinterpret_cast<const float4*>(GT + d * kLD + 4 * ty);
                float4 ks = *reinterpret_cast<const float4*>(kT + d * kLD + 4 * tx);
                float4 gs = *reinterpret_cast<const float4*>(GT + d * kLD + 4 * tx);
                const float qa[4] = {qi.x, qi.y, qi.z, qi.w}, ka[4] = {ki.x, ki.y, ki.z, ki.w};
                const float ga[4] = {gi.x, gi.y, gi.z, gi.w}, kb[4] = {ks.x, ks.y, ks.z, ks.w};
                const float gb[4] = {gs.x, gs.y, gs.z, gs.w};
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if (4 * ty + r >= 4 * tx + c) {
                            float t = kb[c] * expf(ga[r] - gb[c]);
                            accA[r][c] += qa[r] * t;
                            accM[r][c] += ka[r] * t;
                        }
                    }
            }
        }
    }
    __syncthreads();
    const float* bet = w.beta + ch * kChunk;
    float* Ao = w.A + ch * 4096;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = 4 * ty + r;
        const float bi = bet[i];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int s = 4 * tx + c;
            Ao[i * 64 + s] = (s <= i) ? accA[r][c] : 0.f;
            Ms[i * kLD + s] = (s < i) ? bi * accM[r][c] : 0.f;
        }
    }
    __syncthreads();
    unit_lower_inverse(Ms, Ts, tmp);
    float* To = w.T + ch * 4096;
    for (int idx = threadIdx.x; idx < 4096; idx += 256) To[idx] = Ts[(idx >> 6) * kLD + (idx & 63)];
}

// ---------------------------------------------------------------------------------------------
// K3  U = T (beta v),  W = T (beta exp(G) kn); one 64-column tile per CTA
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) uw_kernel(Ws w, const void* __restrict__ v, int bf16) {
    extern __shared__ __align__(16) float sm[];
    float* Tt = sm;               // [s][i] = T[i][s]
    float* Bs = Tt + 64 * kLD;    // [s][col]
    const int slot = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int len = w.chunk_len[slot];
    if (len == 0) return;
    const size_t ch = (size_t)slot * w.H + h;
    const int Kp = w.Kp, Vp = w.Vp, KT = Kp / 64;
    const float* bet = w.beta + ch * kChunk;
    ld_tile<true>(Tt, w.T + ch * 4096, 64);
    if (z < KT) {
        const float* kn = w.kn + ch * kChunk * Kp + z * 64;
        const float* G = w.G + ch * kChunk * Kp + z * 64;
        for (int idx = threadIdx.x; idx < 4096; idx += 256) {
            int s = idx >> 6, d = idx & 63;
            Bs[s * kLD + d] = bet[s] * expf(G[(size_t)s * Kp + d]) * kn[(size_t)s * Kp + d];
        }
    } else {
        const int vt = z - KT;
        const int tok0 = w.chunk_tok0[slot];
        const int nc = min(64, w.V - vt * 64);
        ld_tile_io<false>(Bs, v, bf16, ((size_t)tok0 * w.H + h) * w.V + vt * 64, (size_t)w.H * w.V, len, nc);
        __syncthreads();
        for (int idx = threadIdx.x; idx < 4096; idx += 256) Bs[(idx >> 6) * kLD + (idx & 63)] *= bet[idx >> 6];
    }
    __syncthreads();
    float acc[4][4];
    zero_acc(acc);
    mm64(acc, Tt, Bs);
    if (z < KT) st_acc_g(w.W + ch * kChunk * Kp + z * 64, Kp, acc);
    else st_acc_g(w.Z + ch * kChunk * Vp + (z - KT) * 64, Vp, acc);
}

// ---------------------------------------------------------------------------------------------
// K4  forward state scan over the chunks of one (sequence, head, 16-column value strip)
// ---------------------------------------------------------------------------------------------
constexpr int kVS = 16;

__global__ void __launch_bounds__(256) scan_fwd_kernel(Ws w, const float* __restrict__ h0, float* __restrict__ final_state) {
    extern __shared__ __align__(16) float sm[];
    const int Kp = w.Kp, Vp = w.Vp, K = w.K, V = w.V, H = w.H;
    const int ldw = Kp + 1;
    float* Ws_ = sm;                       // [64][Kp+1]
    float* Es = Ws_ + 64 * ldw;            // [64][Kp+1]
    float* Hs = Es + 64 * ldw;             // [Kp][16]
    float* Zs = Hs + Kp * kVS;             // [64][16]
    float* eGe = Zs + 64 * kVS;            // [Kp]
    const int seq = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kVS;
    const int tid = threadIdx.x;

    for (int idx = tid; idx < Kp * kVS; idx += 256) {
        int kk = idx / kVS, vv = idx % kVS;
        float x = 0.f;
        if (h0 && kk < K && v0 + vv < V) x = h0[(((size_t)seq * H + h) * V + v0 + vv) * K + kk];
        Hs[idx] = x;
    }
    const int c_begin = w.seq_chunk0[seq], c_end = w.seq_chunk0[seq + 1];
    for (int slot = c_begin; slot < c_end; ++slot) {
        const size_t ch = (size_t)slot * H + h;
        __syncthreads();
        const float* Wg = w.W + ch * kChunk * Kp;
        const float* kng = w.kn + ch * kChunk * Kp;
        const float* Gg = w.G + ch * kChunk * Kp;
        for (int idx = tid; idx < Kp; idx += 256) eGe[idx] = Gg[(size_t)63 * Kp + idx];
        __syncthreads();
        for (int idx = tid; idx < 64 * Kp; idx += 256) {
            int i = idx / Kp, d = idx - i * Kp;
            Ws_[i * ldw + d] = Wg[idx];
            Es[i * ldw + d] = kng[idx] * expf(eGe[d] - Gg[idx]);
        }
        // publish the chunk-start state for the output kernel and the backward
        float* Hg = w.Hc + ch * Kp * Vp;
        for (int idx = tid; idx < Kp * kVS; idx += 256) Hg[(size_t)(idx / kVS) * Vp + v0 + (idx % kVS)] = Hs[idx];
        __syncthreads();
        // Z = U - W H   (thread: row i, 4 value columns)
        {
            const int i = tid >> 2, vq = (tid & 3) << 2;
            float* Zg = w.Z + (ch * kChunk + i) * Vp + v0 + vq;
            float4 u = *reinterpret_cast<const float4*>(Zg);
            float a0 = u.x, a1 = u.y, a2 = u.z, a3 = u.w;
            const float* wr = Ws_ + i * ldw;
            for (int kk = 0; kk < Kp; ++kk) {
                float wv = wr[kk];
                float4 hv = *reinterpret_cast<const float4*>(Hs + kk * kVS + vq);
                a0 -= wv * hv.x; a1 -= wv * hv.y; a2 -= wv * hv.z; a3 -= wv * hv.w;
            }
            *reinterpret_cast<float4*>(Zg) = make_float4(a0, a1, a2, a3);
            *reinterpret_cast<float4*>(Zs + i * kVS + vq) = make_float4(a0, a1, a2, a3);
        }
        __syncthreads();
        for (int idx = tid; idx < Kp; idx += 256) eGe[idx] = expf(eGe[idx]);
        __syncthreads();
        // H <- exp(G_end) H + E^T Z   (thread: key row kk, 4 value columns)
        for (int o = tid; o < Kp * 4; o += 256) {
            const int kk = o >> 2, vq = (o & 3) << 2;
            float4 hv = *reinterpret_cast<const float4*>(Hs + kk * kVS + vq);
            const float dec = eGe[kk];
            float a0 = dec * hv.x, a1 = dec * hv.y, a2 = dec * hv.z, a3 = dec * hv.w;
            for (int i = 0; i < 64; ++i) {
                float e = Es[i * ldw + kk];
                float4 zv = *reinterpret_cast<const float4*>(Zs + i * kVS + vq);
                a0 += e * zv.x; a1 += e * zv.y; a2 += e * zv.z; a3 += e * zv.w;
            }
            *reinterpret_cast<float4*>(Hs + kk * kVS + vq) = make_float4(a0, a1, a2, a3);
        }
    }
    __syncthreads();
    if (final_state) {
        for (int idx = tid; idx < Kp * kVS; idx += 256) {
            int vv = idx / Kp, kk = idx - vv * Kp;
            if (kk < K && v0 + vv < V) final_state[(((size_t)seq * H + h) * V + v0 + vv) * K + kk] = Hs[kk * kVS + vv];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// K5  output  O = (qn exp(G)) H + A Z; one 64-column value tile per CTA
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) out_kernel(Ws w, void* __restrict__ o, int bf16) {
    extern __shared__ __align__(16) float sm[];
    float* At = sm;
    float* Bs = At + 64 * kLD;
    const int slot = blockIdx.x, h = blockIdx.y, vt = blockIdx.z;
    const int len = w.chunk_len[slot];
    if (len == 0) return;
    const size_t ch = (size_t)slot * w.H + h;
    const int Kp = w.Kp, Vp = w.Vp;
    float acc[4][4];
    zero_acc(acc);
    for (int kt = 0; kt < Kp / 64; ++kt) {
        __syncthreads();
        const float* qn = w.qn + ch * kChunk * Kp + kt * 64;
        const float* G = w.G + ch * kChunk * Kp + kt * 64;
        for (int idx = threadIdx.x; idx < 4096; idx += 256) {
            int i = idx >> 6, d = idx & 63;
            At[d * kLD + i] = qn[(size_t)i * Kp + d] * expf(G[(size_t)i * Kp + d]);
        }
        ld_tile<false>(Bs, w.Hc + (ch * Kp + kt * 64) * Vp + vt * 64, Vp);
        __syncthreads();
        mm64(acc, At, Bs);
    }
    __syncthreads();
    ld_tile<true>(At, w.A + ch * 4096, 64);
    ld_tile<false>(Bs, w.Z + ch * kChunk * Vp + vt * 64, Vp);
    __syncthreads();
    mm64(acc, At, Bs);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int tok0 = w.chunk_tok0[slot];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = 4 * ty + r;
        if (i >= len) continue;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int vv = vt * 64 + 4 * tx + c;
            if (vv < w.V) st_io(o, ((size_t)(tok0 + i) * w.H + h) * w.V + vv, bf16, acc[r][c]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// K6  reverse scan of the state adjoint
//   dZ = A^T dO + E dH' ;  dH = R^T dO + exp(G_end) dH' - W^T dZ
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) scan_bwd_kernel(Ws w, Scr s, const void* __restrict__ d_o, int bf16,
                                                       const float* __restrict__ d_final, float* __restrict__ dh0) {
    extern __shared__ __align__(16) float sm[];
    const int Kp = w.Kp, Vp = w.Vp, K = w.K, V = w.V, H = w.H;
    const int ldw = Kp + 1;
    float* B1 = sm;                      // [64][Kp+1]  E, then R
    float* B2 = B1 + 64 * ldw;           // [64][Kp+1]  W
    float* As = B2 + 64 * ldw;           // [64][kLD]   A row-major
    float* dHs = As + 64 * kLD;          // [Kp][16]
    float* dHn = dHs + Kp * kVS;         // [Kp][16]   new value
    float* dOs = dHn + Kp * kVS;         // [64][16]
    float* dZs = dOs + 64 * kVS;         // [64][16]
    float* eGe = dZs + 64 * kVS;         // [Kp]
    const int seq = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kVS;
    const int tid = threadIdx.x;

    for (int idx = tid; idx < Kp * kVS; idx += 256) {
        int kk = idx / kVS, vv = idx % kVS;
        float x = 0.f;
        if (d_final && kk < K && v0 + vv < V) x = d_final[(((size_t)seq * H + h) * V + v0 + vv) * K + kk];
        dHs[idx] = x;
    }
    const int c_begin = w.seq_chunk0[seq], c_end = w.seq_chunk0[seq + 1];
    for (int slot = c_end - 1; slot >= c_begin; --slot) {
        const size_t ch = (size_t)slot * H + h;
        const int len = w.chunk_len[slot], tok0 = w.chunk_tok0[slot];
        __syncthreads();
        const float* kng = w.kn + ch * kChunk * Kp;
        const float* qng = w.qn + ch * kChunk * Kp;
        const float* Gg = w.G + ch * kChunk * Kp;
        const float* Wg = w.W + ch * kChunk * Kp;
        for (int idx = tid; idx < Kp; idx += 256) eGe[idx] = Gg[(size_t)63 * Kp + idx];
        ld_tile<false>(As, w.A + ch * 4096, 64);
        for (int idx = tid; idx < 64 * kVS; idx += 256) {
            int i = idx / kVS, vv = idx % kVS;
            dOs[idx] = (i < len && v0 + vv < V) ? ld_io(d_o, ((size_t)(tok0 + i) * H + h) * V + v0 + vv, bf16) : 0.f;
        }
        __syncthreads();
        for (int idx = tid; idx < 64 * Kp; idx += 256) {
            int i = idx / Kp, d = idx - i * Kp;
            B1[i * ldw + d] = kng[idx] * expf(eGe[d] - Gg[idx]);
            B2[i * ldw + d] = Wg[idx];
        }
        // publish dH' (adjoint of this chunk's outgoing state)
        float* dHg = s.dHn + ch * Kp * Vp;
        for (int idx = tid; idx < Kp * kVS; idx += 256) dHg[(size_t)(idx / kVS) * Vp + v0 + (idx % kVS)] = dHs[idx];
        __syncthreads();
        // dZ[i] = sum_{s>=i} A[s][i] dO[s] + sum_k E[i][k] dH'[k]
        {
            const int i = tid >> 2, vq = (tid & 3) << 2;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            for (int ss = i; ss < 64; ++ss) {
                float av = As[ss * kLD + i];
                float4 dv = *reinterpret_cast<const float4*>(dOs + ss * kVS + vq);
                a0 += av * dv.x; a1 += av * dv.y; a2 += av * dv.z; a3 += av * dv.w;
            }
            const float* er = B1 + i * ldw;
            for (int kk = 0; kk < Kp; ++kk) {
                float ev = er[kk];
                float4 hv = *reinterpret_cast<const float4*>(dHs + kk * kVS + vq);
                a0 += ev * hv.x; a1 += ev * hv.y; a2 += ev * hv.z; a3 += ev * hv.w;
            }
            *reinterpret_cast<float4*>(dZs + i * kVS + vq) = make_float4(a0, a1, a2, a3);
            *reinterpret_cast<float4*>(s.dZ + (ch * kChunk + i) * Vp + v0 + vq) = make_float4(a0, a1, a2, a3);
        }
        __syncthreads();
        // B1 <- R = qn exp(G)
        for (int idx = tid; idx < 64 * Kp; idx += 256) {
            int i = idx / Kp, d = idx - i * Kp;
            B1[i * ldw + d] = qng[idx] * expf(Gg[idx]);
        }
        for (int idx = tid; idx < Kp; idx += 256) eGe[idx] = expf(eGe[idx]);
        __syncthreads();
        for (int o = tid; o < Kp * 4; o += 256) {
            const int kk = o >> 2, vq = (o & 3) << 2;
            float4 hv = *reinterpret_cast<const float4*>(dHs + kk * kVS + vq);
            const float dec = eGe[kk];
            float a0 = dec * hv.x, a1 = dec * hv.y, a2 = dec * hv.z, a3 = dec * hv.w;
            for (int i = 0; i < 64; ++i) {
                float rv = B1[i * ldw + kk], wv = B2[i * ldw + kk];
                float4 ov = *reinterpret_cast<const float4*>(dOs + i * kVS + vq);
                float4 zv = *reinterpret_cast<const float4*>(dZs + i * kVS + vq);
                a0 += rv * ov.x - wv * zv.x; a1 += rv * ov.y - wv * zv.y;
                a2 += rv * ov.z - wv * zv.z; a3 += rv * ov.w - wv * zv.w;
            }
            *reinterpret_cast<float4*>(dHn + kk * kVS + vq) = make_float4(a0, a1, a2, a3);
        }
        __syncthreads();
        for (int idx = tid; idx < Kp * kVS; idx += 256) dHs[idx] = dHn[idx];
    }
    __syncthreads();
    if (dh0) {
        for (int idx = tid; idx < Kp * kVS; idx += 256) {
            int vv = idx / Kp, kk = idx - vv * Kp;
            if (kk < K && v0 + vv < V) dh0[(((size_t)seq * H + h) * V + v0 + vv) * K + kk] = dHs[kk * kVS + vv];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// K7  chunk-local adjoints: dv, dA, dM and the direct parts of dqn, dkn, dG, dbeta
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_local_kernel(Ws w, Scr s, const void* __restrict__ v,
                                                        const void* __restrict__ d_o, void* __restrict__ dv, int bf16) {
    extern __shared__ __align__(16) float sm[];
    float* Tr = sm;                 // T row-major  [s][i] view gives T^T products
    float* Tt = Tr + 64 * kLD;      // T transposed
    float* P0 = Tt + 64 * kLD;      // operand tiles
    float* P1 = P0 + 64 * kLD;
    float* P2 = P1 + 64 * kLD;
    float* P3 = P2 + 64 * kLD;
    float* P4 = P3 + 64 * kLD;
    float* red = P4 + 64 * kLD;     // [64][17] row partials / [16][64] column partials
    float* dbv = red + 64 * 17;     // [64]
    const int slot = blockIdx.x, h = blockIdx.y;
    const int len = w.chunk_len[slot];
    if (len == 0) return;
    const int tok0 = w.chunk_tok0[slot];
    const size_t ch = (size_t)slot * w.H + h;
    const int Kp = w.Kp, Vp = w.Vp, KT = Kp / 64, VT = Vp / 64, H = w.H, V = w.V;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const float* bet = w.beta + ch * kChunk;

    ld_tile<false>(Tr, w.T + ch * 4096, 64);
    ld_tile<true>(Tt, w.T + ch * 4096, 64);
    if (tid < 64) dbv[tid] = 0.f;
    float accX[4][4], accA[4][4], acc[4][4];
    zero_acc(accX);
    zero_acc(accA);

    // ---- value tiles: dA += dO Z^T ; X += dZ P^T ; dP = T^T dZ
    for (int vt = 0; vt < VT; ++vt) {
        const int nc = min(64, V - vt * 64);
        const size_t voff = ((size_t)tok0 * H + h) * V + vt * 64;
        __syncthreads();
        ld_tile_io<true>(P0, d_o, bf16, voff, (size_t)H * V, len, nc);          // [v][i] = dO[i][v]
        ld_tile<true>(P1, w.Z + ch * kChunk * Vp + vt * 64, Vp);                 // [v][s] = Z[s][v]
        ld_tile<true>(P2, s.dZ + ch * kChunk * Vp + vt * 64, Vp);                // [v][i] = dZ[i][v]
        ld_tile_io<true>(P3, v, bf16, voff, (size_t)H * V, len, nc);             // [v][s] = v[s][v]
        ld_tile<false>(P4, s.dZ + ch * kChunk * Vp + vt * 64, Vp);               // [s][v] = dZ[s][v]
        __syncthreads();
        for (int idx = tid; idx < 4096; idx += 256) P3[(idx >> 6) * kLD + (idx & 63)] *= bet[idx & 63];  // P^T
        mm64(accA, P0, P1);
        __syncthreads();
        mm64(accX, P2, P3);
        zero_acc(acc);
        mm64(acc, Tr, P4);   // dP[i][v] = sum_s T[s][i] dZ[s][v]
        // dv = beta dP ; dbeta += sum_v dP * v   (v[i][vv] = P3[vv][i] / beta_i, so reload v directly)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = 4 * ty + r;
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int vv = vt * 64 + 4 * tx + c;
                if (i < len && vv < V) {
                    const size_t o = ((size_t)(tok0 + i) * H + h) * V + vv;
                    part += acc[r][c] * ld_io(v, o, bf16);
                    st_io(dv, o, bf16, bet[i] * acc[r][c]);
                }
            }
            red[i * 17 + tx] = part;
        }
        __syncthreads();
        if (tid < 64) {
            float t = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) t += red[tid * 17 + j];
            dbv[tid] += t;
        }
    }

    // ---- key tiles
    for (int kt = 0; kt < KT; ++kt) {
        float aR[4][4], aE[4][4], aW[4][4];
        zero_acc(aR);
        zero_acc(aE);
        zero_acc(aW);
        float dd = 0.f;   // threads < 64: sum_v dH'[k][v] H[k][v]
        for (int vt = 0; vt < VT; ++vt) {
            const int nc = min(64, V - vt * 64);
            const size_t voff = ((size_t)tok0 * H + h) * V + vt * 64;
            __syncthreads();
            ld_tile_io<true>(P0, d_o, bf16, voff, (size_t)H * V, len, nc);                   // dO^T
            ld_tile<true>(P1, w.Z + ch * kChunk * Vp + vt * 64, Vp);                          // Z^T
            ld_tile<true>(P2, s.dZ + ch * kChunk * Vp + vt * 64, Vp);                         // dZ^T
            ld_tile<true>(P3, w.Hc + (ch * Kp + kt * 64) * Vp + vt * 64, Vp);                 // [v][k] = H[k][v]
            ld_tile<true>(P4, s.dHn + (ch * Kp + kt * 64) * Vp + vt * 64, Vp);                // [v][k] = dH'[k][v]
            __syncthreads();
            mm64(aR, P0, P3);
            mm64(aE, P1, P4);
            mm64(aW, P2, P3);
            if (tid < 64) {
                for (int vv = 0; vv < 64; ++vv) dd += P3[vv * kLD + tid] * P4[vv * kLD + tid];
            }
        }
        __syncthreads();
        // dW to shared in both orientations; Q^T tile for X -= dW Q^T
        st_acc<true>(P0, aW);    // [k][i]
        st_acc<false>(P1, aW);   // [s][k]
        {
            const float* kn = w.kn + ch * kChunk * Kp + kt * 64;
            const float* G = w.G + ch * kChunk * Kp + kt * 64;
            for (int idx = tid; idx < 4096; idx += 256) {
                int ss = idx >> 6, d = idx & 63;
                P2[d * kLD + ss] = bet[ss] * expf(G[(size_t)ss * Kp + d]) * kn[(size_t)ss * Kp + d];   // [k][s] = Q[s][k]
            }
        }
        __syncthreads();
        zero_acc(acc);
        mm64(acc, P0, P2);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) accX[r][c] -= acc[r][c];
        zero_acc(acc);
        mm64(acc, Tr, P1);     // (T^T dW)[i][k];  dQ = -that
        // element-wise part on this thread's 4x4 patch
        const float* Gp = w.G + ch * kChunk * Kp + kt * 64;
        const float* qp = w.qn + ch * kChunk * Kp + kt * 64;
        const float* kp = w.kn + ch * kChunk * Kp + kt * 64;
        float colE[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = 4 * ty + r;
            const float bi = bet[i];
            float4 g4 = *reinterpret_cast<const float4*>(Gp + (size_t)i * Kp + 4 * tx);
            float4 q4 = *reinterpret_cast<const float4*>(qp + (size_t)i * Kp + 4 * tx);
            float4 k4 = *reinterpret_cast<const float4*>(kp + (size_t)i * Kp + 4 * tx);
            float4 e4 = *reinterpret_cast<const float4*>(Gp + (size_t)63 * Kp + 4 * tx);
            const float ga[4] = {g4.x, g4.y, g4.z, g4.w}, qa[4] = {q4.x, q4.y, q4.z, q4.w};
            const float ka[4] = {k4.x, k4.y, k4.z, k4.w}, ea[4] = {e4.x, e4.y, e4.z, e4.w};
            float oq[4], ok[4], og[4];
            float brow = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float eg = expf(ga[c]);
                const float ee = expf(ea[c] - ga[c]);
                const float R = qa[c] * eg, E = ka[c] * ee;
                const float dQ = -acc[r][c];
                oq[c] = aR[r][c] * eg;
                ok[c] = aE[r][c] * ee + dQ * bi * eg;
                og[c] = aR[r][c] * R - aE[r][c] * E + dQ * bi * eg * ka[c];
                brow += dQ * eg * ka[c];
                colE[c] += aE[r][c] * E;
            }
            *reinterpret_cast<float4*>(s.dqn + (ch * kChunk + i) * Kp + kt * 64 + 4 * tx) = make_float4(oq[0], oq[1], oq[2], oq[3]);
            *reinterpret_cast<float4*>(s.dkn + (ch * kChunk + i) * Kp + kt * 64 + 4 * tx) = make_float4(ok[0], ok[1], ok[2], ok[3]);
            *reinterpret_cast<float4*>(s.dG + (ch * kChunk + i) * Kp + kt * 64 + 4 * tx) = make_float4(og[0], og[1], og[2], og[3]);
            red[i * 17 + tx] = brow;
        }
        __syncthreads();
        if (tid < 64) {
            float t = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) t += red[tid * 17 + j];
            dbv[tid] += t;
        }
        __syncthreads();
        // column sums of dE*E over the 64 rows -> dG_end
#pragma unroll
        for (int c = 0; c < 4; ++c) red[ty * 64 + 4 * tx + c] = colE[c];
        __syncthreads();
        if (tid < 64) {
            float t = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) t += red[j * 64 + tid];
            const float ge = Gp[(size_t)63 * Kp + tid];
            s.dGend[ch * Kp + kt * 64 + tid] = t + expf(ge) * dd;
        }
    }

    // ---- dM = -stril(T^T X T^T),  dA = tril(dO Z^T)
    __syncthreads();
    st_acc<false>(P0, accX);         // X row-major: [s][j]
    __syncthreads();
    zero_acc(acc);
    mm64(acc, Tr, P0);               // Y[i][j] = sum_s T[s][i] X[s][j]
    __syncthreads();
    st_acc<true>(P1, acc);           // [s][i] = Y[i][s]
    __syncthreads();
    zero_acc(acc);
    mm64(acc, P1, Tt);               // sum_s Y[i][s] T[j][s]   (Tt[s][j] = T[j][s])
    float* dAo = s.dA + ch * 4096;
    float* dMo = s.dM + ch * 4096;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = 4 * ty + r;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int j = 4 * tx + c;
            dAo[i * 64 + j] = (j <= i) ? accA[r][c] : 0.f;
            dMo[i * 64 + j] = (j < i) ? -acc[r][c] : 0.f;
        }
    }
    __syncthreads();
    if (tid < 64) s.dbl[ch * kChunk + tid] = dbv[tid];
}

// ---------------------------------------------------------------------------------------------
// K8  pull dA, dM back through the decay-masked products; finish dG and emit dg
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pullback_kernel(Ws w, Scr s, void* __restrict__ dg, int bf16) {
    extern __shared__ __align__(16) float sm[];
    float* dAs = sm;                // [i][s]
    float* dMs = dAs + 64 * kLD;    // [i][s]
    float* qs = dMs + 64 * kLD;     // [i][d]
    float* ks = qs + 64 * kLD;
    float* Gs = ks + 64 * kLD;
    float* dGs = Gs + 64 * kLD;     // [i][d] accumulated dG
    float* red = dGs + 64 * kLD;    // [64][2]
    const int slot = blockIdx.x, h = blockIdx.y, kt = blockIdx.z;
    const int len = w.chunk_len[slot];
    if (len == 0) return;
    const size_t ch = (size_t)slot * w.H + h;
    const int Kp = w.Kp, KT = Kp / 64, K = w.K;
    const int tid = threadIdx.x;
    const float* bet = w.beta + ch * kChunk;
    ld_tile<false>(dAs, s.dA + ch * 4096, 64);
    ld_tile<false>(dMs, s.dM + ch * 4096, 64);
    ld_tile<false>(qs, w.qn + ch * kChunk * Kp + kt * 64, Kp);
    ld_tile<false>(ks, w.kn + ch * kChunk * Kp + kt * 64, Kp);
    ld_tile<false>(Gs, w.G + ch * kChunk * Kp + kt * 64, Kp);
    ld_tile<false>(dGs, s.dG + ch * kChunk * Kp + kt * 64, Kp);
    __syncthreads();
    const int d = tid & 63, rg = tid >> 6;
    float* dqn = s.dqn + ch * kChunk * Kp + kt * 64;
    float* dkn = s.dkn + ch * kChunk * Kp + kt * 64;
    for (int j = 0; j < 16; ++j) {
        const int i = rg + 4 * j;
        const float gi = Gs[i * kLD + d], qi = qs[i * kLD + d], ki = ks[i * kLD + d], bi = bet[i];
        // row part: sources s <= i
        float aq = 0.f, am = 0.f;
        for (int ss = 0; ss <= i; ++ss) {
            const float t = expf(gi - Gs[ss * kLD + d]) * ks[ss * kLD + d];
            aq += dAs[i * kLD + ss] * t;
            am += dMs[i * kLD + ss] * t;   // dM[i][i] == 0
        }
        // column part: targets i2 >= i for source row i
        float a2 = 0.f;
        for (int i2 = i; i2 < 64; ++i2) {
            const float rho = expf(Gs[i2 * kLD + d] - gi);
            a2 += rho * (dAs[i2 * kLD + i] * qs[i2 * kLD + d] + bet[i2] * dMs[i2 * kLD + i] * ks[i2 * kLD + d]);
        }
        dqn[(size_t)i * Kp + d] += aq;
        dkn[(size_t)i * Kp + d] += bi * am + a2;
        dGs[i * kLD + d] += qi * aq + bi * ki * am - ki * a2;
        // dbeta_i += sum_d kn[i][d] * am
        float pb = warp_sum(ki * am);
        if ((tid & 31) == 0) red[i * 2 + ((tid >> 5) & 1)] = pb;
    }
    __syncthreads();
    if (tid < 64) s.dbp[(ch * KT + kt) * kChunk + tid] = red[tid * 2] + red[tid * 2 + 1];
    // reverse cumulative sum over the rows; the chunk-end term enters at the last row
    if (tid < 64) {
        float run = s.dGend[ch * Kp + kt * 64 + tid];
        const int tok0 = w.chunk_tok0[slot];
        const int kk = kt * 64 + tid;
        for (int i = 63; i >= 0; --i) {
            run += dGs[i * kLD + tid];
            if (i < len && kk < K) st_io(dg, ((size_t)(tok0 + i) * w.H + h) * K + kk, bf16, run);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// K9  finalize: L2-normalisation VJP for dq, dk; collect dbeta
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) finalize_kernel(Ws w, Scr s, const void* __restrict__ q, const void* __restrict__ k,
                                                       void* __restrict__ dq, void* __restrict__ dk,
                                                       void* __restrict__ dbeta, int bf16, int gbf16, int l2norm, float scale) {
    const int slot = blockIdx.x, h = blockIdx.y;
    const int len = w.chunk_len[slot];
    if (len == 0) return;
    const int tok0 = w.chunk_tok0[slot];
    const size_t ch = (size_t)slot * w.H + h;
    const int K = w.K, Kp = w.Kp, KT = Kp / 64, H = w.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = warp; i < len; i += 8) {
        const size_t off = ((size_t)(tok0 + i) * H + h) * K;
        const float* dqn = s.dqn + (ch * kChunk + i) * Kp;
        const float* dkn = s.dkn + (ch * kChunk + i) * Kp;
        const float qi = w.qinv[ch * kChunk + i], ki = w.kinv[ch * kChunk + i];
        if (l2norm) {
            float pq = 0.f, pk = 0.f;
            for (int d = lane; d < K; d += 32) {
                pq += ld_io(q, off + d, bf16) * qi * dqn[d] * scale;
                pk += ld_io(k, off + d, bf16) * ki * dkn[d];
            }
            pq = warp_sum(pq);
            pk = warp_sum(pk);
            for (int d = lane; d < K; d += 32) {
                const float qh = ld_io(q, off + d, bf16) * qi, kh = ld_io(k, off + d, bf16) * ki;
                st_io(dq, off + d, bf16, qi * (dqn[d] * scale - qh * pq));
                st_io(dk, off + d, bf16, ki * (dkn[d] - kh * pk));
            }
        } else {
            for (int d = lane; d < K; d += 32) {
                st_io(dq, off + d, bf16, dqn[d] * scale);
                st_io(dk, off + d, bf16, dkn[d]);
            }
        }
        if (lane == 0) {
            float b = s.dbl[ch * kChunk + i];
            for (int kt = 0; kt < KT; ++kt) b += s.dbp[(ch * KT + kt) * kChunk + i];
            st_io(dbeta, (size_t)(tok0 + i) * H + h, gbf16, b);
        }
    }
}

}  // namespace simt

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
using simt::Scr;
using simt::Ws;

int tc_scan_forward(const simt::Ws& w, const tc::TcWs& t, int n_seq, int tokens, const float* h0, float* final_state, void* o,
                    const tc::NormEpilogue& norm, cudaStream_t st);
int tc_intra_forward(const simt::Ws& w, const tc::TcWs& t, const void* q, const void* k, const void* v, const void* g,
                     const void* beta, int gbf16, int l2norm, float scale, int tokens, const tc::ConvPrep* conv, cudaStream_t st);
int tc_scan_backward(const simt::Ws& w, const simt::Scr& s, const tc::TcWs& t, int n_seq, int tokens, const void* d_o,
                     const float* d_final, float* dh0, cudaStream_t st);
int tc_intra_backward(const simt::Ws& w, const tc::TcWs& t, int tokens, const void* q, const void* k, const void* v,
                      const void* g, const void* d_o, int gbf16, int l2norm, float scale, void* dq, void* dk, void* dv,
                      void* dg, void* dbeta, cudaStream_t st);

template <class Kern>
static int set_smem(Kern kern, size_t bytes) {
    if (bytes > 48 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
            return KDA_ERR_CUDA;
    }
    return KDA_OK;
}

int simt_chunk_fwd(const KdaChunkShape* sh, const void* q, const void* k, const void* v, const void* g, const void* beta,
                   const float* h0, const int32_t* cu, void* o, float* final_state, void* workspace, cudaStream_t st,
                   const tc::NormEpilogue* norm, const tc::ConvPrep* conv) {
    Ws w = simt::carve_ws(*sh, workspace);
    if (conv != nullptr && (sh->lane != KDA_LANE_TC || !sh->forward_only)) return KDA_ERR_UNSUPPORTED;
    if (norm != nullptr && norm->gate != nullptr && sh->lane != KDA_LANE_TC) return KDA_ERR_UNSUPPORTED;
    const int bf16 = sh->io_dtype == KDA_DTYPE_BF16, gbf16 = sh->gate_dtype == KDA_DTYPE_BF16;
    const int KT = w.Kp / 64, VT = w.Vp / 64;
    if (sh->lane == KDA_LANE_TC) {
        // chunk-parallel operand panels and transitions on tcgen05, the affine state scan, then the chunk outputs
        size_t ws_bytes = 0;
        simt::carve_ws(*sh, nullptr, &ws_bytes);
        tc::TcWs t = tc::carve_tc(*sh, static_cast<char*>(workspace) + ws_bytes);
        t.status = w.status;      // one status word per workspace, shared by both lanes
        KDA_LAUNCH("chunk_table_kernel", st, simt::chunk_table_kernel<<<1, 256, 0, st>>>(w, cu, sh->n_seq, sh->seq_len, sh->tokens, w.status));
        if (w.nslots > 0) {
            int rc = tc_intra_forward(w, t, q, k, v, g, beta, gbf16, sh->l2norm, sh->scale, sh->tokens, conv, st);
            if (rc) return rc;
            rc = tc_scan_forward(w, t, sh->n_seq, sh->tokens, h0, final_state, o,
                                 norm != nullptr ? *norm : tc::NormEpilogue{nullptr, nullptr, 0.f, nullptr, nullptr}, st);
            if (rc) return rc;
        }
        return launch_status();
    }
    KDA_LAUNCH("chunk_table_kernel", st, simt::chunk_table_kernel<<<1, 256, 0, st>>>(w, cu, sh->n_seq, sh->seq_len, sh->tokens, w.status));
    if (w.nslots > 0) {
        dim3 gch(w.nslots, w.H);
        KDA_LAUNCH("prep_kernel", st, simt::prep_kernel<<<gch, 256, 0, st>>>(w, q, k, g, beta, bf16, gbf16, sh->l2norm, sh->scale));
        size_t sm_am = (size_t)(5 * 64 + 32) * kLD * sizeof(float);
        if (set_smem(simt::build_am_kernel, sm_am)) return KDA_ERR_CUDA;
        KDA_LAUNCH("build_am_kernel", st, simt::build_am_kernel<<<gch, 256, sm_am, st>>>(w));
        size_t sm_uw = (size_t)2 * 64 * kLD * sizeof(float);
        KDA_LAUNCH("uw_kernel", st, simt::uw_kernel<<<dim3(w.nslots, w.H, KT + VT), 256, sm_uw, st>>>(w, v, bf16));
    }
    {
        size_t sm_scan = ((size_t)2 * 64 * (w.Kp + 1) + (size_t)w.Kp * simt::kVS + 64 * simt::kVS + w.Kp) * sizeof(float);
        if (set_smem(simt::scan_fwd_kernel, sm_scan)) return KDA_ERR_CUDA;
        KDA_LAUNCH("scan_fwd_kernel", st, simt::scan_fwd_kernel<<<dim3(sh->n_seq, w.H, w.Vp / simt::kVS), 256, sm_scan, st>>>(w, h0, final_state));
    }
    if (w.nslots > 0) {
        size_t sm_out = (size_t)2 * 64 * kLD * sizeof(float);
        KDA_LAUNCH("out_kernel", st, simt::out_kernel<<<dim3(w.nslots, w.H, VT), 256, sm_out, st>>>(w, o, bf16));
    }
    return launch_status();
}

// Device status word of a forward / backward pair that used `workspace`: 0, kStatusBadCuSeqlens, or the code of the
// bounded wait that expired in the tensor-core lane.
static int status_code(int v) {
    return v == 0 ? KDA_OK : (v == simt::kStatusBadCuSeqlens ? KDA_ERR_CU_SEQLENS : KDA_ERR_DEVICE_STATUS);
}

// Reads the word back over the stream, i.e. synchronises the stream - for tests and post-mortems, not for the hot
// path (and not under stream capture).
int chunk_status(const KdaChunkShape* sh, const void* workspace, cudaStream_t st) {
    Ws w = simt::carve_ws(*sh, const_cast<void*>(workspace));
    int v = 0;
    if (cudaMemcpyAsync(&v, w.status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return KDA_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return KDA_ERR_CUDA;
    return status_code(v);
}

// Queues a copy of the word into caller-owned page-locked host memory; nothing waits.
int chunk_status_async(const KdaChunkShape* sh, const void* workspace, int32_t* host_word, cudaStream_t st) {
    Ws w = simt::carve_ws(*sh, const_cast<void*>(workspace));
    return cudaMemcpyAsync(host_word, w.status, sizeof(int), cudaMemcpyDeviceToHost, st) == cudaSuccess ? KDA_OK : KDA_ERR_CUDA;
}

int status_word_to_code(int v) { return status_code(v); }

int simt_chunk_bwd(const KdaChunkShape* sh, const void* q, const void* k, const void* v, const void* g, const void* beta,
                   const int32_t* cu, const void* d_o, const float* d_final, const void* workspace, void* scratch,
                   void* dq, void* dk, void* dv, void* dg, void* dbeta, float* dh0, cudaStream_t st) {
    (void)beta; (void)cu;
    Ws w = simt::carve_ws(*sh, const_cast<void*>(workspace));
    Scr s = simt::carve_scr(*sh, scratch);
    const int bf16 = sh->io_dtype == KDA_DTYPE_BF16, gbf16 = sh->gate_dtype == KDA_DTYPE_BF16;
    const int KT = w.Kp / 64;
    if (sh->lane == KDA_LANE_TC) {
        size_t ws_bytes = 0;
        simt::carve_ws(*sh, nullptr, &ws_bytes);
        tc::TcWs t = tc::carve_tc(*sh, static_cast<char*>(const_cast<void*>(workspace)) + ws_bytes);
        t.status = w.status;
        if (w.nslots > 0) {
            int rc = tc_scan_backward(w, s, t, sh->n_seq, sh->tokens, d_o, d_final, dh0, st);
            if (rc) return rc;
            rc = tc_intra_backward(w, t, sh->tokens, q, k, v, g, d_o, gbf16, sh->l2norm, sh->scale, dq, dk, dv, dg, dbeta, st);
            return rc ? rc : launch_status();
        } else if (dh0) {
            return KDA_ERR_UNSUPPORTED;
        }
    } else {
        size_t sm_scan = ((size_t)2 * 64 * (w.Kp + 1) + 64 * kLD + (size_t)2 * w.Kp * simt::kVS + 2 * 64 * simt::kVS + w.Kp) *
                         sizeof(float);
        if (set_smem(simt::scan_bwd_kernel, sm_scan)) return KDA_ERR_CUDA;
        KDA_LAUNCH("scan_bwd_kernel", st, simt::scan_bwd_kernel<<<dim3(sh->n_seq, w.H, w.Vp / simt::kVS), 256, sm_scan, st>>>(w, s, d_o, bf16, d_final, dh0));
    }
    if (w.nslots > 0) {
        dim3 gch(w.nslots, w.H);
        size_t sm_loc = ((size_t)7 * 64 * kLD + 64 * 17 + 128) * sizeof(float);
        if (set_smem(simt::bwd_local_kernel, sm_loc)) return KDA_ERR_CUDA;
        KDA_LAUNCH("bwd_local_kernel", st, simt::bwd_local_kernel<<<gch, 256, sm_loc, st>>>(w, s, v, d_o, dv, bf16));
        size_t sm_pb = ((size_t)6 * 64 * kLD + 128) * sizeof(float);
        if (set_smem(simt::pullback_kernel, sm_pb)) return KDA_ERR_CUDA;
        KDA_LAUNCH("pullback_kernel", st, simt::pullback_kernel<<<dim3(w.nslots, w.H, KT), 256, sm_pb, st>>>(w, s, dg, gbf16));
        KDA_LAUNCH("finalize_kernel", st, simt::finalize_kernel<<<gch, 256, 0, st>>>(w, s, q, k, dq, dk, dbeta, bf16, gbf16, sh->l2norm, sh->scale));
    }
    return launch_status();
}

}  // namespace kda
