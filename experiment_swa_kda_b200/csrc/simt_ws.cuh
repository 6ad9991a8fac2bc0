// Workspace layout of the float32 chunk lane: what the forward leaves for the
// backward (Ws) and the backward's own scratch (Scr).  All arrays are padded to
// 64-wide tiles: Kp = ceil64(K), Vp = ceil64(V); chunk-head index ch = slot*H + h.
#pragma once

#include "common.cuh"

namespace kda {
namespace simt {

struct Ws {
    int *chunk_seq, *chunk_tok0, *chunk_len, *seq_chunk0;
    int* seq_order;             // [n_seq] sequences by falling chunk count: the order the state scans start them in
    float *qn, *kn, *G, *W;     // [nch][64][Kp]   scaled unit q, unit k, cumulative log-decay, W
    float* Z;                   // [nch][64][Vp]   U after the intra-chunk step, Z after the scan
    float *A, *T;               // [nch][64][64]
    float* Hc;                  // [nch][Kp][Vp]   state at the start of each chunk
    float *qinv, *kinv, *beta;  // [nch][64]
    int* status;                // device status word of the forward / backward pair that owns this workspace (0 = ok)
    int nslots, H, K, V, Kp, Vp;
};

struct Scr {
    float* dZ;              // [nch][64][Vp]
    float* dHn;             // [nch][Kp][Vp]   adjoint of each chunk's outgoing state
    float *dqn, *dkn, *dG;  // [nch][64][Kp]
    float *dA, *dM;         // [nch][64][64]
    float* dGend;           // [nch][Kp]
    float* dbl;             // [nch][64]
    float* dbp;             // [nch][KT][64]
};

inline int slots_for(const KdaChunkShape& sh, bool varlen_hint) {
    // Upper bound on the number of 64-token chunk slots.  Packed batches may end every
    // sequence with a ragged chunk; the same bound is used for fixed-length batches so
    // that forward and backward agree without knowing whether cu_seqlens was given.
    (void)varlen_hint;
    if (sh.seq_len > 0 && (long long)sh.n_seq * sh.seq_len == sh.tokens)
        return sh.n_seq * ceil_div(sh.seq_len, kChunk);
    return sh.tokens / kChunk + sh.n_seq;
}

struct Carver {
    char* base;
    size_t off = 0;
    explicit Carver(void* p) : base(static_cast<char*>(p)) {}
    template <class T>
    T* take(size_t n) {
        off = align_up(off, 256);
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += n * sizeof(T);
        return p;
    }
};

// The tensor-core lane keeps only the chunk table and the per-row scalars here (its operand panels live in
// tc::TcWs); the large float32 arrays are carved with zero length for it.
inline Ws carve_ws(const KdaChunkShape& sh, void* mem, size_t* bytes = nullptr) {
    Ws w;
    const size_t big = sh.lane == KDA_LANE_TC ? 0 : 1;
    w.H = sh.heads; w.K = sh.key_dim; w.V = sh.value_dim;
    w.Kp = ceil_div(sh.key_dim, 64) * 64;
    w.Vp = ceil_div(sh.value_dim, 64) * 64;
    w.nslots = slots_for(sh, false);
    const size_t nch = (size_t)w.nslots * w.H;
    Carver c(mem);
    w.chunk_seq = c.take<int>(w.nslots + 1);
    w.chunk_tok0 = c.take<int>(w.nslots + 1);
    w.chunk_len = c.take<int>(w.nslots + 1);
    w.seq_chunk0 = c.take<int>(sh.n_seq + 1);
    w.seq_order = c.take<int>(sh.n_seq);
    w.qn = c.take<float>(big * nch * 64 * w.Kp);
    w.kn = c.take<float>(big * nch * 64 * w.Kp);
    w.G = c.take<float>(big * nch * 64 * w.Kp);
    w.W = c.take<float>(big * nch * 64 * w.Kp);
    w.Z = c.take<float>(big * nch * 64 * w.Vp);
    w.A = c.take<float>(big * nch * 4096);
    w.T = c.take<float>(big * nch * 4096);
    w.Hc = c.take<float>(big * nch * w.Kp * w.Vp);
    w.qinv = c.take<float>(nch * 64);
    w.kinv = c.take<float>(nch * 64);
    w.beta = c.take<float>(nch * 64);
    w.status = c.take<int>(64);
    if (bytes) *bytes = align_up(c.off, 256);
    return w;
}

inline Scr carve_scr(const KdaChunkShape& sh, void* mem, size_t* bytes = nullptr) {
    Scr s;
    const int Kp = ceil_div(sh.key_dim, 64) * 64, Vp = ceil_div(sh.value_dim, 64) * 64;
    const size_t nch = sh.lane == KDA_LANE_TC ? 0 : (size_t)slots_for(sh, false) * sh.heads;   // float32 lane only
    Carver c(mem);
    s.dZ = c.take<float>(nch * 64 * Vp);
    s.dHn = c.take<float>(nch * Kp * Vp);
    s.dqn = c.take<float>(nch * 64 * Kp);
    s.dkn = c.take<float>(nch * 64 * Kp);
    s.dG = c.take<float>(nch * 64 * Kp);
    s.dA = c.take<float>(nch * 4096);
    s.dM = c.take<float>(nch * 4096);
    s.dGend = c.take<float>(nch * Kp);
    s.dbl = c.take<float>(nch * 64);
    s.dbp = c.take<float>(nch * (Kp / 64) * 64);
    if (bytes) *bytes = align_up(c.off, 256);
    return s;
}

}  // namespace simt
}  // namespace kda
