// Workspace of the tensor-core lane: bf16 operand panels per chunk-head (ch = slot*H + h), K = V = 128.
#pragma once

#include <cuda_bf16.h>

#include "simt_ws.cuh"

namespace kda {
namespace tc {

// Short causal convolution (width 4, SiLU) folded into the intra-chunk forward of a forward-only call: q, k, v of that
// call are the convolutions' INPUTS and the kernel forms the activations itself, so they are never written to memory.
struct ConvPrep {
    const void* w[3];       // weights of the q, k, v convolutions, [H*128][4]
    int wf32;               // 1: float32 weights (rounded to bf16 as loaded, like the stand-alone kernel), 0: bf16
};

struct TcWs {
    __nv_bfloat16 *WT, *RT;     // [nch][128][64]   rows = key, cols = token
    __nv_bfloat16* E;           // [nch][64][128]   rows = token, cols = key
    __nv_bfloat16* AT;          // [nch][64][64]    A transposed: [source s][target i]
    __nv_bfloat16* UT;          // [nch][128][64]   U transposed: [value][token]
    __nv_bfloat16* Tp;          // [nch][64][64]    T = (I + M)^-1, row-major
    __nv_bfloat16* Mt;          // [nch][64][64]    M before the beta scaling, strictly lower, row-major
    __nv_bfloat16* Hp;          // [nch][128][128]  chunk-start state, V-first [value][key]
    __nv_bfloat16* ZT;          // [nch][128][64]   Z transposed: [value][token]
    __nv_bfloat16* dHp;         // [nch][128][128]  adjoint of each chunk's outgoing state, V-first
    __nv_bfloat16* dZT;         // [nch][128][64]   dZ transposed
    __nv_bfloat16* Pn;          // [nch][128][128]  W^T E: [key k][key k'], the state-to-state part of the chunk transition
    __nv_bfloat16* RmT;         // [nch][128][64]   (R - A W)^T: [key][token]
    __nv_bfloat16* Pp;          // [nch][128][128]  split scans only: composite state-to-state maps at each chunk start
    __nv_bfloat16* fin_panel;   // [n_seq*H*units][128][128]  split scans only: final state of every scan unit as a bf16 panel
    float* seg_fin;             // [n_seq*H*units][128][128]  split scans only: the same in float32
    int nseg;                   // scan segments per (sequence, head): 1 (no split), 2 or 4; units = 2 * nseg - 1
    float* decay_end;           // [nch][128]       exp(G_end)
    int* status;                // device status word (0 = ok); points at the workspace's word (simt::Ws::status)
    int fwd_only;               // 1: the backward-only panels (T, M~, Z^T, dH', dZ^T, Rm^T) have no storage and are not written
};

// Optional epilogue of the chunk-output kernel: the gated RMSNorm that follows the operator in the layer
// (y = o * rsqrt(mean(o^2) + eps) * weight * sigmoid(gate) over the 128 values of a token and head), applied to the
// output tile while it is still on chip.  o is written as well: the norm's backward needs it.
struct NormEpilogue {
    const __nv_bfloat16* gate;   // [tokens][H][128], or nullptr: no epilogue
    const float* weight;         // [128]
    float eps;
    __nv_bfloat16* y;            // [tokens][H][128]
    float* inv_rms;              // [tokens][H]
};

// Scans are split when a batch has so few (sequence, head) recurrences that most SMs would idle behind them, and the
// sequences are long enough for a shorter chain to outweigh the fix-up pass.  The decision uses the shape alone (a packed
// batch is judged by its mean sequence length: the lengths themselves live on the device), so the forward and the
// backward of a call agree; every sequence of the batch is cut into the same number of segments, short ones into
// segments of one chunk or none.
inline int scan_segments(const KdaChunkShape& sh) {
    if (sh.n_seq <= 0) return 1;
    const bool fixed = sh.seq_len > 0 && (long long)sh.n_seq * sh.seq_len == sh.tokens;
    const long long rec = (long long)sh.n_seq * sh.heads;
    const long long chunks = fixed ? (sh.seq_len + 63) / 64 : (sh.tokens / 64) / sh.n_seq;
    if (rec * 7 <= 148 && chunks >= 32) return 4;
    if (rec * 3 <= 148 && chunks >= 16) return 2;
    return 1;
}

inline TcWs carve_tc(const KdaChunkShape& sh, void* mem, size_t* bytes = nullptr) {
    TcWs t;
    const size_t nch = (size_t)simt::slots_for(sh, false) * sh.heads;
    const size_t bw = sh.forward_only ? 0 : 1;      // panels only the backward reads
    simt::Carver c(mem);
    t.WT = c.take<__nv_bfloat16>(nch * 8192);
    t.RT = c.take<__nv_bfloat16>(nch * 8192);
    t.E = c.take<__nv_bfloat16>(nch * 8192);
    t.AT = c.take<__nv_bfloat16>(nch * 4096);
    t.UT = c.take<__nv_bfloat16>(nch * 8192);
    t.Tp = c.take<__nv_bfloat16>(bw * nch * 4096);
    t.Mt = c.take<__nv_bfloat16>(bw * nch * 4096);
    t.Hp = c.take<__nv_bfloat16>(nch * 16384);
    t.ZT = c.take<__nv_bfloat16>(bw * nch * 8192);
    t.dHp = c.take<__nv_bfloat16>(bw * nch * 16384);
    t.dZT = c.take<__nv_bfloat16>(bw * nch * 8192);
    t.Pn = c.take<__nv_bfloat16>(nch * 16384);
    t.RmT = c.take<__nv_bfloat16>(bw * nch * 8192);
    t.nseg = scan_segments(sh);
    const size_t units = t.nseg > 1 ? (size_t)sh.n_seq * sh.heads * (2 * t.nseg - 1) : 0;
    t.Pp = c.take<__nv_bfloat16>(t.nseg > 1 ? nch * 16384 : 0);
    t.fin_panel = c.take<__nv_bfloat16>(units * 16384);
    t.seg_fin = c.take<float>(units * 16384);
    t.decay_end = c.take<float>(nch * 128);
    t.status = c.take<int>(64);
    t.fwd_only = sh.forward_only ? 1 : 0;
    if (bytes) *bytes = align_up(c.off, 256);
    return t;
}

}  // namespace tc
}  // namespace kda
