// Tensor-core lane (K = V = 128): the state recurrences as affine scans.
//
// With Z = U - W H substituted, one chunk maps its incoming state H to
//     H' = exp(G_end) . H  -  (W^T E)^T-contracted H  +  E^T U          i.e.  H'^T = dec . H^T - H^T Pn + U^T E
// and the adjoint recurrence of the backward is its transpose,
//     dH^T = dec . dH'^T - dH'^T Pn^T + dO^T (R - A W).
// Pn = W^T E and Rm = R - A W do not depend on the state, so they are computed for all chunks in parallel
// (at the end of the intra-chunk forward kernel) and the sequential part of a chunk step shrinks to ONE UMMA chain between two register passes:
//     pack state -> bf16 A operand | D = state-independent term (issued a step early) - state x Pn | state = dec . state + D
// Everything else that used to sit inside the scans runs chunk-parallel on all SMs afterwards:
//     forward   Z^T = U^T - (W H)^T,  O^T = (R H)^T + (A Z)^T      from the chunk-start states the scan stored
//     backward  dZ^T = dO^T A + dH'^T E^T                          from the state adjoints the scan stored
// All products are written transposed so that M = 128 (value index = TMEM lane) for every UMMA.
// Restates reference chunk_wy_forward.cu:940-1275 (state scan), 1498-1588 (output) and
// chunk_wy_backward.cu:2445-2562 (adjoint scan); the algebraic regrouping is this implementation's.

#include "common.cuh"
#include "simt_ws.cuh"
#include "tc_common.cuh"
#include "tc_ws.cuh"

namespace kda {
namespace tc {

int make_map_bf16(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows);

// ---------------------------------------------------------------------------------------------
// affine scan: one CTA per (sequence, head) walks the chunks in order (forward) or in reverse (backward)
//     forward    S = H^T   [v][k]:   S' = dec . S - S Pn   + U^T E           stores S (chunk-start state) per chunk
//     backward   S = dH'^T [v][k]:   S' = dec . S - S Pn^T + dO^T Rm         stores S (adjoint of the chunk's outgoing state)
// Threads are specialised by warp; they meet only through mbarriers:
//   state warpgroups (kScanGroups of them): thread (g, v) owns S[v][g*kScanCols .. (g+1)*kScanCols) in registers
//   next warp   one lane issues the TMA loads, two chunks ahead
//   last warp   one lane issues every UMMA and the TMA stores of the state panels
// TMEM: the accumulator is double-buffered (columns 0 / 128) so that the state-independent product of step c+1 is
// issued while the state threads still read the accumulator of step c; the bf16 state panel the state product reads as
// its A operand sits at column 256.  Its shared-memory copy (for the TMA store) is double-buffered, so the store of
// panel c has a whole step to read it before it is written again.
// ---------------------------------------------------------------------------------------------
struct AffineScanArgs {
    const int* seq_chunk0;
    const int* seq_order;     // unsplit scans: grid = (heads, sequences), block (h, r) walks sequence seq_order[r]
    const int* chunk_tok0;
    const int* chunk_len;
    const float* decay_end;   // [nch][128] exp(G_end)
    const float* s_in;        // V-first initial state (forward: h0, backward: cotangent of the final state), or null
    float* s_out;             // V-first final state of the scan (forward: final state, backward: dh0), or null
    int H;
    int* status;
    // Split scans (few long sequences: most SMs would idle behind a handful of 64-step chains).  The steps of every
    // (sequence, head) are cut into nseg segments that run side by side as 2 nseg - 1 units: unit 0 walks segment 0 from
    // s_in; for every later segment k, unit 2k-1 walks it from a zero state (its "local" states L) and unit 2k walks its
    // state-to-state map alone, from the identity and without the state-independent term (the composites P of the
    // affine maps).  The true state at a chunk of segment k is S_k P + L with S_k the state at the segment's start;
    // tc_scan_fixup_kernel forms the S_k (a chain of nseg - 1 small products) and then the chunk states, chunk-parallel.
    // Units leave their final state as float32 (seg_fin) and as a bf16 panel (through mF).
    int nseg;                 // 1: no split
    float* seg_fin;           // [n_seq*H*(2 nseg - 1)][128][128]
};

// first scan step of segment k of a sequence of n steps
__host__ __device__ __forceinline__ int seg_begin(int k, int nseg, int n) { return (int)(((long long)k * n) / nseg); }

constexpr int kPStage = 65536;                              // Pn 32 KB | X 16 KB (U^T or Rm^T) | Y 16 KB (E or dO)
constexpr int kPStageBytes = kPStage + 512;                 // + exp(G_end), which lands in a ring of its own
constexpr int kAffineScanSmem = 2 * kPStage + 2 * 32768 + 1024;
constexpr int kScanGroups = 2;                              // state warpgroups: each thread owns 128 / kScanGroups columns of a row
constexpr int kScanCols = 128 / kScanGroups;
constexpr uint32_t kScanPanelCol = 256;                     // TMEM column of the bf16 state panel (64 columns: 128 keys as pairs)
constexpr int kAffineScanThreads = (4 * kScanGroups + 2) * 32;

template <bool kBwd>
__global__ void __launch_bounds__(kAffineScanThreads, 1)
    tc_affine_scan_kernel(const __grid_constant__ CUtensorMap mP, const __grid_constant__ CUtensorMap mX,
                          const __grid_constant__ CUtensorMap mY, const __grid_constant__ CUtensorMap mS,
                          const __grid_constant__ CUtensorMap mS2, const __grid_constant__ CUtensorMap mF, AffineScanArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
    uint8_t* Sop = sm + 2 * kPStage;               // 2 x [2 k-blocks][128 rows x 128 B]: bf16 state panel of step c in c % 2
    __shared__ __align__(16) float dec_ring[4][128];   // exp(G_end) of step c in slot c % 4
    // full: a stage has landed.  free: every product that reads a stage is complete (one per stage, so that the load
    // thread can never miss a phase).  sop: all state threads have packed the state panel.  mma: the step's
    // accumulator is complete.
    __shared__ uint64_t bar_full[2], bar_free[2], bar_sop, bar_pan, bar_mma;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int v = (warp & 3) * 32 + lane;          // value row = TMEM lane
    const bool split = p.nseg > 1;
    const int units = 2 * p.nseg - 1;
    // split: grid (sequences x units, heads); unsplit with an order table: grid (heads, sequences), longest first, so that
    // the blocks the hardware starts first are the longest chains
    const bool lpt = !split && p.seq_order != nullptr;
    const int seq = split ? blockIdx.x / units : (lpt ? p.seq_order[blockIdx.y] : blockIdx.x), role = split ? blockIdx.x % units : 0;
    const int h = lpt ? blockIdx.x : blockIdx.y, H = p.H;
    const int c_begin = p.seq_chunk0[seq], c_end = p.seq_chunk0[seq + 1];
    const int n_total = c_end - c_begin;
    const int seg = (role + 1) >> 1;                             // segment this unit walks
    const int step0 = seg_begin(seg, p.nseg, n_total);           // its first step, in the sequence's scan order
    const int n = seg_begin(seg + 1, p.nseg, n_total) - step0;
    const bool composite = role > 0 && (role & 1) == 0;          // state-to-state map only: no state-independent term
    const int unit = (seq * H + h) * units + role;
    auto slot_of = [&](int c) { return kBwd ? c_end - 1 - (step0 + c) : c_begin + step0 + c; };   // chunk slot of step c

    if (tid == 0) {
        mbar_init(&bar_full[0], 1);
        mbar_init(&bar_full[1], 1);
        mbar_init(&bar_free[0], 1);
        mbar_init(&bar_free[1], 1);
        mbar_init(&bar_sop, 4 * kScanGroups);      // one arrival per state warp
        mbar_init(&bar_pan, 4 * kScanGroups);
        mbar_init(&bar_mma, 1);
        mbar_fence_init();
        abort_flag = 0;
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

    if (warp == 4 * kScanGroups) {
        // ------------------------------------------------------------------ load warp
        if (lane == 0) {
            auto issue_loads = [&](int c) {
                const int st = c & 1;
                const int slot = slot_of(c);
                const int ch = slot * H + h;
                uint8_t* b = sm + st * kPStage;
                mbar_expect_tx(&bar_full[st], composite ? 32768 + 512 : kPStageBytes);
                bulk_load_1d(dec_ring[c & 3], p.decay_end + (size_t)ch * 128, 512, &bar_full[st]);
                for (int nb = 0; nb < 2; ++nb) tma_load_2d(b + nb * 16384, &mP, &bar_full[st], nb * 64, ch * 128);
                if (composite) return;
                tma_load_2d(b + 32768, &mX, &bar_full[st], 0, ch * 128);                  // U^T / Rm^T: [128][64]
                if (!kBwd) {
                    for (int nb = 0; nb < 2; ++nb) tma_load_2d(b + 49152 + nb * 8192, &mY, &bar_full[st], nb * 64, ch * 64);
                } else {
                    const int tok0 = p.chunk_tok0[slot];
                    for (int nb = 0; nb < 2; ++nb) tma_load_2d(b + 49152 + nb * 8192, &mY, &bar_full[st], h * 128 + nb * 64, tok0);
                }
            };
            int issued = 0;
            for (; issued < 2 && issued < n; ++issued) issue_loads(issued);
            bool ok = true;
            for (int c = 0; c + 2 < n && ok; ++c) {     // stage c % 2 is free once every product of step c is complete
                ok = mbar_wait(&bar_free[c & 1], (c >> 1) & 1, p.status, 50);
                if (ok) { issue_loads(c + 2); issued = c + 3; }
                else abort_flag = 1;
            }
            if (!ok)   // unwinding: the copies in flight must land before the block may exit
                for (int c = issued > 2 ? issued - 2 : 0; c < issued; ++c) mbar_wait(&bar_full[c & 1], (c >> 1) & 1, nullptr, 0);
        }
    } else if (warp == 4 * kScanGroups + 1) {
        // ------------------------------------------------------------------ UMMA / panel-store thread
        if (kBwd && n > 0 && !composite && step0 == 0) {
            // Only a sequence's last chunk (the adjoint scan's first step) can be ragged; the dO rows past its tail
            // belong to the next sequence and are blanked by the whole warp before lane 0 issues the product on them.
            const int len0 = p.chunk_len[slot_of(0)];
            if (len0 < 64) {
                if (mbar_wait(&bar_full[0], 0, p.status, 51)) {
                    for (int idx = lane; idx < (64 - len0) * 16; idx += 32) {
                        const int r = len0 + (idx >> 4), c = idx & 15;
                        *reinterpret_cast<uint4*>(sm + 49152 + (c >> 3) * 8192 + sw128_off(r, c & 7)) = make_uint4(0, 0, 0, 0);
                    }
                    fence_async_smem();
                }
                __syncwarp();
            }
        }
        if (lane == 0 && n == 0 && split) {
            if (mbar_wait(&bar_pan, 0, p.status, 55)) {
                tma_store_2d(&mF, Sop, 0, unit * 128);
                tma_store_2d(&mF, Sop + 16384, 64, unit * 128);
                tma_store_commit();
            }
            tma_store_wait_all();
        }
        if (lane == 0 && n > 0) {
            // state-independent product:  forward U^T E (A K-major, B MN-major), backward dO^T Rm (A MN-major, B K-major)
            const uint32_t id_ind = kBwd ? umma_idesc_bf16(128, 128, kMajorMN, kMajorK) : umma_idesc_bf16(128, 128, kMajorK, kMajorMN);
            // state product, negated:  forward -S Pn (B MN-major: rows of Pn are the contraction index),
            //                          backward -S Pn^T (B K-major: rows of Pn are the output index)
            const uint32_t id_st = umma_idesc_bf16(128, 128, kMajorK, kBwd ? kMajorK : kMajorMN, 1);
            auto issue_independent = [&](int c) {
                const uint32_t s0 = smem_u32(sm + (c & 1) * kPStage);
                const uint32_t d = tmem + 128 * (c & 1);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16) {
                    if (!kBwd)
                        umma_bf16_ss(d, umma_smem_desc_sw128(s0 + 32768 + k16 * 32, 16, 1024),
                                     umma_smem_desc_sw128(s0 + 49152 + k16 * 2048, 8192, 1024), id_ind, k16 > 0);
                    else
                        umma_bf16_ss(d, umma_smem_desc_sw128(s0 + 49152 + k16 * 2048, 8192, 1024),
                                     umma_smem_desc_sw128(s0 + 32768 + k16 * 32, 16, 1024), id_ind, k16 > 0);
                }
            };
            const CUtensorMap* mstore = composite ? &mS2 : &mS;      // composites go to their own panel array
            bool ok = mbar_wait(&bar_full[0], 0, p.status, 51);
            if (ok) {
                tc_fence_after();
                if (!composite) issue_independent(0);
            } else abort_flag = 1;
            for (int c = 0; c < n && ok; ++c) {
                const int st = c & 1;
                const int ch = slot_of(c) * H + h;
                const uint32_t s0 = smem_u32(sm + st * kPStage);
                if (!mbar_wait(&bar_sop, c & 1, p.status, 52)) { abort_flag = 1; break; }
                tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < 8; ++k16) {   // A = the packed state in tensor memory, 8 columns per K = 16
                    const uint64_t bd = kBwd ? umma_smem_desc_sw128(s0 + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024)
                                             : umma_smem_desc_sw128(s0 + k16 * 2048, 16384, 1024);
                    umma_bf16_ts(tmem + 128 * st, tmem + kScanPanelCol + 8 * k16, bd, id_st, (composite && k16 == 0) ? 0u : 1u);
                }
                // The store of panel c-1 has read its buffer before this commit lets the state threads write panel c+1
                // into it.
                tma_store_wait_read();
                umma_commit(&bar_mma);
                umma_commit(&bar_free[st]);
                // the copy of the panel in shared memory (written after the tensor-memory one, off the critical path)
                if (!mbar_wait(&bar_pan, c & 1, p.status, 55)) { abort_flag = 1; break; }
                tma_store_2d(mstore, Sop + st * 32768, 0, ch * 128);
                tma_store_2d(mstore, Sop + st * 32768 + 16384, 64, ch * 128);
                tma_store_commit();
                if (c + 1 < n) {
                    // accumulator (c+1) % 2 was last read by the state threads in step c-1, before they packed panel c
                    if (!mbar_wait(&bar_full[(c + 1) & 1], ((c + 1) >> 1) & 1, p.status, 51)) { abort_flag = 1; break; }
                    tc_fence_after();
                    if (!composite) issue_independent(c + 1);
                }
            }
            if (ok && split && abort_flag == 0) {
                // the unit's final state as one more bf16 panel (the state threads pack it after their last step)
                if (mbar_wait(&bar_pan, n & 1, p.status, 55)) {
                    tma_store_2d(&mF, Sop + (n & 1) * 32768, 0, unit * 128);
                    tma_store_2d(&mF, Sop + (n & 1) * 32768 + 16384, 64, unit * 128);
                    tma_store_commit();
                }
            }
            tma_store_wait_all();
        }
    } else {
        // ------------------------------------------------------------------ state warpgroups
        const int col0 = (warp >> 2) * kScanCols;  // first key column of this thread
        float s[kScanCols];
        if (composite) {
#pragma unroll
            for (int j = 0; j < kScanCols; ++j) s[j] = (col0 + j == v) ? 1.f : 0.f;
        } else if (p.s_in && role == 0) {
            const float4* src = reinterpret_cast<const float4*>(p.s_in + (((size_t)seq * H + h) * 128 + v) * 128 + col0);
#pragma unroll
            for (int j = 0; j < kScanCols / 4; ++j) {
                float4 x = src[j];
                s[4 * j] = x.x; s[4 * j + 1] = x.y; s[4 * j + 2] = x.z; s[4 * j + 3] = x.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < kScanCols; ++j) s[j] = 0.f;
        }
        // This thread's half of the state row as bf16 pairs: first into tensor memory, where the state product reads its
        // A operand (lane = value row, 32 columns per key half), then - after the arrival that releases the UMMA
        // thread - into the shared-memory panel that the TMA store sends to the chunk-parallel kernels.
        static_assert(kScanCols == 64, "the tensor-memory panel is written with one 32-column store per thread");
        const int kh = col0 / 64;
        // The stage of step c is observed HERE, before the arrival that lets the UMMA thread run step c: the commit of
        // step c frees the stage for the loads of step c + 2, so a state warp that looked at the stage barrier only
        // after that commit could find it two phases on and read the parity as "not yet complete".
        auto pack_state = [&](int c) -> bool {
            const bool last = c >= n;      // the final state's panel: shared-memory copy only, nothing consumes it on chip
            if (!last && !mbar_wait(&bar_full[c & 1], (c >> 1) & 1, p.status, 54)) return false;
            uint32_t w[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = pack_bf16(s[2 * j], s[2 * j + 1]);
            if (!last) {
                tmem_st32(tmem + lane_base + kScanPanelCol + 32 * kh, w);
                tmem_st_wait();
                tc_fence_before();
                warp_arrive(&bar_sop, lane);
            }
            uint8_t* dst = Sop + (c & 1) * 32768 + kh * 16384;
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4*>(dst + sw128_off(v, q)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
            fence_async_smem();
            warp_arrive(&bar_pan, lane);
            return true;
        };
        bool ok = true;
        if ((n > 0 || split) && !pack_state(0)) { abort_flag = 1; ok = false; }
        for (int c = 0; c < n && ok; ++c) {
            if (!mbar_wait(&bar_mma, c & 1, p.status, 53)) {
                abort_flag = 1; ok = false;
                break;
            }
            tc_fence_after();
            const float* dc = dec_ring[c & 3] + col0;
            {
                uint32_t r[kScanCols / 32][32];    // every part in flight before the wait
#pragma unroll
                for (int b = 0; b < kScanCols / 32; ++b) tmem_ld32(tmem + lane_base + 128 * (c & 1) + col0 + 32 * b, r[b]);
                tmem_ld_wait();
#pragma unroll
                for (int b = 0; b < kScanCols / 32; ++b)
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        const float4 dv = *reinterpret_cast<const float4*>(dc + 32 * b + 4 * j4);
                        s[32 * b + 4 * j4 + 0] = dv.x * s[32 * b + 4 * j4 + 0] + __uint_as_float(r[b][4 * j4 + 0]);
                        s[32 * b + 4 * j4 + 1] = dv.y * s[32 * b + 4 * j4 + 1] + __uint_as_float(r[b][4 * j4 + 1]);
                        s[32 * b + 4 * j4 + 2] = dv.z * s[32 * b + 4 * j4 + 2] + __uint_as_float(r[b][4 * j4 + 2]);
                        s[32 * b + 4 * j4 + 3] = dv.w * s[32 * b + 4 * j4 + 3] + __uint_as_float(r[b][4 * j4 + 3]);
                    }
            }
            tc_fence_before();
            if ((c + 1 < n || split) && !pack_state(c + 1)) { abort_flag = 1; ok = false; }
        }
        float* fin = split ? p.seg_fin + (size_t)unit * 16384 : (p.s_out ? p.s_out + ((size_t)seq * H + h) * 16384 : nullptr);
        if (ok && abort_flag == 0 && fin) {
            // split units leave their final state thread-major (float4 j of state thread tid at [j][tid]: every warp
            // store is one contiguous 512-byte run, and the fix-up's threads own the same elements); the scan's final
            // state goes out in the caller's row-major layout
            float4* dst = split ? reinterpret_cast<float4*>(fin) + tid : reinterpret_cast<float4*>(fin + (size_t)v * 128 + col0);
            const int dstep = split ? 256 : 1;
#pragma unroll
            for (int j = 0; j < kScanCols / 4; ++j) dst[j * dstep] = make_float4(s[4 * j], s[4 * j + 1], s[4 * j + 2], s[4 * j + 3]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------
// split scans, second pass: from the units' local states to the true states (see tc_scan_fixup_kernel)
// ---------------------------------------------------------------------------------------------
struct ScanFixArgs {
    const int* seq_chunk0;
    const int* chunk_seq;
    const int* chunk_len;
    const float* seg_fin;      // [rec*units][128][128]
    __nv_bfloat16* Hp;         // [nch][128][128]: local states in, true states out
    float* s_out;              // final state of the scan, V-first [n_seq][H][128][128], or null
    int H, nseg, bwd, nslots;
    int* status;
};

constexpr int kFixSmem = 3 * 32768 + 1024;          // S hi | S lo | P

// D[tmem] = (A_hi + A_lo) B: A K-major [128 v][128 k] in two bf16 terms, B = P [k][n] MN-major
__device__ __forceinline__ void issue_hilo_product(uint32_t tmem, const uint8_t* a_hi, const uint8_t* b) {
    const uint32_t b0 = smem_u32(b);
    const uint32_t idesc = umma_idesc_bf16(128, 128, kMajorK, kMajorMN);
#pragma unroll
    for (int part = 0; part < 2; ++part) {
        const uint32_t a0 = smem_u32(a_hi + part * 32768);
#pragma unroll
        for (int k16 = 0; k16 < 8; ++k16)
            umma_bf16_ss(tmem, umma_smem_desc_sw128(a0 + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                         umma_smem_desc_sw128(b0 + k16 * 2048, 16384, 1024), idesc, (part | k16) != 0);
    }
}

// Chunk-parallel fix-up of a split scan, one CTA per chunk-head of segments 1 .. nseg-1 (2 CTAs per SM).  The true state
// at the start of segment k obeys S_1 = final state of segment 0, S_{j+1} = S_j Pfin_j + Lfin_j (final composite and final
// local state of segment j); every CTA of segment k walks that short chain itself (k - 1 products; the panels sit in L2
// and all CTAs run side by side, which costs less than a separate launch chaining them once on a handful of SMs), then
// adds S_k Pp_c to the local state the scan published for its chunk.  S is carried between products as a bf16 hi + lo
// pair in shared memory (the A operand), so the correction keeps float32-class accuracy.  When the caller wants the scan's
// final state, one more CTA per (sequence, head) walks the last segment's chain and applies that segment's final maps:
// the same number of products as a chunk of that segment, so it does not lengthen the launch.
// A thread owns one accumulator row (TMEM lane), so nothing it touches in global memory is addressed row-per-thread:
// the float32 states come thread-major (see the scan kernel), the chunk's bf16 panel comes and goes by TMA through the
// B-operand buffer, and the final state is transposed through shared memory.
__global__ void __launch_bounds__(256, 2)
    tc_scan_fixup_kernel(const __grid_constant__ CUtensorMap mPp, const __grid_constant__ CUtensorMap mF,
                         const __grid_constant__ CUtensorMap mHp, ScanFixArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
    __shared__ uint64_t bar_in, bar_mma;
    __shared__ uint32_t tmem_slot;
    const int h = blockIdx.y, H = p.H, units = 2 * p.nseg - 1;
    // blocks past the chunk slots (launched only when the caller wants the scan's final state) form that state, one per
    // sequence: the chain of the last segment plus one product, the same length as a chunk's work in that segment
    const bool fin = (int)blockIdx.x >= p.nslots;
    const int slot = fin ? 0 : blockIdx.x;
    if (!fin && p.chunk_len[slot] == 0) return;
    const int seq = fin ? (int)blockIdx.x - p.nslots : p.chunk_seq[slot];
    const int c_begin = p.seq_chunk0[seq], c_end = p.seq_chunk0[seq + 1];
    const int n_total = c_end - c_begin;         // 0 for an empty sequence: its final state is its initial state, which the
    int k = p.nseg - 1;                          // chain below reproduces (identity composites, zero local states)
    if (!fin) {
        const int step = p.bwd ? c_end - 1 - slot : slot - c_begin;
        while (k > 0 && step < seg_begin(k, p.nseg, n_total)) --k;
        if (k == 0) return;                         // segment 0 holds true states already
    }
    const int rec = seq * H + h;
    const int ch = slot * H + h;
    // products 0 .. k-2 walk the chain S_1 -> S_k; product k-1 is the chunk's own (S_k Pp_c) or, in a final-state block,
    // S_k Pfin_k
    const int nprod = k;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;                        // key half handled by this warpgroup
    const int v = (warp & 3) * 32 + lane;           // value row = TMEM lane;  tid == g * 128 + v
    uint8_t* Pbuf = sm + 65536;
    uint32_t inph = 0;                              // completed phases of bar_in (uniform)
    auto load_panel = [&](const CUtensorMap* map, int row) {
        mbar_expect_tx(&bar_in, 32768);
        for (int nb = 0; nb < 2; ++nb) tma_load_2d(Pbuf + nb * 16384, map, &bar_in, nb * 64, row);
    };
    auto load_p = [&](int t) {                      // B operand of product t
        if (t == k - 1 && !fin) load_panel(&mPp, ch * 128);
        else load_panel(&mF, (rec * units + 2 * (t + 1)) * 128);
    };
    if (tid == 0) {
        mbar_init(&bar_in, 1);
        mbar_init(&bar_mma, 1);
        mbar_fence_init();
        if (k == 1 && !fin) load_panel(&mHp, ch * 128);     // the first product is the chunk's own: its local state comes first
        else load_p(0);
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 128);
    auto split_store = [&](const float (&x)[32], int b) {      // 32 keys starting at 64 g + 32 b -> hi / lo operand panels
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 hh = __floats2bfloat162_rn(x[8 * c + 2 * e], x[8 * c + 2 * e + 1]);
                const float2 back = __bfloat1622float2(hh);
                hi[e] = *reinterpret_cast<const uint32_t*>(&hh);
                lo[e] = pack_bf16(x[8 * c + 2 * e] - back.x, x[8 * c + 2 * e + 1] - back.y);
            }
            *reinterpret_cast<uint4*>(sm + g * 16384 + sw128_off(v, 4 * b + c)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(sm + 32768 + g * 16384 + sw128_off(v, 4 * b + c)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
    };
    auto load_f32 = [&](const float* unit_base, float (&x)[32], int b) {     // thread-major float32 state of a scan unit
        const float4* src = reinterpret_cast<const float4*>(unit_base) + tid;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 a = src[(8 * b + c) * 256];
            x[4 * c] = a.x; x[4 * c + 1] = a.y; x[4 * c + 2] = a.z; x[4 * c + 3] = a.w;
        }
    };
    // S_1 = final state of segment 0
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        float x[32];
        load_f32(p.seg_fin + (size_t)rec * units * 16384, x, b);
        split_store(x, b);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    for (int t = 0; t < nprod && ok; ++t) {
        const bool own = t == k - 1 && !fin;
        const bool final_state = t == k - 1 && fin;
        float add[2][32];                           // what is added to the product
        if (own) {
            // the chunk's local state sits in the B-operand buffer (TMA): take this thread's row, then make room for P
            ok = mbar_wait(&bar_in, inph & 1, p.status, 82);
            ++inph;
            if (ok) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float l[8];
                    unpack_bf16x8(*reinterpret_cast<const uint4*>(Pbuf + g * 16384 + sw128_off(v, c)), l);
#pragma unroll
                    for (int e = 0; e < 8; ++e) add[c >> 2][8 * (c & 3) + e] = l[e];
                }
            }
            fence_async_smem();
            ok = __syncthreads_and(ok);
            if (ok && tid == 0) load_p(t);
        } else {
            // the final local state of the segment this chain step crosses (float32, thread-major): flies during the product
            const float* L = p.seg_fin + (size_t)(rec * units + 2 * (t + 1) - 1) * 16384;
            load_f32(L, add[0], 0);
            load_f32(L, add[1], 1);
        }
        if (tid == 0 && ok) {
            ok = mbar_wait(&bar_in, inph & 1, p.status, 80);
            if (ok) {
                tc_fence_after();
                issue_hilo_product(tmem, sm, Pbuf);
                umma_commit(&bar_mma);
            }
        }
        ++inph;
        if (ok) ok = mbar_wait(&bar_mma, (uint32_t)t & 1, p.status, 81);
        ok = __syncthreads_and(ok);                 // the product has read both operand buffers
        tc_fence_after();
        if (ok && tid == 0 && t + 1 < nprod) {      // next panel into the free buffer while this result is read out
            if (t + 1 == k - 1 && !fin) load_panel(&mHp, ch * 128);
            else load_p(t + 1);
        }
        if (ok) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_base + 64 * g + 32 * b, r);
                tmem_ld_wait();
                float x[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]) + add[b][j];
                if (own) {                          // the chunk's true state -> B-operand buffer -> TMA store; S_k stays put
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        *reinterpret_cast<uint4*>(Pbuf + g * 16384 + sw128_off(v, 4 * b + c)) =
                            make_uint4(pack_bf16(x[8 * c], x[8 * c + 1]), pack_bf16(x[8 * c + 2], x[8 * c + 3]),
                                       pack_bf16(x[8 * c + 4], x[8 * c + 5]), pack_bf16(x[8 * c + 6], x[8 * c + 7]));
                } else if (final_state) {
                    // the scan's final state, row-major for the caller: rows through the dead operand panels (16-byte
                    // pieces XOR-swizzled by row so that the stores spread over the banks), written out below
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *reinterpret_cast<float4*>(sm + v * 512 + (((16 * g + 8 * b + c) ^ (v & 7)) << 4)) =
                            make_float4(x[4 * c], x[4 * c + 1], x[4 * c + 2], x[4 * c + 3]);
                } else {
                    split_store(x, b);              // S_{t+2}: the next product's A operand
                }
            }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();                            // operand panels rewritten, accumulator read: next product may go
        tc_fence_after();
        if (ok && own && tid == 0) {
            for (int nb = 0; nb < 2; ++nb) tma_store_2d(&mHp, Pbuf + nb * 16384, nb * 64, ch * 128);
            tma_store_commit();
        }
        if (ok && final_state) {
            float4* dst = reinterpret_cast<float4*>(p.s_out + (size_t)rec * 16384);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int f = i * 256 + tid, row = f >> 5, c16 = f & 31;       // float4 f of the row-major 128 x 128 tile
                dst[f] = *reinterpret_cast<const float4*>(sm + row * 512 + ((c16 ^ (row & 7)) << 4));
            }
        }
    }
    if (tid == 0) tma_store_wait_read();            // shared memory must outlive the reads of the bulk store
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 128);
}

// ---------------------------------------------------------------------------------------------
// chunk output (forward), one CTA per chunk-head, from the chunk-start state the scan stored:
//     [ (W H)^T | (R H)^T ] = H^T [ W^T | R^T ]      M=128, N=128, K=128
//     Z^T = U^T - (W H)^T                             registers -> bf16 panel (kept for the backward) and A operand
//     (A Z)^T = Z^T A^T                               M=128, N=64,  K=64
//     O^T = (R H)^T + (A Z)^T                         transposed through shared memory into o[token][head][value]
// 256 threads: thread (g, v) handles value row v, tokens 32g .. 32g+31.
// ---------------------------------------------------------------------------------------------
struct ChunkOutArgs {
    const int* chunk_tok0;
    const int* chunk_len;
    __nv_bfloat16* ZT;
    __nv_bfloat16* o;          // [tokens][H][128]
    int H;
    int* status;
    NormEpilogue norm;
};

// Z^T reuses the [W^T|R^T] tile and the output tile reuses the state tile: both are dead once the first UMMA chain has
// completed, and the smaller footprint lets two CTAs share an SM.
constexpr int kOutH = 0, kOutWR = 32768, kOutU = 65536, kOutA = 81920, kOutZ = kOutWR, kOutO = kOutH, kOutG = 90112;
constexpr int kChunkOutSmem = kOutA + 8192 + 1024;
constexpr int kChunkOutNormSmem = kOutG + 16384 + 1024;      // + the norm gate's tile when the epilogue is on

__global__ void __launch_bounds__(256, 2)
    tc_chunk_out_kernel(const __grid_constant__ CUtensorMap mH, const __grid_constant__ CUtensorMap mW,
                        const __grid_constant__ CUtensorMap mR, const __grid_constant__ CUtensorMap mUT,
                        const __grid_constant__ CUtensorMap mAT, const __grid_constant__ CUtensorMap mG,
                        const __grid_constant__ CUtensorMap mZT, ChunkOutArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
    uint8_t* Zop = sm + kOutZ;                     // [128 rows x 128 B] K-major A operand
    __nv_bfloat16* Ot = reinterpret_cast<__nv_bfloat16*>(sm + kOutO);   // [64 tokens][128 values]
    __shared__ uint64_t bar_in, bar_mma1, bar_mma2;
    __shared__ uint32_t tmem_slot;
    const int slot = blockIdx.x, h = blockIdx.y, H = p.H;
    const int len = p.chunk_len[slot];
    if (len == 0) return;
    const int tok0 = p.chunk_tok0[slot];
    const int ch = slot * H + h;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;
    const int v = (warp & 3) * 32 + lane;
    if (tid == 0) {
        mbar_init(&bar_in, 1);
        mbar_init(&bar_mma1, 1);
        mbar_init(&bar_mma2, 1);
        mbar_fence_init();
        mbar_expect_tx(&bar_in, 32768 + 32768 + 16384 + 8192 + (p.norm.gate != nullptr ? 16384 : 0));
        if (p.norm.gate != nullptr)      // the norm gate's tile, needed last: its latency hides under the products
            for (int kb = 0; kb < 2; ++kb) tma_load_2d(sm + kOutG + kb * 8192, &mG, &bar_in, h * 128 + kb * 64, tok0);
        for (int kb = 0; kb < 2; ++kb) tma_load_2d(sm + kOutH + kb * 16384, &mH, &bar_in, kb * 64, ch * 128);
        tma_load_2d(sm + kOutWR, &mW, &bar_in, 0, ch * 128);
        tma_load_2d(sm + kOutWR + 16384, &mR, &bar_in, 0, ch * 128);
        tma_load_2d(sm + kOutU, &mUT, &bar_in, 0, ch * 128);
        tma_load_2d(sm + kOutA, &mAT, &bar_in, 0, ch * 64);
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    if (tid == 0) {
        ok = mbar_wait(&bar_in, 0, p.status, 60);
        if (ok) {
            tc_fence_after();
            const uint32_t a0 = smem_u32(sm + kOutH), b0 = smem_u32(sm + kOutWR);
            const uint32_t idesc = umma_idesc_bf16(128, 128, kMajorK, kMajorMN);
#pragma unroll
            for (int k16 = 0; k16 < 8; ++k16)
                umma_bf16_ss(tmem, umma_smem_desc_sw128(a0 + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                             umma_smem_desc_sw128(b0 + k16 * 2048, 16384, 1024), idesc, k16 > 0);
            umma_commit(&bar_mma1);
        }
    }
    ok = mbar_wait(&bar_mma1, 0, p.status, 61) && ok;
    // the U^T tile was written by TMA: every reader observes the barrier it completed on
    ok = mbar_wait(&bar_in, 0, p.status, 60) && ok;
    tc_fence_after();
    {   // Z^T for tokens 32g .. 32g+31 of row v
        const uint8_t* UTs = sm + kOutU;
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + 32 * g, r);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const int c16 = g * 4 + q4;
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
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok) {
        if (p.ZT != nullptr) {                      // kept for the backward only: the operand tile is the panel, as TMA lays it out
            tma_store_2d(&mZT, Zop, 0, ch * 128);
            tma_store_commit();
        }
        tc_fence_after();
        const uint32_t a0 = smem_u32(Zop), b0 = smem_u32(sm + kOutA);
        const uint32_t idesc = umma_idesc_bf16(128, 64, kMajorK, kMajorMN);
#pragma unroll
        for (int k16 = 0; k16 < 4; ++k16)
            umma_bf16_ss(tmem + 128, umma_smem_desc_sw128(a0 + k16 * 32, 16, 1024),
                         umma_smem_desc_sw128(b0 + k16 * 2048, 8192, 1024), idesc, k16 > 0);
        umma_commit(&bar_mma2);
    }
    if (ok) ok = mbar_wait(&bar_mma2, 0, p.status, 62);
    tc_fence_after();
    if (ok) {
        uint32_t r1[32], r2[32];
        tmem_ld32(tmem + lane_base + 64 + 32 * g, r1);
        tmem_ld32(tmem + lane_base + 128 + 32 * g, r2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) Ot[(32 * g + j) * 128 + v] = __float2bfloat16(__uint_as_float(r1[j]) + __uint_as_float(r2[j]));
    }
    ok = __syncthreads_and(ok);
    if (ok && p.norm.gate == nullptr) {
        // 64 token rows of 256 bytes: 16 threads per row, 16 rows per pass
        const int c = tid & 15;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int i = pass * 16 + (tid >> 4);
            if (i < len)
                *reinterpret_cast<uint4*>(p.o + ((size_t)(tok0 + i) * H + h) * 128 + 8 * c) =
                    *reinterpret_cast<const uint4*>(Ot + i * 128 + 8 * c);
        }
    } else if (ok) {
        // Gated RMSNorm on the tile: a warp per token row, lane = 4 adjacent values - the decomposition (per-lane sum of
        // four squares, xor-shuffle tree, one rsqrt) of the stand-alone norm kernel, so both give the same bits.
        const float4 ww = *reinterpret_cast<const float4*>(p.norm.weight + 4 * lane);
        const float wa[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
        for (int pass = 0; pass < 8; ++pass) {
            const int i = pass * 8 + warp;
            const size_t row = (size_t)(tok0 + min(i, len - 1)) * H + h;
            const uint2 ou = *reinterpret_cast<const uint2*>(Ot + i * 128 + 4 * lane);
            const uint2 gu = *reinterpret_cast<const uint2*>(sm + kOutG + (lane >> 4) * 8192 + sw128_off(i, (lane >> 1) & 7) + (lane & 1) * 8);
            const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&ou);
            const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gu);
            const float2 o01 = __bfloat1622float2(oh[0]), o23 = __bfloat1622float2(oh[1]);
            const float2 g01 = __bfloat1622float2(gh[0]), g23 = __bfloat1622float2(gh[1]);
            const float a[4] = {o01.x, o01.y, o23.x, o23.y}, gt[4] = {g01.x, g01.y, g23.x, g23.y};
            float ss = a[0] * a[0] + a[1] * a[1] + a[2] * a[2] + a[3] * a[3];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            if (i < len) {
                const float inv = rsqrtf(ss * (1.0f / 128.0f) + p.norm.eps);
                if (lane == 0) p.norm.inv_rms[row] = inv;
                float out[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float th;
                    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * gt[e]));
                    out[e] = a[e] * inv * wa[e] * fmaf(0.5f, th, 0.5f);
                }
                *reinterpret_cast<uint2*>(p.o + row * 128 + 4 * lane) = ou;
                *reinterpret_cast<uint2*>(p.norm.y + row * 128 + 4 * lane) =
                    make_uint2(pack_bf16(out[0], out[1]), pack_bf16(out[2], out[3]));
            }
        }
    }
    if (tid == 0) tma_store_wait_read();            // the Z^T tile must outlive the reads of its bulk store
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------
// dZ (backward), one CTA per chunk-head, from the state adjoint the scan stored:
//     dZ^T = dO^T A + dH'^T E^T          M=128, N=64: K=64 (MN-major A) then K=128
// ---------------------------------------------------------------------------------------------
struct ChunkDzArgs {
    const int* chunk_tok0;
    const int* chunk_len;
    __nv_bfloat16* dZT;
    int H;
    int* status;
};

constexpr int kDzH = 0, kDzE = 32768, kDzO = 49152, kDzA = 65536;
constexpr int kChunkDzSmem = kDzA + 8192 + 1024;

__global__ void __launch_bounds__(256, 3)
    tc_chunk_dz_kernel(const __grid_constant__ CUtensorMap mdH, const __grid_constant__ CUtensorMap mE,
                       const __grid_constant__ CUtensorMap mdO, const __grid_constant__ CUtensorMap mAT,
                       const __grid_constant__ CUtensorMap mdZT, ChunkDzArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
    __shared__ uint64_t bar_in, bar_mma;
    __shared__ uint32_t tmem_slot;
    const int slot = blockIdx.x, h = blockIdx.y, H = p.H;
    const int len = p.chunk_len[slot];
    if (len == 0) return;
    const int tok0 = p.chunk_tok0[slot];
    const int ch = slot * H + h;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = warp >> 2;
    const int v = (warp & 3) * 32 + lane;
    if (tid == 0) {
        mbar_init(&bar_in, 1);
        mbar_init(&bar_mma, 1);
        mbar_fence_init();
        mbar_expect_tx(&bar_in, 32768 + 16384 + 16384 + 8192);
        for (int kb = 0; kb < 2; ++kb) {
            tma_load_2d(sm + kDzH + kb * 16384, &mdH, &bar_in, kb * 64, ch * 128);
            tma_load_2d(sm + kDzE + kb * 8192, &mE, &bar_in, kb * 64, ch * 64);
            tma_load_2d(sm + kDzO + kb * 8192, &mdO, &bar_in, h * 128 + kb * 64, tok0);
        }
        tma_load_2d(sm + kDzA, &mAT, &bar_in, 0, ch * 64);
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 64);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    if (len < 64) {
        // ragged tail: the dO rows past it belong to the next sequence; blank them before they feed the UMMA
        ok = mbar_wait(&bar_in, 0, p.status, 70);
        if (ok) {
            for (int idx = tid; idx < (64 - len) * 16; idx += 256) {
                const int r = len + (idx >> 4), c = idx & 15;
                *reinterpret_cast<uint4*>(sm + kDzO + (c >> 3) * 8192 + sw128_off(r, c & 7)) = make_uint4(0, 0, 0, 0);
            }
            fence_async_smem();
        }
        ok = __syncthreads_and(ok);
    }
    if (tid == 0 && ok) {
        ok = mbar_wait(&bar_in, 0, p.status, 70);
        if (ok) {
            tc_fence_after();
            const uint32_t s0 = smem_u32(sm);
            const uint32_t ida = umma_idesc_bf16(128, 64, kMajorMN, kMajorK);
            const uint32_t idb = umma_idesc_bf16(128, 64, kMajorK, kMajorK);
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16)     // dO^T A
                umma_bf16_ss(tmem, umma_smem_desc_sw128(s0 + kDzO + k16 * 2048, 8192, 1024),
                             umma_smem_desc_sw128(s0 + kDzA + k16 * 32, 16, 1024), ida, k16 > 0);
#pragma unroll
            for (int k16 = 0; k16 < 8; ++k16)     // + dH'^T E^T
                umma_bf16_ss(tmem, umma_smem_desc_sw128(s0 + kDzH + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                             umma_smem_desc_sw128(s0 + kDzE + (k16 >> 2) * 8192 + (k16 & 3) * 32, 16, 1024), idb, 1);
            umma_commit(&bar_mma);
        }
    }
    ok = mbar_wait(&bar_mma, 0, p.status, 71) && ok;
    ok = __syncthreads_and(ok);
    tc_fence_after();
    if (ok) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + 32 * g, r);
        tmem_ld_wait();
        // the panel leaves through the dead dH' tile in the swizzled layout and one TMA store: a thread owns a row, and
        // row-per-thread global stores would touch 32 sectors per warp instruction
#pragma unroll
        for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(sm + kDzH + sw128_off(v, 4 * g + c)) =
                make_uint4(pack_bf16(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                           pack_bf16(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                           pack_bf16(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                           pack_bf16(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (tid == 0 && ok) {
        tma_store_2d(&mdZT, sm + kDzH, 0, ch * 128);
        tma_store_commit();
        tma_store_wait_read();
    }
    if (warp == 1) tmem_dealloc(tmem, 64);
}

}  // namespace tc

// ---------------------------------------------------------------------------------------------
// host entries used by the chunk forward / backward when the tensor-core lane is selected
// ---------------------------------------------------------------------------------------------
// split scans: segment-start states (and the scan's final state), then the chunk states of segments >= 1
static int scan_fixup(const simt::Ws& w, const tc::TcWs& t, int n_seq, __nv_bfloat16* panels, float* s_out, int bwd,
                      const CUtensorMap& mPp, const CUtensorMap& mF, cudaStream_t st) {
    using namespace tc;
    if (cudaFuncSetAttribute(tc_scan_fixup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFixSmem) != cudaSuccess)
        return KDA_ERR_CUDA;
    ScanFixArgs f;
    f.seq_chunk0 = w.seq_chunk0; f.chunk_seq = w.chunk_seq; f.chunk_len = w.chunk_len; f.seg_fin = t.seg_fin;
    f.Hp = panels; f.s_out = s_out; f.H = w.H; f.nseg = t.nseg; f.bwd = bwd; f.nslots = w.nslots; f.status = t.status;
    CUtensorMap mHp;
    if (make_map_bf16(&mHp, panels, (uint64_t)w.nslots * w.H * 128, 128, 64, 128)) return KDA_ERR_CUDA;
    KDA_LAUNCH("tc_scan_fixup_kernel", st, tc_scan_fixup_kernel<<<dim3(w.nslots + (s_out != nullptr ? n_seq : 0), w.H), 256, kFixSmem, st>>>(mPp, mF, mHp, f));
    return launch_status();
}

int tc_scan_forward(const simt::Ws& w, const tc::TcWs& t, int n_seq, int tokens, const float* h0, float* final_state, void* o,
                    const tc::NormEpilogue& norm, cudaStream_t st) {
    using namespace tc;
    const uint64_t nch = (uint64_t)w.nslots * w.H;
    CUtensorMap mW, mR, mE, mAT, mUT, mH, mP, mG, mZT;
    int rc = 0;
    rc |= make_map_bf16(&mW, t.WT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mR, t.RT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mE, t.E, nch * 64, 128, 64, 64);
    rc |= make_map_bf16(&mAT, t.AT, nch * 64, 64, 64, 64);
    rc |= make_map_bf16(&mUT, t.UT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mH, t.Hp, nch * 128, 128, 64, 128);
    rc |= make_map_bf16(&mP, t.Pn, nch * 128, 128, 64, 128);
    rc |= make_map_bf16(&mZT, t.fwd_only ? t.UT : t.ZT, nch * 128, 64, 64, 128);      // not stored in a forward-only call
    const bool fused_norm = norm.gate != nullptr;
    if (fused_norm) rc |= make_map_bf16(&mG, norm.gate, (uint64_t)tokens, (uint64_t)w.H * 128, 64, 64);
    else mG = mAT;
    if (rc) return KDA_ERR_CUDA;
    const int out_smem = fused_norm ? kChunkOutNormSmem : kChunkOutSmem;
    if (cudaFuncSetAttribute(tc_affine_scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAffineScanSmem) != cudaSuccess ||
        cudaFuncSetAttribute(tc_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kChunkOutNormSmem) != cudaSuccess)
        return KDA_ERR_CUDA;
    AffineScanArgs a;
    a.seq_chunk0 = w.seq_chunk0; a.chunk_tok0 = w.chunk_tok0; a.chunk_len = w.chunk_len; a.decay_end = t.decay_end; a.s_in = h0; a.s_out = final_state;
    a.H = w.H; a.status = t.status; a.nseg = t.nseg; a.seg_fin = t.seg_fin;
    const int units = 2 * t.nseg - 1;
    const bool lpt = t.nseg == 1 && n_seq > 1 && n_seq <= 65535;
    a.seq_order = lpt ? w.seq_order : nullptr;
    const dim3 scan_grid = lpt ? dim3(w.H, n_seq) : dim3(n_seq * units, w.H);
    CUtensorMap mPp = mH, mF = mH;
    if (t.nseg > 1) {
        if (make_map_bf16(&mPp, t.Pp, nch * 128, 128, 64, 128) ||
            make_map_bf16(&mF, t.fin_panel, (uint64_t)n_seq * w.H * units * 128, 128, 64, 128))
            return KDA_ERR_CUDA;
    }
    KDA_LAUNCH("tc_affine_scan_fwd_kernel", st,
               tc_affine_scan_kernel<false><<<scan_grid, kAffineScanThreads, kAffineScanSmem, st>>>(mP, mUT, mE, mH, mPp, mF, a));
    if (int e = launch_status()) return e;
    if (t.nseg > 1) {
        if (int e = scan_fixup(w, t, n_seq, t.Hp, final_state, 0, mPp, mF, st)) return e;
    }
    ChunkOutArgs oa;
    oa.chunk_tok0 = w.chunk_tok0; oa.chunk_len = w.chunk_len; oa.ZT = t.fwd_only ? nullptr : t.ZT; oa.o = static_cast<__nv_bfloat16*>(o); oa.H = w.H;
    oa.status = t.status;
    oa.norm = norm;
    KDA_LAUNCH("tc_chunk_out_kernel", st,
               tc_chunk_out_kernel<<<dim3(w.nslots, w.H), 256, out_smem, st>>>(mH, mW, mR, mUT, mAT, mG, mZT, oa));
    return launch_status();
}

int tc_scan_backward(const simt::Ws& w, const simt::Scr& s, const tc::TcWs& t, int n_seq, int tokens, const void* d_o,
                     const float* d_final, float* dh0, cudaStream_t st) {
    using namespace tc;
    (void)s;
    const uint64_t nch = (uint64_t)w.nslots * w.H;
    CUtensorMap mE, mAT, mdO, mdH, mP, mRm, mdZT;
    int rc = 0;
    rc |= make_map_bf16(&mE, t.E, nch * 64, 128, 64, 64);
    rc |= make_map_bf16(&mAT, t.AT, nch * 64, 64, 64, 64);
    rc |= make_map_bf16(&mdO, d_o, (uint64_t)tokens, (uint64_t)w.H * 128, 64, 64);
    rc |= make_map_bf16(&mdH, t.dHp, nch * 128, 128, 64, 128);
    rc |= make_map_bf16(&mP, t.Pn, nch * 128, 128, 64, 128);
    rc |= make_map_bf16(&mRm, t.RmT, nch * 128, 64, 64, 128);
    rc |= make_map_bf16(&mdZT, t.dZT, nch * 128, 64, 64, 128);
    if (rc) return KDA_ERR_CUDA;
    if (cudaFuncSetAttribute(tc_affine_scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAffineScanSmem) != cudaSuccess ||
        cudaFuncSetAttribute(tc_chunk_dz_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kChunkDzSmem) != cudaSuccess)
        return KDA_ERR_CUDA;
    AffineScanArgs a;
    a.seq_chunk0 = w.seq_chunk0; a.chunk_tok0 = w.chunk_tok0; a.chunk_len = w.chunk_len; a.decay_end = t.decay_end; a.s_in = d_final; a.s_out = dh0;
    a.H = w.H; a.status = t.status; a.nseg = t.nseg; a.seg_fin = t.seg_fin;
    const int units = 2 * t.nseg - 1;
    const bool lpt = t.nseg == 1 && n_seq > 1 && n_seq <= 65535;
    a.seq_order = lpt ? w.seq_order : nullptr;
    const dim3 scan_grid = lpt ? dim3(w.H, n_seq) : dim3(n_seq * units, w.H);
    CUtensorMap mPp = mdH, mF = mdH;
    if (t.nseg > 1) {
        if (make_map_bf16(&mPp, t.Pp, nch * 128, 128, 64, 128) ||
            make_map_bf16(&mF, t.fin_panel, (uint64_t)n_seq * w.H * units * 128, 128, 64, 128))
            return KDA_ERR_CUDA;
    }
    KDA_LAUNCH("tc_affine_scan_bwd_kernel", st,
               tc_affine_scan_kernel<true><<<scan_grid, kAffineScanThreads, kAffineScanSmem, st>>>(mP, mRm, mdO, mdH, mPp, mF, a));
    if (int e = launch_status()) return e;
    if (t.nseg > 1) {
        if (int e = scan_fixup(w, t, n_seq, t.dHp, dh0, 1, mPp, mF, st)) return e;
    }
    ChunkDzArgs da;
    da.chunk_tok0 = w.chunk_tok0; da.chunk_len = w.chunk_len; da.dZT = t.dZT; da.H = w.H; da.status = t.status;
    KDA_LAUNCH("tc_chunk_dz_kernel", st,
               tc_chunk_dz_kernel<<<dim3(w.nslots, w.H), 256, kChunkDzSmem, st>>>(mdH, mE, mdO, mAT, mdZT, da));
    return launch_status();
}

}  // namespace kda
