/* C ABI of libkda_b200: Kimi Delta Attention (KDA) kernels for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a cudaStream_t
 * (passed as void*), launches on that stream, allocates nothing, never
 * synchronises the host and returns KDA_OK or a negative KDA_ERR_* code.
 * All tensors are dense and contiguous in the layouts named below.
 *
 * Each declaration names the reference interface it stands in for (paths are
 * relative to the reference project: vpareek2/experiment_swa_kda).
 *
 * Tensor layouts
 *   q, k, g, dq, dk, dg : [tokens, H, K]      v, o, dv, do : [tokens, H, V]
 *   beta, dbeta         : [tokens, H]
 *   memory state        : V-first [n_seq, H, V, K], always float32
 *   tokens = n_seq * seq_len for fixed-length batches, or the packed total when
 *   cu_seqlens (device int32 [n_seq + 1]) is given.
 */
#ifndef KDA_B200_H
#define KDA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KDA_OK 0
#define KDA_ERR_BAD_SHAPE (-1)     /* a dimension is zero/negative or above the supported maximum */
#define KDA_ERR_UNSUPPORTED (-2)   /* the requested lane cannot run this shape / dtype */
#define KDA_ERR_WORKSPACE (-3)     /* workspace pointer null, misaligned or too small */
#define KDA_ERR_CUDA (-4)          /* a CUDA launch or runtime call reported an error */
#define KDA_ERR_NULL (-5)          /* a required pointer is null */
#define KDA_ERR_DEVICE_STATUS (-6) /* a kernel raised its device-side status word (bounded wait expired) */
#define KDA_ERR_CU_SEQLENS (-7)    /* cu_seqlens (read on the device) is inconsistent with tokens / the workspace */

#define KDA_DTYPE_F32 0
#define KDA_DTYPE_BF16 1
/* kda_conv_fwd / kda_conv_bwd only: OR this into io_dtype when `weight` is float32 although the activations are
 * not; each weight is then rounded to the activation dtype as it is loaded (the result a cast of the weight tensor
 * would give) and no converted copy of the weights is needed. */
#define KDA_WEIGHT_F32 0x100

#define KDA_LANE_FP32 0 /* CUDA-core float32 arithmetic, any K, V <= 256 */
#define KDA_LANE_TC 1   /* tcgen05 BF16 tensor-core tiles, float32 accumulation and state */

#define KDA_MAX_DIM 256

typedef struct KdaChunkShape {
    int32_t n_seq;      /* sequences: batch size, or number of packed segments */
    int32_t seq_len;    /* tokens per sequence for fixed-length batches; ignored when cu_seqlens != NULL */
    int32_t tokens;     /* total tokens = n_seq*seq_len, or the packed total */
    int32_t heads;      /* H */
    int32_t key_dim;    /* K */
    int32_t value_dim;  /* V */
    int32_t io_dtype;   /* KDA_DTYPE_* of q,k,v,o,do and dq,dk,dv */
    int32_t gate_dtype; /* KDA_DTYPE_* of g, beta and of dg, dbeta */
    int32_t lane;       /* KDA_LANE_* */
    int32_t l2norm;     /* 1: L2-normalise q and k inside the kernels (reference behaviour) */
    float scale;        /* multiplies the normalised q */
    int32_t forward_only; /* 1: inference / prefill - no backward will follow: the forward skips every panel only the
                             backward reads, kda_chunk_workspace_bytes shrinks accordingly, and the workspace is free
                             again as soon as the call's kernels have run; kda_chunk_bwd rejects such a shape */
} KdaChunkShape;

const char* kda_error_string(int code);
/* Compile-time facts: returns e.g. "sm_100a". */
const char* kda_build_arch(void);

/* ---- chunked KDA, forward -------------------------------------------------
 * Stands in for nanochat_kda::chunk_forward on already-activated inputs
 * (reference nanochat/mixers/cuda_kda/chunk.cu:1665-1756 and
 * chunk_wy_forward.cu:1592-1723).  The raw-input form of the reference is
 * kda_gate_fwd followed by this call.
 *
 * workspace: kda_chunk_workspace_bytes(shape) bytes, 256-byte aligned.  The
 * forward leaves in it everything the backward needs; keep it untouched until
 * kda_chunk_bwd has run.  h0 and final_state may be NULL.
 * With shape->forward_only set this is the no-grad prefill path (the reference
 * sends such calls to its token loop, chunk.cu:1694-1698).
 */
size_t kda_chunk_workspace_bytes(const KdaChunkShape* shape);
int kda_chunk_fwd(const KdaChunkShape* shape, const void* q, const void* k, const void* v, const void* g,
                  const void* beta, const float* h0, const int32_t* cu_seqlens, void* o, float* final_state,
                  void* workspace, size_t workspace_bytes, void* stream);

/* The no-grad forward with the layer's three short convolutions folded in: xq, xk, xv [tokens,H,128] bf16 are the
 * INPUTS of the q, k, v convolutions (width 4, SiLU, no carried-in window: zero padding at every sequence start), wq, wk,
 * wv [H*128,4] their weights (weight_dtype KDA_DTYPE_F32: rounded to bf16 as loaded, or KDA_DTYPE_BF16); the activations
 * are formed inside the intra-chunk kernel and never written to memory.  o and final_state equal
 * kda_conv_fwd x3 followed by kda_chunk_fwd bit for bit.  Tensor-core lane with forward_only = 1 only (a backward would
 * need the activations), otherwise KDA_ERR_UNSUPPORTED.  Fuses the operator boundary between
 * causal_convolution_forward and chunk_forward (nanochat/mixers/kda.py:745-767); no counterpart operator in the
 * reference. */
int kda_chunk_fwd_conv(const KdaChunkShape* shape, const void* xq, const void* xk, const void* xv, const void* wq,
                       const void* wk, const void* wv, int32_t conv_width, int32_t weight_dtype, const void* g,
                       const void* beta, const float* h0, const int32_t* cu_seqlens, void* o, float* final_state,
                       void* workspace, size_t workspace_bytes, void* stream);

/* The forward with the layer's gated RMSNorm applied in the output kernel's epilogue, while the output tile is still on
 * chip (tensor-core lane only, otherwise KDA_ERR_UNSUPPORTED and the caller runs kda_rmsnorm_gate_fwd itself):
 *   y = o * rsqrt(mean_v(o^2) + eps) * norm_weight * sigmoid(gate),   gate, y [tokens,H,V] bf16, inv_rms [tokens,H] float32.
 * o is written too (the norm's backward, kda_rmsnorm_gate_bwd, takes it as x); y and inv_rms equal the stand-alone
 * kernel's results bit for bit.  Fuses the operator boundary the reference layer crosses between chunk_forward and
 * rmsnorm_gate_forward (nanochat/mixers/kda.py:768-795); no counterpart operator in the reference. */
int kda_chunk_fwd_norm(const KdaChunkShape* shape, const void* q, const void* k, const void* v, const void* g,
                       const void* beta, const float* h0, const int32_t* cu_seqlens, void* o, float* final_state,
                       void* workspace, size_t workspace_bytes, const void* gate, const float* norm_weight, float eps,
                       void* y, float* inv_rms, void* stream);

/* ---- chunked KDA, backward ------------------------------------------------
 * Stands in for nanochat_kda::chunk_backward (reference chunk.cu:1758-2113,
 * chunk_wy_backward.cu:3991-4323).  `workspace` is the buffer the matching
 * forward filled; `scratch` is kda_chunk_bwd_scratch_bytes(shape) bytes of
 * uninitialised memory.  d_final_state (cotangent of final_state) and dh0 may be NULL.
 */
size_t kda_chunk_bwd_scratch_bytes(const KdaChunkShape* shape);
int kda_chunk_bwd(const KdaChunkShape* shape, const void* q, const void* k, const void* v, const void* g,
                  const void* beta, const int32_t* cu_seqlens, const void* d_o, const float* d_final_state,
                  const void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes, void* dq,
                  void* dk, void* dv, void* dg, void* dbeta, float* dh0, void* stream);

/* ---- device status word ---------------------------------------------------
 * Every forward starts by checking cu_seqlens on the device and clearing the status word that lives in its workspace;
 * a tensor-core-lane kernel whose bounded wait expires writes its wait code there (its results are then undefined).
 * kda_chunk_status copies the word back over `stream` and SYNCHRONISES it - for tests and post-mortems, not for the hot
 * path and not under stream capture.  It returns KDA_OK, KDA_ERR_CU_SEQLENS (segments that were inconsistent were
 * treated as empty, so no kernel left the tensors) or KDA_ERR_DEVICE_STATUS.
 * kda_chunk_status_async only queues the 4-byte copy into caller-owned page-locked host memory (nothing waits, so it
 * may sit at the end of every call); the caller reads the word once the stream has passed that point and turns it
 * into a code with kda_status_word_code.  No reference counterpart (the reference's kernels have no device-side waits
 * and no packed batches). */
int kda_chunk_status(const KdaChunkShape* shape, const void* workspace, void* stream);
int kda_chunk_status_async(const KdaChunkShape* shape, const void* workspace, int32_t* host_word, void* stream);
int kda_status_word_code(int32_t word);
/* Self-test of the bounded wait: a one-warp kernel waits poll_limit (<= 1,000,000) polls on a barrier nothing arrives
 * at, then returns.  device_words[0] receives the status word (non-zero after the wait ran out), device_words[1] is 2
 * when the kernel carried on past the expired wait.  Never traps and never spins without bound.  No reference
 * counterpart. */
int kda_selftest_bounded_wait(int32_t* device_words, uint32_t poll_limit, void* stream);

/* ---- gate / beta activations ----------------------------------------------
 * g = lower_bound * sigmoid(exp(A_log[h]) * (raw_gate + dt_bias[h,k])), beta = sigmoid(beta_logits)
 * (reference chunk.cu:98-132, chunk_wy_forward.cu:188-264; oracle tests/kda_oracle.py:31-47).
 * g_out and beta_out are float32 regardless of io_dtype.
 */
int kda_gate_fwd(int32_t tokens, int32_t heads, int32_t key_dim, int32_t io_dtype, const void* raw_gate,
                 const void* beta_logits, const float* A_log, const float* dt_bias, float lower_bound, float* g_out,
                 float* beta_out, void* stream);
/* VJP of kda_gate_fwd (reference chunk_wy_backward.cu:3881-3987): d_raw_gate, d_beta_logits in io_dtype;
 * dA_log [H] and ddt_bias [H*K] float32, reduced deterministically.  scratch: kda_gate_bwd_scratch_bytes. */
size_t kda_gate_bwd_scratch_bytes(int32_t tokens, int32_t heads, int32_t key_dim);
int kda_gate_bwd(int32_t tokens, int32_t heads, int32_t key_dim, int32_t io_dtype, const void* raw_gate,
                 const void* beta_logits, const float* A_log, const float* dt_bias, float lower_bound, const float* dg,
                 const float* dbeta, void* d_raw_gate, void* d_beta_logits, float* dA_log, float* ddt_bias,
                 void* scratch, size_t scratch_bytes, void* stream);

/* ---- recurrent decode step --------------------------------------------------
 * One token per sequence on activated inputs: reads state_in, writes state_out
 * (may alias state_in for an in-place update) and o.  Stands in for
 * nanochat_kda::recurrent_decode (reference recurrent_decode.cu:24-181).
 * q,k,g [n_seq,H,K]; v,o [n_seq,H,V]; beta [n_seq,H]; io_dtype for q,k,v,o and gate_dtype for g, beta.
 */
int kda_decode_step(int32_t n_seq, int32_t heads, int32_t key_dim, int32_t value_dim, int32_t io_dtype,
                    int32_t gate_dtype, int32_t l2norm, float scale, const void* q, const void* k, const void* v, const void* g, const void* beta,
                    const float* state_in, float* state_out, void* o, void* stream);

/* The decode step on RAW inputs: raw_gate [n_seq,H,K] and beta_logits [n_seq,H] (io_dtype) are activated inside the
 * kernel (g = lower_bound * sigmoid(exp(A_log[h]) * (raw + dt_bias[h,k])), beta = sigmoid(logit)), which is exactly
 * nanochat_kda::recurrent_decode's signature (reference recurrent_decode.cu:96-181) in one launch instead of two.
 * q and k are L2-normalised.  state_out may alias state_in. */
int kda_decode_step_raw(int32_t n_seq, int32_t heads, int32_t key_dim, int32_t value_dim, int32_t io_dtype, float scale,
                        const void* q, const void* k, const void* v, const void* raw_gate, const void* beta_logits,
                        const float* A_log, const float* dt_bias, float lower_bound, const float* state_in, float* state_out,
                        void* o, void* stream);

/* n_steps consecutive decode steps in one call: step i reads q,k,g [n_steps,n_seq,H,K], v [n_steps,n_seq,H,V],
 * beta [n_steps,n_seq,H] at index i, updates `state` in place and writes o[i].  One kernel launch per step (the state
 * crosses HBM once each way per step, exactly as n_steps calls of kda_decode_step would), without a host round trip
 * per token; the reference's decode loop makes one operator call per token and layer (nanochat/engine.py:83-226,
 * recurrent_decode.cu:96-181). */
int kda_decode_steps(int32_t n_steps, int32_t n_seq, int32_t heads, int32_t key_dim, int32_t value_dim, int32_t io_dtype,
                     int32_t gate_dtype, int32_t l2norm, float scale, const void* q, const void* k, const void* v,
                     const void* g, const void* beta, float* state, void* o, void* stream);

/* ---- short causal depthwise convolution + SiLU --------------------------------
 * x,y [B,T,C]; weight [C,W] in io_dtype; cache [B,C,W] in io_dtype holds the last W
 * inputs including the current token.  Stands in for
 * nanochat_kda::causal_convolution_forward / _backward
 * (reference causal_convolution_forward.cu:149-237, causal_convolution_backward.cu:303-451).
 * initial_state, final_state, d_final_state, d_initial_state may be NULL.
 * dweight is float32 [C,W]; scratch: kda_conv_bwd_scratch_bytes.
 */
int kda_conv_fwd(int32_t batch, int32_t seq_len, int32_t channels, int32_t width, int32_t io_dtype, int32_t silu,
                 const void* x, const void* weight, const void* initial_state, void* y, void* final_state,
                 void* stream);
size_t kda_conv_bwd_scratch_bytes(int32_t batch, int32_t seq_len, int32_t channels, int32_t width);
int kda_conv_bwd(int32_t batch, int32_t seq_len, int32_t channels, int32_t width, int32_t io_dtype, int32_t silu,
                 const void* x, const void* weight, const void* initial_state, const void* d_y,
                 const void* d_final_state, void* dx, float* dweight, void* d_initial_state, void* scratch,
                 size_t scratch_bytes, void* stream);

/* n_items (1..4) same-shaped convolutions in ONE launch each way - the q, k and v branches of a layer (the reference
 * issues three separate operator calls, nanochat/mixers/kda.py:758-766; there is no batched counterpart there).
 * Training path only: no carried-in window, no final state, width <= 4, even channel count, 16-byte aligned tensors;
 * any other case returns KDA_ERR_UNSUPPORTED and the caller issues the per-tensor calls.  x, weight, y, d_y, dx, dweight
 * are HOST arrays of n_items device pointers; io_dtype may carry KDA_WEIGHT_F32.  scratch:
 * kda_conv_bwd_multi_scratch_bytes. */
/* One decode token through n_items (1..4) same-shaped convolutions in ONE launch, caches updated IN PLACE: for every
 * (batch, channel) the cache row [W] drops its oldest value, takes x (x, y [batch, channels]) and y = act(w . row).
 * The reference's decode path makes three non-mutating operator calls per layer and token, each allocating a new cache
 * (nanochat/mixers/kda.py:758-766, nanochat/engine.py:160-170); this is the opt-in in-place form for a serving loop that
 * owns its state.  width <= 4; io_dtype may carry KDA_WEIGHT_F32.  x, weight, cache, y: HOST arrays of device pointers. */
int kda_conv_step_multi(int32_t n_items, int32_t batch, int32_t channels, int32_t width, int32_t io_dtype, int32_t silu,
                        const void* const* x, const void* const* weight, void* const* cache, void* const* y, void* stream);
int kda_conv_fwd_multi(int32_t n_items, int32_t batch, int32_t seq_len, int32_t channels, int32_t width, int32_t io_dtype,
                       int32_t silu, const void* const* x, const void* const* weight, void* const* y, void* stream);
size_t kda_conv_bwd_multi_scratch_bytes(int32_t n_items, int32_t batch, int32_t seq_len, int32_t channels, int32_t width);
int kda_conv_bwd_multi(int32_t n_items, int32_t batch, int32_t seq_len, int32_t channels, int32_t width, int32_t io_dtype,
                       int32_t silu, const void* const* x, const void* const* weight, const void* const* d_y,
                       void* const* dx, float* const* dweight, void* scratch, size_t scratch_bytes, void* stream);

/* ---- gated RMSNorm --------------------------------------------------------------
 * y = x * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate) over the last dimension.
 * x, gate, y [rows, dim] in io_dtype; weight float32 [dim]; inv_rms float32 [rows].
 * Stands in for nanochat_kda::rmsnorm_gate_forward / _backward (reference rmsnorm_gate.cu:31-273).
 */
int kda_rmsnorm_gate_fwd(int64_t rows, int32_t dim, int32_t io_dtype, float eps, const void* x, const void* gate,
                         const float* weight, void* y, float* inv_rms, void* stream);
size_t kda_rmsnorm_gate_bwd_scratch_bytes(int64_t rows, int32_t dim);
int kda_rmsnorm_gate_bwd(int64_t rows, int32_t dim, int32_t io_dtype, const void* x, const void* gate,
                         const float* weight, const float* inv_rms, const void* d_y, void* dx, void* dgate,
                         float* dweight, void* scratch, size_t scratch_bytes, void* stream);

/* ---- gated RMSNorm backward without a scratch argument (no counterpart in the reference) ----
 * Same result as kda_rmsnorm_gate_bwd, for callers that cannot supply scratch memory: a serving
 * process whose device memory was planned once at start-up, a plugin that receives tensors but no
 * allocator, or a latency-critical path that must avoid cudaMalloc because it stalls the device.
 * The partial sums live in a 1.2 MB array built into the library (held by every GPU that loads it
 * until the process exits).  Limits: dim <= 256, otherwise KDA_ERR_UNSUPPORTED.  Calls no
 * cudaMalloc / cudaFree and no allocating library routine.  The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress, with that device current); make that first
 * call before starting any stream capture.  All calls share the one array and nothing in it needs
 * to start at zero (every partial read is written earlier in the same call), but two calls that
 * overlap on the GPU (different streams, no ordering between them) race on it. */
int kda_rmsnorm_gate_bwd_static(int64_t rows, int32_t dim, int32_t io_dtype, const void* x, const void* gate,
                                const float* weight, const float* inv_rms, const void* d_y, void* dx, void* dgate,
                                float* dweight, void* stream);

/* ---- launch accounting (diagnostics; no counterpart in the reference) ---------------
 * kda_launch_count: kernels this library has launched in this process so far.
 * kda_profile_enable(1): from now on every launch is bracketed by CUDA events on its stream.
 * kda_profile_report: waits for those events, writes "kernel,launches,total_ms" lines into
 * out (NUL-terminated, at most cap bytes), clears the records and returns the text length. */
unsigned long long kda_launch_count(void);
void kda_profile_enable(int on);
int kda_profile_report(char* out, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* KDA_B200_H */
