// Native registration of the reference mixer's operator namespace over libkda_b200's C ABI.
//
// The reference loads a shared library whose static initialisers register `nanochat_kda::*` with the
// dispatcher (TORCH_LIBRARY in nanochat/mixers/cuda_kda/recurrent_decode.cu:185-190, TORCH_LIBRARY_FRAGMENT in
// chunk.cu:2116-2131, causal_convolution_forward.cu:240-247, causal_convolution_backward.cu:454-463,
// rmsnorm_gate.cu:276-286) and reaches the operators as torch.ops.nanochat_kda.<name>
// (nanochat/mixers/kda.py:374-380).  This file is that library for the B200 kernels: the seven schemas are the
// reference's (argument names, order, types and return names), chunk_forward / chunk_backward carry one more trailing,
// defaulted `Tensor? cu_seqlens=None` for packed batches, so the reference's positional callers keep working.  Every
// implementation validates its inputs the way the reference's validate_chunk_inputs does (chunk.cu:1613-1663) before
// anything is launched, allocates its outputs with ATen, takes the current stream of the tensors' device and calls the
// C ABI declared in include/kda_b200.h.  A non-zero return code becomes a RuntimeError carrying kda_error_string().
// There is no CPU implementation: a CPU tensor fails in the dispatcher.
//
// chunk_backward receives only the operator inputs and the forward output (the reference's fixed ABI).  Like the
// reference (chunk_wy_forward.cu:1623-1651, found again by pointer arithmetic in chunk_wy_backward.cu:4026-4054) the
// forward therefore returns `output` as the visible head of one larger allocation whose tail - the sidecar - holds the
// activated gate, beta and the kernels' workspace; the backward finds the sidecar behind `output` and runs only the
// backward kernels.  An `output` that is not such a head (a copy, or a forward that ran without gradients) makes the
// backward run the forward again into a fresh workspace first.

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGraphsC10Utils.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <deque>
#include <mutex>
#include <tuple>
#include <unordered_map>

#include "kda_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

void check(int rc, const char* what) {
    TORCH_CHECK(rc == 0, "libkda_b200: ", what, " failed: ", kda_error_string(rc), " (", rc, ")");
}

void* stream_of(const Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

bool has(const OptTensor& t) { return t.has_value() && t->defined(); }
const void* ptr(const OptTensor& t) { return has(t) ? t->data_ptr() : nullptr; }

Tensor bytes(size_t n, const Tensor& like) {
    return at::empty({(int64_t)(n < 256 ? 256 : n)}, like.options().dtype(at::kByte));
}

size_t up256(size_t n) { return (n + 255) / 256 * 256; }

// ------------------------------------------------------------------------------------------------ validation
struct Dims {
    int64_t B, T, H, K, V, N;      // N: number of memory states (B, or the number of packed segments)
};

// Shapes first, then value ranges, then dtypes, then devices - so that a shape mistake is reported as such whatever
// device the tensors live on, and nothing reaches a kernel with a pointer or an extent it cannot take.
Dims validate_chunk_inputs(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& raw_gate, const Tensor& beta_logits,
                           const Tensor& A_log, const Tensor& dt_bias, const OptTensor& initial_state, double lower_bound,
                           const OptTensor& cu_seqlens) {
    TORCH_CHECK(q.dim() == 4, "q must have shape [B, T, H, K]");
    TORCH_CHECK(k.sizes() == q.sizes() && raw_gate.sizes() == q.sizes(), "q, k, and raw_gate shapes must match");
    TORCH_CHECK(v.dim() == 4 && v.size(0) == q.size(0) && v.size(1) == q.size(1) && v.size(2) == q.size(2),
                "v must match q in B, T, and H");
    TORCH_CHECK(beta_logits.dim() == 3 && beta_logits.size(0) == q.size(0) && beta_logits.size(1) == q.size(1) &&
                    beta_logits.size(2) == q.size(2),
                "beta_logits must have shape [B, T, H]");
    Dims d{q.size(0), q.size(1), q.size(2), q.size(3), v.size(3), q.size(0)};
    TORCH_CHECK(d.K >= 1 && d.K <= KDA_MAX_DIM && d.V >= 1 && d.V <= KDA_MAX_DIM, "head dimensions must be in [1, ", KDA_MAX_DIM, "]");
    TORCH_CHECK(d.B * d.T < (int64_t(1) << 31), "too many tokens for one call");
    TORCH_CHECK(A_log.numel() == d.H, "A_log must be contiguous CUDA float32 [H]");
    TORCH_CHECK(dt_bias.numel() == d.H * d.K, "dt_bias must be contiguous CUDA float32 with H*K elements");
    if (has(cu_seqlens)) {
        TORCH_CHECK(cu_seqlens->dim() == 1 && cu_seqlens->numel() >= 2, "cu_seqlens must be int32 [N+1]");
        TORCH_CHECK(d.B == 1, "packed inputs (cu_seqlens) require batch size 1");
        d.N = cu_seqlens->numel() - 1;
    }
    if (has(initial_state)) {
        const Tensor& s = *initial_state;
        TORCH_CHECK(s.dim() == 4 && s.size(0) == d.N && s.size(1) == d.H && s.size(2) == d.V && s.size(3) == d.K,
                    "initial_state must have shape [B, H, V, K]");
    }
    TORCH_CHECK(lower_bound >= -5.0 && lower_bound < 0.0, "safe-gate lower_bound must be in [-5, 0)");
    for (const Tensor* t : {&q, &k, &v, &raw_gate, &beta_logits})
        TORCH_CHECK(t->scalar_type() == at::kBFloat16, "activation tensors must be bfloat16");
    TORCH_CHECK(A_log.scalar_type() == at::kFloat && dt_bias.scalar_type() == at::kFloat, "A_log and dt_bias must be float32");
    TORCH_CHECK(A_log.is_contiguous() && dt_bias.is_contiguous(), "A_log and dt_bias must be contiguous");
    if (has(initial_state))
        TORCH_CHECK(initial_state->scalar_type() == at::kFloat && initial_state->is_contiguous(),
                    "initial_state must be contiguous CUDA float32");
    if (has(cu_seqlens)) TORCH_CHECK(cu_seqlens->scalar_type() == at::kInt && cu_seqlens->is_contiguous(), "cu_seqlens must be int32 [N+1]");
    TORCH_CHECK(q.is_cuda(), "q must be a CUDA tensor");
    auto same_device = [&](const Tensor& t, const char* name) {
        TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
        TORCH_CHECK(t.device() == q.device(), name, " must be on the same device as q");
    };
    same_device(k, "k"); same_device(v, "v"); same_device(raw_gate, "raw_gate"); same_device(beta_logits, "beta_logits");
    same_device(A_log, "A_log"); same_device(dt_bias, "dt_bias");
    if (has(initial_state)) same_device(*initial_state, "initial_state");
    if (has(cu_seqlens)) same_device(*cu_seqlens, "cu_seqlens");
    return d;
}

// The checks alone, callable with tensors of any device (registered as nanochat_kda::_validate_chunk_inputs).
void validate_only(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& raw_gate, const Tensor& beta_logits, const Tensor& A_log,
                   const Tensor& dt_bias, const OptTensor& initial_state, double lower_bound, const OptTensor& cu_seqlens) {
    validate_chunk_inputs(q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state, lower_bound, cu_seqlens);
}

// ------------------------------------------------------------------------------------------------ device status
// Every chunk forward / backward queues a 4-byte copy of its workspace's status word into a page-locked ring and an
// event behind it; the next call on that device reads the words whose events have completed (a host memory read, no
// synchronisation) and raises if one is non-zero - an expired bounded wait or an inconsistent cu_seqlens therefore
// cannot pass silently, and the hot path never waits.  Skipped while a stream capture is in progress.
struct StatusRing {
    Tensor words;      // pinned int32 [kSlots]
    struct Pending {
        at::cuda::CUDAEvent ev;
        int slot;
    };
    std::deque<Pending> pending;
    int next = 0;
};
constexpr int kSlots = 64;
std::mutex status_mu;
std::unordered_map<int, StatusRing> rings;

bool capturing() { return c10::cuda::currentStreamCaptureStatusMayInitCtx() != c10::cuda::CaptureStatus::None; }

void poll_status(int device) {
    if (capturing()) return;
    std::lock_guard<std::mutex> lk(status_mu);
    auto it = rings.find(device);
    if (it == rings.end()) return;
    StatusRing& r = it->second;
    int bad = 0;
    while (!r.pending.empty() && r.pending.front().ev.query()) {
        int32_t* w = r.words.data_ptr<int32_t>() + r.pending.front().slot;
        if (*w != 0 && bad == 0) bad = *w;
        *w = 0;
        r.pending.pop_front();
    }
    if (bad != 0) {
        const int rc = kda_status_word_code(bad);
        TORCH_CHECK(false, "libkda_b200: an earlier KDA call on cuda:", device, " reported device status ", bad, ": ", kda_error_string(rc),
                    " (", rc, "); its results are undefined");
    }
}

void queue_status(const KdaChunkShape& sh, const void* workspace, const Tensor& like) {
    if (capturing()) return;
    const int device = like.device().index();
    std::lock_guard<std::mutex> lk(status_mu);
    StatusRing& r = rings[device];
    if (!r.words.defined()) r.words = at::zeros({kSlots}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
    if ((int)r.pending.size() >= kSlots) return;      // the host is far ahead of the device: skip this sample
    const int slot = r.next++ % kSlots;
    auto stream = c10::cuda::getCurrentCUDAStream(device);
    if (kda_chunk_status_async(&sh, workspace, r.words.data_ptr<int32_t>() + slot, stream.stream()) != KDA_OK) return;
    r.pending.emplace_back();
    r.pending.back().slot = slot;
    r.pending.back().ev.record(stream);
}

// ------------------------------------------------------------------------------------------------ chunked operator
KdaChunkShape chunk_shape(const Dims& d, double scale, bool packed, bool forward_only) {
    KdaChunkShape sh;
    sh.n_seq = (int32_t)d.N;
    sh.seq_len = packed ? 0 : (int32_t)d.T;
    sh.tokens = (int32_t)(d.B * d.T);
    sh.heads = (int32_t)d.H;
    sh.key_dim = (int32_t)d.K;
    sh.value_dim = (int32_t)d.V;
    sh.io_dtype = KDA_DTYPE_BF16;
    sh.gate_dtype = KDA_DTYPE_F32;
    sh.lane = (d.K == 128 && d.V == 128) ? KDA_LANE_TC : KDA_LANE_FP32;
    sh.l2norm = 1;
    sh.scale = (float)scale;
    sh.forward_only = forward_only ? 1 : 0;
    return sh;
}

// one allocation: [output | activated gate g (float32) | beta (float32) | kernel workspace], 256-byte aligned parts
struct Layout {
    size_t out_bytes, g_off, beta_off, ws_off, ws_bytes, total;
};

Layout layout_for(const Dims& d, const KdaChunkShape& sh) {
    Layout l;
    l.out_bytes = (size_t)(d.B * d.T * d.H * d.V) * 2;
    l.g_off = up256(l.out_bytes);
    l.beta_off = l.g_off + up256((size_t)(d.B * d.T * d.H * d.K) * 4);
    l.ws_off = l.beta_off + up256((size_t)(d.B * d.T * d.H) * 4);
    l.ws_bytes = up256(kda_chunk_workspace_bytes(&sh));
    l.total = l.ws_off + l.ws_bytes;
    return l;
}

// forwards whose sidecar may still be alive, keyed by the address of `output`
struct Kept {
    Dims d;
    KdaChunkShape sh;
    Layout l;
    double lower_bound;
};
std::mutex kept_mu;
std::unordered_map<const void*, Kept> kept;

bool same_dims(const Dims& a, const Dims& b) { return a.B == b.B && a.T == b.T && a.H == b.H && a.K == b.K && a.V == b.V && a.N == b.N; }

void run_gate(const Tensor& raw_gate, const Tensor& beta_logits, const Tensor& A_log, const Tensor& dt_bias, double lower_bound, const Dims& d,
              float* g, float* beta) {
    check(kda_gate_fwd((int32_t)(d.B * d.T), (int32_t)d.H, (int32_t)d.K, KDA_DTYPE_BF16, raw_gate.data_ptr(), beta_logits.data_ptr(),
                       A_log.data_ptr<float>(), dt_bias.data_ptr<float>(), (float)lower_bound, g, beta, stream_of(raw_gate)),
          "kda_gate_fwd");
}

std::tuple<Tensor, OptTensor> chunk_forward(const Tensor& q_, const Tensor& k_, const Tensor& v_, const Tensor& raw_gate_,
                                            const Tensor& beta_logits_, const Tensor& A_log, const Tensor& dt_bias,
                                            const OptTensor& initial_state, bool output_final_state, double lower_bound, double scale,
                                            const OptTensor& cu_seqlens) {
    const Dims d = validate_chunk_inputs(q_, k_, v_, raw_gate_, beta_logits_, A_log, dt_bias, initial_state, lower_bound, cu_seqlens);
    c10::cuda::CUDAGuard guard(q_.device());
    poll_status(q_.device().index());
    const Tensor q = q_.contiguous(), k = k_.contiguous(), v = v_.contiguous(), raw_gate = raw_gate_.contiguous(),
                 beta_logits = beta_logits_.contiguous();
    // A call none of whose inputs takes part in a graph is inference / prefill: nothing is kept for a backward.
    bool needs_grad = false;
    for (const Tensor* t : {&q_, &k_, &v_, &raw_gate_, &beta_logits_, &A_log, &dt_bias}) needs_grad = needs_grad || t->requires_grad();
    if (has(initial_state)) needs_grad = needs_grad || initial_state->requires_grad();
    const KdaChunkShape sh = chunk_shape(d, scale, has(cu_seqlens), !needs_grad);
    const Layout l = layout_for(d, sh);
    Tensor buf = at::empty({(int64_t)l.total}, q.options().dtype(at::kByte));
    char* base = static_cast<char*>(buf.data_ptr());
    Tensor output = buf.narrow(0, 0, (int64_t)l.out_bytes).view(at::kBFloat16).view({d.B, d.T, d.H, d.V});
    float* g = reinterpret_cast<float*>(base + l.g_off);
    float* beta = reinterpret_cast<float*>(base + l.beta_off);
    OptTensor final_state;
    if (output_final_state) final_state = at::empty({d.N, d.H, d.V, d.K}, q.options().dtype(at::kFloat));
    if (d.B * d.T > 0) {
        run_gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound, d, g, beta);
        check(kda_chunk_fwd(&sh, q.data_ptr(), k.data_ptr(), v.data_ptr(), g, beta, static_cast<const float*>(ptr(initial_state)),
                            static_cast<const int32_t*>(ptr(cu_seqlens)), output.data_ptr(),
                            output_final_state ? final_state->data_ptr<float>() : nullptr, base + l.ws_off, l.ws_bytes, stream_of(q)),
              "kda_chunk_fwd");
        queue_status(sh, base + l.ws_off, q);
    } else if (output_final_state) {
        if (has(initial_state)) final_state->copy_(*initial_state);
        else final_state->zero_();
    }
    if (needs_grad) {
        std::lock_guard<std::mutex> lk(kept_mu);
        if (kept.size() > 4096) kept.clear();      // entries of outputs long gone; a miss only costs a recompute
        kept[output.data_ptr()] = Kept{d, sh, l, lower_bound};
    }
    return {output, final_state};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, OptTensor> chunk_backward(
    const Tensor& q_, const Tensor& k_, const Tensor& v_, const Tensor& raw_gate_, const Tensor& beta_logits_, const Tensor& A_log,
    const Tensor& dt_bias, const OptTensor& initial_state, const Tensor& output, const OptTensor& /*final_state*/,
    const Tensor& grad_output, const OptTensor& grad_final_state, double lower_bound, double scale, const OptTensor& cu_seqlens) {
    const Dims d = validate_chunk_inputs(q_, k_, v_, raw_gate_, beta_logits_, A_log, dt_bias, initial_state, lower_bound, cu_seqlens);
    TORCH_CHECK(grad_output.dim() == 4 && grad_output.size(0) == d.B && grad_output.size(1) == d.T && grad_output.size(2) == d.H &&
                    grad_output.size(3) == d.V,
                "grad_output must have shape [B, T, H, V]");
    TORCH_CHECK(grad_output.is_cuda() && grad_output.device() == q_.device(), "grad_output must be on the same device as q");
    if (has(grad_final_state)) {
        TORCH_CHECK(grad_final_state->dim() == 4 && grad_final_state->size(0) == d.N && grad_final_state->size(1) == d.H &&
                        grad_final_state->size(2) == d.V && grad_final_state->size(3) == d.K,
                    "grad_final_state must have shape [B, H, V, K]");
        TORCH_CHECK(grad_final_state->is_cuda() && grad_final_state->device() == q_.device(), "grad_final_state must be on the same device as q");
    }
    c10::cuda::CUDAGuard guard(q_.device());
    poll_status(q_.device().index());
    const Tensor q = q_.contiguous(), k = k_.contiguous(), v = v_.contiguous(), raw_gate = raw_gate_.contiguous(),
                 beta_logits = beta_logits_.contiguous();
    const bool packed = has(cu_seqlens);
    KdaChunkShape sh = chunk_shape(d, scale, packed, false);
    Layout l = layout_for(d, sh);
    // the sidecar behind `output`, if this is the tensor a gradient-tracking forward returned
    const char* base = nullptr;
    Tensor recomputed;
    {
        std::lock_guard<std::mutex> lk(kept_mu);
        auto it = kept.find(output.defined() ? output.data_ptr() : nullptr);
        if (it != kept.end() && same_dims(it->second.d, d) && it->second.lower_bound == lower_bound && it->second.sh.scale == sh.scale &&
            it->second.sh.n_seq == sh.n_seq && it->second.sh.seq_len == sh.seq_len && output.is_cuda() && output.device() == q.device() &&
            output.scalar_type() == at::kBFloat16 && output.is_contiguous() && output.storage_offset() == 0 &&
            output.storage().nbytes() >= it->second.l.total)
            base = static_cast<const char*>(output.data_ptr());
    }
    if (base == nullptr && d.B * d.T > 0) {
        recomputed = at::empty({(int64_t)l.total}, q.options().dtype(at::kByte));
        char* b = static_cast<char*>(recomputed.data_ptr());
        Tensor scratch_out = recomputed.narrow(0, 0, (int64_t)l.out_bytes);
        run_gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound, d, reinterpret_cast<float*>(b + l.g_off),
                 reinterpret_cast<float*>(b + l.beta_off));
        check(kda_chunk_fwd(&sh, q.data_ptr(), k.data_ptr(), v.data_ptr(), b + l.g_off, b + l.beta_off,
                            static_cast<const float*>(ptr(initial_state)), static_cast<const int32_t*>(ptr(cu_seqlens)),
                            scratch_out.data_ptr(), nullptr, b + l.ws_off, l.ws_bytes, stream_of(q)),
              "kda_chunk_fwd (recomputed for the backward)");
        base = b;
    }
    const Tensor d_o = grad_output.contiguous().to(at::kBFloat16);
    OptTensor dfs;
    if (has(grad_final_state)) dfs = grad_final_state->contiguous().to(at::kFloat);
    Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
    Tensor dg = at::empty({d.B, d.T, d.H, d.K}, q.options().dtype(at::kFloat)), db = at::empty({d.B, d.T, d.H}, q.options().dtype(at::kFloat));
    OptTensor dh0;
    if (has(initial_state)) dh0 = at::empty({d.N, d.H, d.V, d.K}, q.options().dtype(at::kFloat));
    Tensor d_raw = at::empty_like(raw_gate), d_bl = at::empty_like(beta_logits);
    Tensor dA = at::empty({d.H}, q.options().dtype(at::kFloat)), dbias = at::empty({d.H * d.K}, q.options().dtype(at::kFloat));
    if (d.B * d.T == 0) {
        dA.zero_(); dbias.zero_();
        if (dh0.has_value()) {
            if (dfs.has_value()) dh0->copy_(*dfs);
            else dh0->zero_();
        }
        return {dq, dk, dv, d_raw, d_bl, dA, dbias.reshape(dt_bias.sizes()), dh0};
    }
    Tensor scratch = bytes(kda_chunk_bwd_scratch_bytes(&sh), q);
    check(kda_chunk_bwd(&sh, q.data_ptr(), k.data_ptr(), v.data_ptr(), base + l.g_off, base + l.beta_off,
                        static_cast<const int32_t*>(ptr(cu_seqlens)), d_o.data_ptr(), static_cast<const float*>(ptr(dfs)), base + l.ws_off,
                        l.ws_bytes, scratch.data_ptr(), (size_t)scratch.numel(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(),
                        db.data_ptr(), dh0.has_value() ? dh0->data_ptr<float>() : nullptr, stream_of(q)),
          "kda_chunk_bwd");
    queue_status(sh, base + l.ws_off, q);
    Tensor gscr = bytes(kda_gate_bwd_scratch_bytes((int32_t)(d.B * d.T), (int32_t)d.H, (int32_t)d.K), q);
    check(kda_gate_bwd((int32_t)(d.B * d.T), (int32_t)d.H, (int32_t)d.K, KDA_DTYPE_BF16, raw_gate.data_ptr(), beta_logits.data_ptr(),
                       A_log.data_ptr<float>(), dt_bias.data_ptr<float>(), (float)lower_bound, dg.data_ptr<float>(), db.data_ptr<float>(),
                       d_raw.data_ptr(), d_bl.data_ptr(), dA.data_ptr<float>(), dbias.data_ptr<float>(), gscr.data_ptr(),
                       (size_t)gscr.numel(), stream_of(q)),
          "kda_gate_bwd");
    return {dq, dk, dv, d_raw, d_bl, dA, dbias.reshape(dt_bias.sizes()), dh0};
}

std::tuple<Tensor, OptTensor> recurrent_decode(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& raw_gate,
                                               const Tensor& beta_logits, const Tensor& A_log, const Tensor& dt_bias,
                                               const OptTensor& initial_state, bool output_final_state, double lower_bound,
                                               double scale) {
    const Dims d = validate_chunk_inputs(q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state, lower_bound, c10::nullopt);
    TORCH_CHECK(d.T == 1, "recurrent decode requires T=1");
    TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && raw_gate.is_contiguous() && beta_logits.is_contiguous(),
                "all recurrent decode inputs must be contiguous");
    c10::cuda::CUDAGuard guard(q.device());
    Tensor g = at::empty({d.B, 1, d.H, d.K}, q.options().dtype(at::kFloat)), beta = at::empty({d.B, 1, d.H}, q.options().dtype(at::kFloat));
    Tensor state = has(initial_state) ? *initial_state : at::zeros({d.B, d.H, d.V, d.K}, q.options().dtype(at::kFloat));
    Tensor new_state = at::empty_like(state), o = at::empty_like(v);
    if (d.B > 0) {
        run_gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound, d, g.data_ptr<float>(), beta.data_ptr<float>());
        check(kda_decode_step((int32_t)d.B, (int32_t)d.H, (int32_t)d.K, (int32_t)d.V, KDA_DTYPE_BF16, KDA_DTYPE_F32, 1, (float)scale,
                              q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), state.data_ptr<float>(),
                              new_state.data_ptr<float>(), o.data_ptr(), stream_of(q)),
              "kda_decode_step");
    }
    return {o, output_final_state ? OptTensor(new_state) : OptTensor()};
}

// ------------------------------------------------------------------------------------------------ short convolution
int io_dtype_of(const Tensor& t) {
    TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, "nanochat_kda: float32 or bfloat16 tensors only");
    return t.scalar_type() == at::kBFloat16 ? KDA_DTYPE_BF16 : KDA_DTYPE_F32;
}

struct ConvDims {
    int64_t B, T, C, W;
};

ConvDims validate_conv(const Tensor& x, const Tensor& weight, const OptTensor& state, const char* state_name) {
    TORCH_CHECK(x.dim() == 3, "x must have shape [B, T, C]");
    TORCH_CHECK(weight.dim() == 2 && weight.size(0) == x.size(2) && weight.size(1) >= 1, "weight must have shape [C, W]");
    ConvDims d{x.size(0), x.size(1), x.size(2), weight.size(1)};
    if (has(state))
        TORCH_CHECK(state->dim() == 3 && state->size(0) == d.B && state->size(1) == d.C && state->size(2) == d.W, state_name,
                    " must have shape [B, C, W]");
    TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
    TORCH_CHECK(weight.is_cuda() && weight.device() == x.device(), "weight must be on the same device as x");
    if (has(state)) TORCH_CHECK(state->is_cuda() && state->device() == x.device(), state_name, " must be on the same device as x");
    io_dtype_of(x);
    return d;
}

std::tuple<Tensor, OptTensor> causal_convolution_forward(const Tensor& x, const Tensor& weight, const OptTensor& initial_state,
                                                         bool output_final_state) {
    const ConvDims d = validate_conv(x, weight, initial_state, "initial_state");
    TORCH_CHECK(x.is_contiguous(), "nanochat_kda::causal_convolution_forward requires a contiguous input");
    c10::cuda::CUDAGuard guard(x.device());
    const Tensor w = weight.contiguous().to(x.scalar_type());
    OptTensor s0;
    if (has(initial_state)) s0 = initial_state->contiguous().to(x.scalar_type());
    Tensor y = at::empty_like(x);
    OptTensor fin;
    if (output_final_state) fin = at::empty({d.B, d.C, d.W}, x.options());
    if (d.T == 0 || d.B == 0 || d.C == 0) {
        if (fin.has_value()) {
            if (s0.has_value()) fin->copy_(*s0);
            else fin->zero_();
        }
        return {y, fin};
    }
    check(kda_conv_fwd((int32_t)d.B, (int32_t)d.T, (int32_t)d.C, (int32_t)d.W, io_dtype_of(x), 1, x.data_ptr(), w.data_ptr(), ptr(s0),
                       y.data_ptr(), fin.has_value() ? fin->data_ptr() : nullptr, stream_of(x)),
          "kda_conv_fwd");
    return {y, fin};
}

std::tuple<Tensor, Tensor, OptTensor> causal_convolution_backward(const Tensor& x_, const Tensor& weight, const OptTensor& initial_state,
                                                                  const Tensor& /*output*/, const OptTensor& /*final_state*/,
                                                                  const Tensor& grad_output, const OptTensor& grad_final_state) {
    const ConvDims d = validate_conv(x_, weight, initial_state, "initial_state");
    validate_conv(x_, weight, grad_final_state, "grad_final_state");
    TORCH_CHECK(grad_output.sizes() == x_.sizes(), "grad_output must have the shape of x");
    TORCH_CHECK(grad_output.is_cuda() && grad_output.device() == x_.device(), "grad_output must be on the same device as x");
    c10::cuda::CUDAGuard guard(x_.device());
    const Tensor x = x_.contiguous();
    const Tensor w = weight.contiguous().to(x.scalar_type());
    OptTensor s0, dfin, dinit;
    if (has(initial_state)) {
        s0 = initial_state->contiguous().to(x.scalar_type());
        dinit = at::empty_like(*s0);
    }
    if (has(grad_final_state)) dfin = grad_final_state->contiguous().to(x.scalar_type());
    const Tensor dy = grad_output.contiguous().to(x.scalar_type());
    Tensor dx = at::empty_like(x), dw = at::empty({d.C, d.W}, x.options().dtype(at::kFloat));
    if (d.T == 0 || d.B == 0 || d.C == 0) {
        dw.zero_();
        if (dinit.has_value()) {
            if (dfin.has_value()) dinit->copy_(*dfin);
            else dinit->zero_();
        }
        return {dx, dw.to(weight.scalar_type()), dinit};
    }
    Tensor scratch = bytes(kda_conv_bwd_scratch_bytes((int32_t)d.B, (int32_t)d.T, (int32_t)d.C, (int32_t)d.W), x);
    check(kda_conv_bwd((int32_t)d.B, (int32_t)d.T, (int32_t)d.C, (int32_t)d.W, io_dtype_of(x), 1, x.data_ptr(), w.data_ptr(), ptr(s0),
                       dy.data_ptr(), ptr(dfin), dx.data_ptr(), dw.data_ptr<float>(), dinit.has_value() ? dinit->data_ptr() : nullptr,
                       scratch.data_ptr(), (size_t)scratch.numel(), stream_of(x)),
          "kda_conv_bwd");
    return {dx, dw.to(weight.scalar_type()), dinit};
}

// ------------------------------------------------------------------------------------------------ gated RMSNorm
int64_t validate_norm(const Tensor& x, const Tensor& gate, const Tensor& weight) {
    TORCH_CHECK(x.dim() >= 1 && x.size(-1) >= 1, "x must have a non-empty last dimension");
    TORCH_CHECK(gate.sizes() == x.sizes(), "gate must have the shape of x");
    TORCH_CHECK(weight.dim() == 1 && weight.numel() == x.size(-1), "weight must have shape [D]");
    TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
    TORCH_CHECK(gate.is_cuda() && gate.device() == x.device(), "gate must be on the same device as x");
    TORCH_CHECK(weight.is_cuda() && weight.device() == x.device(), "weight must be on the same device as x");
    io_dtype_of(x);
    return x.numel() / x.size(-1);
}

std::tuple<Tensor, Tensor> rmsnorm_gate_forward(const Tensor& x_, const Tensor& gate_, const Tensor& weight, double epsilon) {
    const int64_t rows = validate_norm(x_, gate_, weight);
    c10::cuda::CUDAGuard guard(x_.device());
    const Tensor x = x_.contiguous(), gate = gate_.contiguous().to(x_.scalar_type()), w = weight.contiguous().to(at::kFloat);
    const int64_t D = x.size(-1);
    Tensor y = at::empty_like(x), inv = at::empty({rows}, x.options().dtype(at::kFloat));
    if (rows > 0)
        check(kda_rmsnorm_gate_fwd(rows, (int32_t)D, io_dtype_of(x), (float)epsilon, x.data_ptr(), gate.data_ptr(), w.data_ptr<float>(),
                                   y.data_ptr(), inv.data_ptr<float>(), stream_of(x)),
              "kda_rmsnorm_gate_fwd");
    return {y, inv};
}

std::tuple<Tensor, Tensor, Tensor> rmsnorm_gate_backward(const Tensor& x_, const Tensor& gate_, const Tensor& weight,
                                                         const Tensor& inverse_rms, const Tensor& grad_output, double /*epsilon*/) {
    const int64_t rows = validate_norm(x_, gate_, weight);
    TORCH_CHECK(inverse_rms.numel() == rows, "inverse_rms must hold one value per row");
    TORCH_CHECK(inverse_rms.is_cuda() && inverse_rms.device() == x_.device() && inverse_rms.scalar_type() == at::kFloat,
                "inverse_rms must be CUDA float32 on the same device as x");
    TORCH_CHECK(grad_output.sizes() == x_.sizes(), "grad_output must have the shape of x");
    TORCH_CHECK(grad_output.is_cuda() && grad_output.device() == x_.device(), "grad_output must be on the same device as x");
    c10::cuda::CUDAGuard guard(x_.device());
    const Tensor x = x_.contiguous(), gate = gate_.contiguous().to(x_.scalar_type()), w = weight.contiguous().to(at::kFloat);
    const Tensor inv = inverse_rms.contiguous(), dy = grad_output.contiguous().to(x_.scalar_type());
    const int64_t D = x.size(-1);
    Tensor dx = at::empty_like(x), dgate = at::empty_like(gate), dw = at::empty({D}, x.options().dtype(at::kFloat));
    if (rows == 0) {
        dw.zero_();
        return {dx, dgate, dw.to(weight.scalar_type())};
    }
    Tensor scratch = bytes(kda_rmsnorm_gate_bwd_scratch_bytes(rows, (int32_t)D), x);
    check(kda_rmsnorm_gate_bwd(rows, (int32_t)D, io_dtype_of(x), x.data_ptr(), gate.data_ptr(), w.data_ptr<float>(), inv.data_ptr<float>(),
                               dy.data_ptr(), dx.data_ptr(), dgate.data_ptr(), dw.data_ptr<float>(), scratch.data_ptr(),
                               (size_t)scratch.numel(), stream_of(x)),
          "kda_rmsnorm_gate_bwd");
    return {dx, dgate, dw.to(weight.scalar_type())};
}

}  // namespace

TORCH_LIBRARY(nanochat_kda, m) {
    m.def("chunk_forward(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
          "Tensor? initial_state, bool output_final_state, float lower_bound, float scale, Tensor? cu_seqlens=None) "
          "-> (Tensor output, Tensor? final_state)");
    m.def("chunk_backward(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
          "Tensor? initial_state, Tensor output, Tensor? final_state, Tensor grad_output, Tensor? grad_final_state, "
          "float lower_bound, float scale, Tensor? cu_seqlens=None) -> (Tensor dq, Tensor dk, Tensor dv, Tensor draw_gate, "
          "Tensor dbeta_logits, Tensor dA_log, Tensor ddt_bias, Tensor? dinitial_state)");
    m.def("recurrent_decode(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
          "Tensor? initial_state, bool output_final_state, float lower_bound, float scale) -> (Tensor output, Tensor? final_state)");
    m.def("causal_convolution_forward(Tensor x, Tensor weight, Tensor? initial_state, bool output_final_state) "
          "-> (Tensor output, Tensor? final_state)");
    m.def("causal_convolution_backward(Tensor x, Tensor weight, Tensor? initial_state, Tensor output, Tensor? final_state, "
          "Tensor grad_output, Tensor? grad_final_state) -> (Tensor dx, Tensor dweight, Tensor? dinitial_state)");
    m.def("rmsnorm_gate_forward(Tensor x, Tensor gate, Tensor weight, float epsilon) -> (Tensor output, Tensor inverse_rms)");
    m.def("rmsnorm_gate_backward(Tensor x, Tensor gate, Tensor weight, Tensor inverse_rms, Tensor grad_output, float epsilon) "
          "-> (Tensor dx, Tensor dgate, Tensor dweight)");
    // the input checks of chunk_forward / chunk_backward / recurrent_decode on their own, for any device
    m.def("_validate_chunk_inputs(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
          "Tensor? initial_state, float lower_bound, Tensor? cu_seqlens=None) -> ()");
}

TORCH_LIBRARY_IMPL(nanochat_kda, CUDA, m) {
    m.impl("chunk_forward", &chunk_forward);
    m.impl("chunk_backward", &chunk_backward);
    m.impl("recurrent_decode", &recurrent_decode);
    m.impl("causal_convolution_forward", &causal_convolution_forward);
    m.impl("causal_convolution_backward", &causal_convolution_backward);
    m.impl("rmsnorm_gate_forward", &rmsnorm_gate_forward);
    m.impl("rmsnorm_gate_backward", &rmsnorm_gate_backward);
}

TORCH_LIBRARY_IMPL(nanochat_kda, CompositeExplicitAutograd, m) { m.impl("_validate_chunk_inputs", &validate_only); }
