// Native registration of the reference mixer's operator namespace over libkda_b200's C ABI.
//
// The reference loads a shared library whose static initialisers register `nanochat_kda::*` with the
// dispatcher (TORCH_LIBRARY in nanochat/mixers/cuda_kda/recurrent_decode.cu:185-190, TORCH_LIBRARY_FRAGMENT in
// chunk.cu:2116-2131, causal_convolution_forward.cu:240-247, causal_convolution_backward.cu:454-463,
// rmsnorm_gate.cu:276-286) and reaches the operators as torch.ops.nanochat_kda.<name>
// (nanochat/mixers/kda.py:374-380).  This file is that library for the B200 kernels: the seven schemas are the
// reference's, verbatim; every implementation allocates its outputs with ATen, takes the current stream of the
// tensors' device and calls the C ABI declared in include/kda_b200.h.  A non-zero return code becomes a
// RuntimeError carrying kda_error_string().  There is no CPU implementation: a CPU tensor fails in the dispatcher.
//
// chunk_backward receives only the operator inputs and the forward output (the reference's fixed ABI), so it runs the
// gate and the chunked forward again into a fresh workspace before the backward kernels.

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <tuple>

#include "kda_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

void check(int rc, const char* what) {
    TORCH_CHECK(rc == 0, "libkda_b200: ", what, " failed: ", kda_error_string(rc), " (", rc, ")");
}

void* stream_of(const Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

void need_bf16_cuda(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), "nanochat_kda: ", name, " must be a CUDA tensor");
    TORCH_CHECK(t.scalar_type() == at::kBFloat16, "nanochat_kda: ", name, " must be bfloat16");
}

Tensor bytes(size_t n, const Tensor& like) {
    return at::empty({(int64_t)(n < 256 ? 256 : n)}, like.options().dtype(at::kByte));
}

const void* ptr(const OptTensor& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

struct Gate {
    Tensor g, beta, A32, b32;
};

// (raw_gate, beta_logits, A_log, dt_bias) -> float32 log-decay g [B,T,H,K] and beta [B,T,H]
Gate run_gate(const Tensor& raw_gate, const Tensor& beta_logits, const Tensor& A_log, const Tensor& dt_bias, double lower_bound) {
    const int64_t B = raw_gate.size(0), T = raw_gate.size(1), H = raw_gate.size(2), K = raw_gate.size(3);
    Gate o;
    o.g = at::empty({B, T, H, K}, raw_gate.options().dtype(at::kFloat));
    o.beta = at::empty({B, T, H}, raw_gate.options().dtype(at::kFloat));
    o.A32 = A_log.contiguous().to(at::kFloat);
    o.b32 = dt_bias.contiguous().to(at::kFloat).reshape({-1});
    check(kda_gate_fwd((int32_t)(B * T), (int32_t)H, (int32_t)K, KDA_DTYPE_BF16, raw_gate.data_ptr(), beta_logits.data_ptr(),
                       o.A32.data_ptr<float>(), o.b32.data_ptr<float>(), (float)lower_bound, o.g.data_ptr<float>(),
                       o.beta.data_ptr<float>(), stream_of(raw_gate)),
          "kda_gate_fwd");
    return o;
}

KdaChunkShape chunk_shape(const Tensor& q, const Tensor& v, double scale) {
    KdaChunkShape sh;
    sh.n_seq = (int32_t)q.size(0);
    sh.seq_len = (int32_t)q.size(1);
    sh.tokens = (int32_t)(q.size(0) * q.size(1));
    sh.heads = (int32_t)q.size(2);
    sh.key_dim = (int32_t)q.size(3);
    sh.value_dim = (int32_t)v.size(3);
    sh.io_dtype = KDA_DTYPE_BF16;
    sh.gate_dtype = KDA_DTYPE_F32;
    sh.lane = (q.size(3) == 128 && v.size(3) == 128) ? KDA_LANE_TC : KDA_LANE_FP32;
    sh.l2norm = 1;
    sh.scale = (float)scale;
    return sh;
}

struct Forward {
    Tensor o, final_state, workspace;
    KdaChunkShape sh;
};

Forward run_chunk_forward(const Tensor& q, const Tensor& k, const Tensor& v, const Gate& gt, const OptTensor& h0, bool want_final,
                          double scale) {
    Forward f;
    f.sh = chunk_shape(q, v, scale);
    f.o = at::empty({q.size(0), q.size(1), q.size(2), v.size(3)}, v.options());
    if (want_final) f.final_state = at::empty({q.size(0), q.size(2), v.size(3), q.size(3)}, q.options().dtype(at::kFloat));
    const size_t nbytes = kda_chunk_workspace_bytes(&f.sh);
    f.workspace = bytes(nbytes, q);
    check(kda_chunk_fwd(&f.sh, q.data_ptr(), k.data_ptr(), v.data_ptr(), gt.g.data_ptr(), gt.beta.data_ptr(),
                        static_cast<const float*>(ptr(h0)), nullptr, f.o.data_ptr(),
                        want_final ? f.final_state.data_ptr<float>() : nullptr, f.workspace.data_ptr(), (size_t)f.workspace.numel(),
                        stream_of(q)),
          "kda_chunk_fwd");
    return f;
}

OptTensor contiguous_f32(const OptTensor& t) {
    if (!t.has_value() || !t->defined()) return c10::nullopt;
    return t->contiguous().to(at::kFloat);
}

// ------------------------------------------------------------------------------------------------ chunked operator
std::tuple<Tensor, OptTensor> chunk_forward(const Tensor& q_, const Tensor& k_, const Tensor& v_, const Tensor& raw_gate_,
                                            const Tensor& beta_logits_, const Tensor& A_log, const Tensor& dt_bias,
                                            const OptTensor& initial_state, bool output_final_state, double lower_bound, double scale) {
    need_bf16_cuda(q_, "q"); need_bf16_cuda(k_, "k"); need_bf16_cuda(v_, "v");
    need_bf16_cuda(raw_gate_, "raw_gate"); need_bf16_cuda(beta_logits_, "beta_logits");
    c10::cuda::CUDAGuard guard(q_.device());
    const Tensor q = q_.contiguous(), k = k_.contiguous(), v = v_.contiguous(), raw_gate = raw_gate_.contiguous(),
                 beta_logits = beta_logits_.contiguous();
    const Gate gt = run_gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound);
    const OptTensor h0 = contiguous_f32(initial_state);
    Forward f = run_chunk_forward(q, k, v, gt, h0, output_final_state, scale);
    return {f.o, output_final_state ? OptTensor(f.final_state) : OptTensor()};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, OptTensor> chunk_backward(
    const Tensor& q_, const Tensor& k_, const Tensor& v_, const Tensor& raw_gate_, const Tensor& beta_logits_, const Tensor& A_log,
    const Tensor& dt_bias, const OptTensor& initial_state, const Tensor& /*output*/, const OptTensor& /*final_state*/,
    const Tensor& grad_output, const OptTensor& grad_final_state, double lower_bound, double scale) {
    need_bf16_cuda(q_, "q"); need_bf16_cuda(k_, "k"); need_bf16_cuda(v_, "v");
    need_bf16_cuda(raw_gate_, "raw_gate"); need_bf16_cuda(beta_logits_, "beta_logits");
    c10::cuda::CUDAGuard guard(q_.device());
    const Tensor q = q_.contiguous(), k = k_.contiguous(), v = v_.contiguous(), raw_gate = raw_gate_.contiguous(),
                 beta_logits = beta_logits_.contiguous();
    const int64_t B = q.size(0), T = q.size(1), H = q.size(2), K = q.size(3);
    const Gate gt = run_gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound);
    const OptTensor h0 = contiguous_f32(initial_state);
    Forward f = run_chunk_forward(q, k, v, gt, h0, false, scale);
    const Tensor d_o = grad_output.contiguous().to(v.scalar_type());
    const OptTensor dfs = contiguous_f32(grad_final_state);
    Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
    Tensor dg = at::empty_like(gt.g), db = at::empty_like(gt.beta);
    OptTensor dh0;
    if (h0.has_value()) dh0 = at::empty({B, H, v.size(3), K}, q.options().dtype(at::kFloat));
    Tensor scratch = bytes(kda_chunk_bwd_scratch_bytes(&f.sh), q);
    check(kda_chunk_bwd(&f.sh, q.data_ptr(), k.data_ptr(), v.data_ptr(), gt.g.data_ptr(), gt.beta.data_ptr(), nullptr, d_o.data_ptr(),
                        static_cast<const float*>(ptr(dfs)), f.workspace.data_ptr(), (size_t)f.workspace.numel(), scratch.data_ptr(),
                        (size_t)scratch.numel(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), db.data_ptr(),
                        dh0.has_value() ? dh0->data_ptr<float>() : nullptr, stream_of(q)),
          "kda_chunk_bwd");
    Tensor d_raw = at::empty_like(raw_gate), d_bl = at::empty_like(beta_logits);
    Tensor dA = at::empty({H}, q.options().dtype(at::kFloat)), dbias = at::empty({H * K}, q.options().dtype(at::kFloat));
    Tensor gscr = bytes(kda_gate_bwd_scratch_bytes((int32_t)(B * T), (int32_t)H, (int32_t)K), q);
    check(kda_gate_bwd((int32_t)(B * T), (int32_t)H, (int32_t)K, KDA_DTYPE_BF16, raw_gate.data_ptr(), beta_logits.data_ptr(),
                       gt.A32.data_ptr<float>(), gt.b32.data_ptr<float>(), (float)lower_bound, dg.data_ptr<float>(),
                       db.data_ptr<float>(), d_raw.data_ptr(), d_bl.data_ptr(), dA.data_ptr<float>(), dbias.data_ptr<float>(),
                       gscr.data_ptr(), (size_t)gscr.numel(), stream_of(q)),
          "kda_gate_bwd");
    return {dq, dk, dv, d_raw, d_bl, dA.to(A_log.scalar_type()), dbias.reshape(dt_bias.sizes()).to(dt_bias.scalar_type()), dh0};
}

std::tuple<Tensor, OptTensor> recurrent_decode(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& raw_gate,
                                               const Tensor& beta_logits, const Tensor& A_log, const Tensor& dt_bias,
                                               const OptTensor& initial_state, bool output_final_state, double lower_bound,
                                               double scale) {
    need_bf16_cuda(q, "q"); need_bf16_cuda(k, "k"); need_bf16_cuda(v, "v");
    need_bf16_cuda(raw_gate, "raw_gate"); need_bf16_cuda(beta_logits, "beta_logits");
    TORCH_CHECK(q.size(1) == 1, "nanochat_kda::recurrent_decode takes one token per call");
    TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && raw_gate.is_contiguous() && beta_logits.is_contiguous(),
                "nanochat_kda::recurrent_decode requires contiguous tensors");
    c10::cuda::CUDAGuard guard(q.device());
    const int64_t B = q.size(0), H = q.size(2), K = q.size(3), V = v.size(3);
    const Gate gt = run_gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound);
    Tensor state = initial_state.has_value() && initial_state->defined() ? initial_state->contiguous().to(at::kFloat)
                                                                          : at::zeros({B, H, V, K}, q.options().dtype(at::kFloat));
    Tensor new_state = at::empty_like(state), o = at::empty_like(v);
    check(kda_decode_step((int32_t)B, (int32_t)H, (int32_t)K, (int32_t)V, KDA_DTYPE_BF16, KDA_DTYPE_F32, 1, (float)scale, q.data_ptr(),
                          k.data_ptr(), v.data_ptr(), gt.g.data_ptr(), gt.beta.data_ptr(), state.data_ptr<float>(),
                          new_state.data_ptr<float>(), o.data_ptr(), stream_of(q)),
          "kda_decode_step");
    return {o, output_final_state ? OptTensor(new_state) : OptTensor()};
}

// ------------------------------------------------------------------------------------------------ short convolution
int io_dtype_of(const Tensor& t) {
    TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, "nanochat_kda: float32 or bfloat16 tensors only");
    return t.scalar_type() == at::kBFloat16 ? KDA_DTYPE_BF16 : KDA_DTYPE_F32;
}

std::tuple<Tensor, OptTensor> causal_convolution_forward(const Tensor& x, const Tensor& weight, const OptTensor& initial_state,
                                                         bool output_final_state) {
    TORCH_CHECK(x.is_cuda(), "nanochat_kda: x must be a CUDA tensor");
    TORCH_CHECK(x.is_contiguous(), "nanochat_kda::causal_convolution_forward requires a contiguous input");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t B = x.size(0), T = x.size(1), C = x.size(2), W = weight.size(-1);
    const Tensor w = weight.contiguous().to(x.scalar_type());
    OptTensor s0;
    if (initial_state.has_value() && initial_state->defined()) s0 = initial_state->contiguous().to(x.scalar_type());
    Tensor y = at::empty_like(x);
    OptTensor fin;
    if (output_final_state) fin = at::empty({B, C, W}, x.options());
    check(kda_conv_fwd((int32_t)B, (int32_t)T, (int32_t)C, (int32_t)W, io_dtype_of(x), 1, x.data_ptr(), w.data_ptr(), ptr(s0), y.data_ptr(),
                       fin.has_value() ? fin->data_ptr() : nullptr, stream_of(x)),
          "kda_conv_fwd");
    return {y, fin};
}

std::tuple<Tensor, Tensor, OptTensor> causal_convolution_backward(const Tensor& x_, const Tensor& weight, const OptTensor& initial_state,
                                                                  const Tensor& /*output*/, const OptTensor& /*final_state*/,
                                                                  const Tensor& grad_output, const OptTensor& grad_final_state) {
    TORCH_CHECK(x_.is_cuda(), "nanochat_kda: x must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(x_.device());
    const Tensor x = x_.contiguous();
    const int64_t B = x.size(0), T = x.size(1), C = x.size(2), W = weight.size(-1);
    const Tensor w = weight.contiguous().to(x.scalar_type());
    OptTensor s0, dfin, dinit;
    if (initial_state.has_value() && initial_state->defined()) {
        s0 = initial_state->contiguous().to(x.scalar_type());
        dinit = at::empty_like(*s0);
    }
    if (grad_final_state.has_value() && grad_final_state->defined()) dfin = grad_final_state->contiguous().to(x.scalar_type());
    const Tensor dy = grad_output.contiguous().to(x.scalar_type());
    Tensor dx = at::empty_like(x), dw = at::empty({C, W}, x.options().dtype(at::kFloat));
    Tensor scratch = bytes(kda_conv_bwd_scratch_bytes((int32_t)B, (int32_t)T, (int32_t)C, (int32_t)W), x);
    check(kda_conv_bwd((int32_t)B, (int32_t)T, (int32_t)C, (int32_t)W, io_dtype_of(x), 1, x.data_ptr(), w.data_ptr(), ptr(s0), dy.data_ptr(),
                       ptr(dfin), dx.data_ptr(), dw.data_ptr<float>(), dinit.has_value() ? dinit->data_ptr() : nullptr, scratch.data_ptr(),
                       (size_t)scratch.numel(), stream_of(x)),
          "kda_conv_bwd");
    return {dx, dw.to(weight.scalar_type()), dinit};
}

// ------------------------------------------------------------------------------------------------ gated RMSNorm
std::tuple<Tensor, Tensor> rmsnorm_gate_forward(const Tensor& x_, const Tensor& gate_, const Tensor& weight, double epsilon) {
    TORCH_CHECK(x_.is_cuda(), "nanochat_kda: x must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(x_.device());
    const Tensor x = x_.contiguous(), gate = gate_.contiguous().to(x_.scalar_type()), w = weight.contiguous().to(at::kFloat);
    const int64_t D = x.size(-1), rows = x.numel() / D;
    Tensor y = at::empty_like(x), inv = at::empty({rows}, x.options().dtype(at::kFloat));
    check(kda_rmsnorm_gate_fwd(rows, (int32_t)D, io_dtype_of(x), (float)epsilon, x.data_ptr(), gate.data_ptr(), w.data_ptr<float>(),
                               y.data_ptr(), inv.data_ptr<float>(), stream_of(x)),
          "kda_rmsnorm_gate_fwd");
    return {y, inv};
}

std::tuple<Tensor, Tensor, Tensor> rmsnorm_gate_backward(const Tensor& x_, const Tensor& gate_, const Tensor& weight,
                                                         const Tensor& inverse_rms, const Tensor& grad_output, double /*epsilon*/) {
    TORCH_CHECK(x_.is_cuda(), "nanochat_kda: x must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(x_.device());
    const Tensor x = x_.contiguous(), gate = gate_.contiguous().to(x_.scalar_type()), w = weight.contiguous().to(at::kFloat);
    const Tensor inv = inverse_rms.contiguous(), dy = grad_output.contiguous().to(x_.scalar_type());
    const int64_t D = x.size(-1), rows = x.numel() / D;
    Tensor dx = at::empty_like(x), dgate = at::empty_like(gate), dw = at::empty({D}, x.options().dtype(at::kFloat));
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
          "Tensor? initial_state, bool output_final_state, float lower_bound, float scale) -> (Tensor, Tensor?)");
    m.def("chunk_backward(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
          "Tensor? initial_state, Tensor output, Tensor? final_state, Tensor grad_output, Tensor? grad_final_state, "
          "float lower_bound, float scale) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor?)");
    m.def("recurrent_decode(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
          "Tensor? initial_state, bool output_final_state, float lower_bound, float scale) -> (Tensor, Tensor?)");
    m.def("causal_convolution_forward(Tensor x, Tensor weight, Tensor? initial_state, bool output_final_state) -> (Tensor, Tensor?)");
    m.def("causal_convolution_backward(Tensor x, Tensor weight, Tensor? initial_state, Tensor output, Tensor? final_state, "
          "Tensor grad_output, Tensor? grad_final_state) -> (Tensor, Tensor, Tensor?)");
    m.def("rmsnorm_gate_forward(Tensor x, Tensor gate, Tensor weight, float epsilon) -> (Tensor, Tensor)");
    m.def("rmsnorm_gate_backward(Tensor x, Tensor gate, Tensor weight, Tensor inverse_rms, Tensor grad_output, float epsilon) "
          "-> (Tensor, Tensor, Tensor)");
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
