"""`torch.ops.nanochat_kda.*`: the seven operators the reference mixer calls, bound to libkda_b200.

Schemas are the reference's, verbatim (nanochat/mixers/cuda_kda/chunk.cu:2118-2128, recurrent_decode.cu:186-189,
causal_convolution_forward.cu:242-243, causal_convolution_backward.cu:456-459, rmsnorm_gate.cu:278-282), so
nanochat/mixers/kda.py (`_project_operator`, the three autograd.Functions at 383-466 and the direct rmsnorm /
recurrent_decode calls) routes to these kernels unchanged once `register()` has run and its provenance table
(`experiment_swa_kda_b200.kda_backend_provenance()`) is returned by the loader.

`chunk_backward` receives only the inputs and the forward output (the reference's fixed ABI), so it re-runs the
gate and the chunked forward into a fresh workspace before the backward kernels.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops

_LIB = None
_SCHEMAS = {
    "chunk_forward": "(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
                     "Tensor? initial_state, bool output_final_state, float lower_bound, float scale) -> (Tensor, Tensor?)",
    "chunk_backward": "(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
                      "Tensor? initial_state, Tensor output, Tensor? final_state, Tensor grad_output, Tensor? grad_final_state, "
                      "float lower_bound, float scale) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor?)",
    "recurrent_decode": "(Tensor q, Tensor k, Tensor v, Tensor raw_gate, Tensor beta_logits, Tensor A_log, Tensor dt_bias, "
                        "Tensor? initial_state, bool output_final_state, float lower_bound, float scale) -> (Tensor, Tensor?)",
    "causal_convolution_forward": "(Tensor x, Tensor weight, Tensor? initial_state, bool output_final_state) -> (Tensor, Tensor?)",
    "causal_convolution_backward": "(Tensor x, Tensor weight, Tensor? initial_state, Tensor output, Tensor? final_state, "
                                   "Tensor grad_output, Tensor? grad_final_state) -> (Tensor, Tensor, Tensor?)",
    "rmsnorm_gate_forward": "(Tensor x, Tensor gate, Tensor weight, float epsilon) -> (Tensor, Tensor)",
    "rmsnorm_gate_backward": "(Tensor x, Tensor gate, Tensor weight, Tensor inverse_rms, Tensor grad_output, float epsilon) "
                             "-> (Tensor, Tensor, Tensor)",
}


def _check_activations(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("nanochat_kda operators require CUDA tensors")
        if t.dtype != torch.bfloat16:
            raise RuntimeError("nanochat_kda operators require bfloat16 activations")


def _lane(q, v):
    return _lib.LANE_TC if (q.shape[-1] == 128 and v.shape[-1] == 128) else _lib.LANE_FP32


def _gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound):
    lib = _lib.load()
    B, T, H, K = raw_gate.shape
    dev = raw_gate.device
    g = torch.empty(B, T, H, K, dtype=torch.float32, device=dev)
    beta = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    A32, b32 = A_log.contiguous().float(), dt_bias.contiguous().float().reshape(-1)
    with torch.cuda.device(dev):
        rc = lib.kda_gate_fwd(B * T, H, K, _lib.DTYPE_BF16, raw_gate.data_ptr(), beta_logits.data_ptr(), A32.data_ptr(),
                              b32.data_ptr(), float(lower_bound), g.data_ptr(), beta.data_ptr(),
                              torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "kda_gate_fwd")
    return g, beta, A32, b32


def chunk_forward(q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state, output_final_state, lower_bound, scale):
    _check_activations(q, k, v, raw_gate, beta_logits)
    q, k, v, raw_gate, beta_logits = (t.contiguous() for t in (q, k, v, raw_gate, beta_logits))
    g, beta, _, _ = _gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound)
    h0 = None if initial_state is None else initial_state.contiguous()
    o, fs, _ = ops.chunk_kda_fwd(q, k, v, g, beta, h0, None, float(scale), True, bool(output_final_state), _lane(q, v))
    return o, fs


def chunk_backward(q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state, output, final_state, grad_output,
                   grad_final_state, lower_bound, scale):
    _check_activations(q, k, v, raw_gate, beta_logits)
    lib = _lib.load()
    q, k, v, raw_gate, beta_logits = (t.contiguous() for t in (q, k, v, raw_gate, beta_logits))
    dev = q.device
    g, beta, A32, b32 = _gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound)
    h0 = None if initial_state is None else initial_state.contiguous()
    _, _, saved = ops.chunk_kda_fwd(q, k, v, g, beta, h0, None, float(scale), True, False, _lane(q, v))
    dfs = None if grad_final_state is None else grad_final_state.contiguous().float()
    dq, dk, dv, dg, db, dh0 = ops.chunk_kda_bwd(q, k, v, g, beta, None, grad_output.contiguous().to(v.dtype), dfs, saved,
                                                initial_state is not None)
    B, T, H, K = q.shape
    d_raw, d_bl = torch.empty_like(raw_gate), torch.empty_like(beta_logits)
    dA = torch.empty(H, dtype=torch.float32, device=dev)
    dbias = torch.empty(H * K, dtype=torch.float32, device=dev)
    scr = torch.empty(max(lib.kda_gate_bwd_scratch_bytes(B * T, H, K), 256), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.kda_gate_bwd(B * T, H, K, _lib.DTYPE_BF16, raw_gate.data_ptr(), beta_logits.data_ptr(), A32.data_ptr(),
                              b32.data_ptr(), float(lower_bound), dg.data_ptr(), db.data_ptr(), d_raw.data_ptr(),
                              d_bl.data_ptr(), dA.data_ptr(), dbias.data_ptr(), scr.data_ptr(), scr.numel(),
                              torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "kda_gate_bwd")
    return dq, dk, dv, d_raw, d_bl, dA.to(A_log.dtype), dbias.reshape(dt_bias.shape).to(dt_bias.dtype), dh0


def recurrent_decode(q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state, output_final_state, lower_bound, scale):
    _check_activations(q, k, v, raw_gate, beta_logits)
    if q.shape[1] != 1:
        raise RuntimeError("nanochat_kda::recurrent_decode takes one token per call")
    for t in (q, k, v, raw_gate, beta_logits):
        if not t.is_contiguous():
            raise RuntimeError("nanochat_kda::recurrent_decode requires contiguous tensors")
    g, beta, _, _ = _gate(raw_gate, beta_logits, A_log, dt_bias, lower_bound)
    state = initial_state
    if state is None:
        state = torch.zeros(q.shape[0], q.shape[2], v.shape[3], q.shape[3], dtype=torch.float32, device=q.device)
    o, new_state = ops.decode_step(q, k, v, g, beta, state.contiguous(), float(scale), True)
    return o, (new_state if output_final_state else None)


def causal_convolution_forward(x, weight, initial_state, output_final_state):
    if not x.is_contiguous():
        raise RuntimeError("nanochat_kda::causal_convolution_forward requires a contiguous input")
    w = weight.contiguous().to(x.dtype)
    s0 = None if initial_state is None else initial_state.contiguous().to(x.dtype)
    return ops.conv_fwd(x, w, s0, bool(output_final_state), True)


def causal_convolution_backward(x, weight, initial_state, output, final_state, grad_output, grad_final_state):
    w = weight.contiguous().to(x.dtype)
    s0 = None if initial_state is None else initial_state.contiguous().to(x.dtype)
    dfin = None if grad_final_state is None else grad_final_state.contiguous().to(x.dtype)
    dx, dw, dinit = ops.conv_bwd(x.contiguous(), w, s0, grad_output.contiguous().to(x.dtype), dfin, True)
    return dx, dw.to(weight.dtype), dinit


def rmsnorm_gate_forward(x, gate, weight, epsilon):
    return ops.rmsnorm_gate_fwd(x.contiguous(), gate.contiguous().to(x.dtype), weight.contiguous().float(), float(epsilon))


def rmsnorm_gate_backward(x, gate, weight, inverse_rms, grad_output, epsilon):
    dx, dgate, dw = ops.rmsnorm_gate_bwd(x.contiguous(), gate.contiguous().to(x.dtype), weight.contiguous().float(),
                                         inverse_rms.contiguous(), grad_output.contiguous().to(x.dtype))
    return dx, dgate, dw.to(weight.dtype)


_IMPLS = {
    "chunk_forward": chunk_forward, "chunk_backward": chunk_backward, "recurrent_decode": recurrent_decode,
    "causal_convolution_forward": causal_convolution_forward, "causal_convolution_backward": causal_convolution_backward,
    "rmsnorm_gate_forward": rmsnorm_gate_forward, "rmsnorm_gate_backward": rmsnorm_gate_backward,
}


def schemas() -> dict:
    return dict(_SCHEMAS)


def register() -> None:
    """Define the `nanochat_kda` namespace (once per process) and bind the CUDA implementations."""
    global _LIB
    if _LIB is not None:
        return
    lib = torch.library.Library("nanochat_kda", "DEF")
    for name, schema in _SCHEMAS.items():
        lib.define(name + schema)
        lib.impl(name, _IMPLS[name], "CUDA")
    _LIB = lib
