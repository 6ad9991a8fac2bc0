"""Host-side mirror of the reference's KDA mixer interface, routed to the B200 kernels.

Same names, argument meaning and error behaviour as nanochat/mixers/kda.py of the
reference (KDAState 23-35, RMSNormGated 46-59, ShortConvolution 123-212, k3_decay_gate
230-243, kda 561-673, KimiDeltaAttention 676-798) for the `project_chunk` /
`project_recurrent` modes, which is the path this package replaces.  There is no CPU or
PyTorch fallback: a call that cannot run on the CUDA kernels raises.

New surface beyond the reference: `chunk_kda` takes already-activated inputs
(q, k, v, per-channel log-decay g, beta, initial_state, output_final_state, cu_seqlens)
and packed variable-length batches.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, ops

Tensor = torch.Tensor

MODES = {"project_chunk", "project_recurrent"}


@dataclass
class KDAState:
    """Fixed-size decode state: memory V-first [B,H,V,K] float32; conv caches [B,D,W]
    holding the most recent projected inputs including the current token."""

    memory: Tensor
    q_conv: Tensor
    k_conv: Tensor
    v_conv: Tensor

    @staticmethod
    def zeros(batch: int, num_heads: int, head_dim: int, conv_size: int, device, dtype=torch.bfloat16) -> "KDAState":
        """An empty state a serving loop can own and hand to `KimiDeltaAttention.decode_token`, which updates it in place."""
        hid = num_heads * head_dim
        conv = lambda: torch.zeros(batch, hid, conv_size, device=device, dtype=dtype)
        return KDAState(torch.zeros(batch, num_heads, head_dim, head_dim, device=device, dtype=torch.float32), conv(), conv(), conv())

    def clone(self) -> "KDAState":
        return KDAState(self.memory.clone(), self.q_conv.clone(), self.k_conv.clone(), self.v_conv.clone())


def prepare_kda_backend(backend: str = "project_cuda") -> None:
    """Build (if stale) and load the CUDA library; fail early when it is unavailable."""
    if backend != "project_cuda":
        raise ValueError(f"unknown optimized KDA backend: {backend}")
    _lib.load()


def kda_backend_provenance() -> dict:
    """Operator binding table in the shape the reference consumes
    (nanochat/mixers/cuda_kda/__init__.py:59-132)."""
    import json
    import os
    from . import build

    receipt = {}
    if os.path.exists(build.RECEIPT):
        with open(build.RECEIPT) as f:
            receipt = json.load(f)
    comps = {}
    for name in ("chunk_forward", "chunk_backward", "recurrent_decode", "causal_convolution_forward",
                 "causal_convolution_backward", "rmsnorm_gate_forward", "rmsnorm_gate_backward"):
        comps[name] = {"owner": "project", "torch_operator": f"nanochat_kda::{name}"}
    return {"components": components_with_symbols(comps), "build": receipt, "target_arch": "sm_100a"}


def components_with_symbols(comps: dict) -> dict:
    sym = {"chunk_forward": ["kda_gate_fwd", "kda_chunk_fwd"], "chunk_backward": ["kda_chunk_bwd", "kda_gate_bwd"],
           "recurrent_decode": ["kda_gate_fwd", "kda_decode_step"], "causal_convolution_forward": ["kda_conv_fwd"],
           "causal_convolution_backward": ["kda_conv_bwd"], "rmsnorm_gate_forward": ["kda_rmsnorm_gate_fwd"],
           "rmsnorm_gate_backward": ["kda_rmsnorm_gate_bwd"]}
    for k, v in comps.items():
        v["c_abi"] = sym[k]
    return comps


# ------------------------------------------------------------------------------------------
# validation (same contracts and messages as the reference's protected checks)
# ------------------------------------------------------------------------------------------

def _gate_shapes(raw_gate: Tensor, A_log: Tensor, dt_bias: Tensor) -> Tuple[int, int]:
    if raw_gate.ndim != 4:
        raise ValueError("raw_gate must have shape [B, T, H, K]")
    heads, key_dim = raw_gate.shape[-2:]
    if tuple(A_log.shape) != (heads,):
        raise ValueError(f"A_log must have shape {(heads,)}")
    if dt_bias.numel() != heads * key_dim:
        raise ValueError(f"dt_bias must contain {heads * key_dim} values")
    return heads, key_dim


def _validate_operator_inputs(q, k, v, gate, beta, initial_state, n_states=None):
    if q.shape != k.shape or q.shape != gate.shape or q.ndim != 4:
        raise ValueError("q, k, and raw_gate must share shape [B, T, H, K]")
    if v.ndim != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError("v must have shape [B, T, H, V]")
    if beta.shape != q.shape[:3]:
        raise ValueError("beta logits must have shape [B, T, H]")
    batch, length, heads, key_dim = q.shape
    value_dim = v.shape[-1]
    if initial_state is not None:
        n = batch if n_states is None else n_states
        expected = (n, heads, value_dim, key_dim)
        if tuple(initial_state.shape) != expected:
            raise ValueError(f"initial_state must be V-first [B, H, V, K] with shape {expected}")
    return batch, length, heads, key_dim, value_dim


def _backend_reason(q, k, v, gate, beta, A_log, dt_bias, initial_state, *, lower_bound, allow_fp32=False):
    if not q.is_cuda:
        return "project KDA requires CUDA"
    acts = (q, k, v, gate, beta)
    params = tuple(t for t in (A_log, dt_bias) if t is not None)
    if any(t.device != q.device for t in (*acts, *params)):
        return "all KDA tensors must be on the same CUDA device"
    ok_dtypes = (torch.bfloat16, torch.float32) if allow_fp32 else (torch.bfloat16,)
    if any(t.dtype not in ok_dtypes for t in (q, k, v)) or len({q.dtype, k.dtype, v.dtype}) != 1:
        return "project KDA currently requires bfloat16 activations"
    if not allow_fp32 and any(t.dtype != torch.bfloat16 for t in (gate, beta)):
        return "project KDA currently requires bfloat16 activations"
    if any(t.dtype != torch.float32 for t in params):
        return "A_log and dt_bias must be float32"
    if q.shape[-1] > 256 or v.shape[-1] > 256:
        return "project KDA supports head dimensions up to 256"
    if not (-5.0 <= lower_bound < 0.0):
        return "safe-gate lower_bound must be in [-5, 0)"
    if initial_state is not None:
        if initial_state.device != q.device:
            return "initial_state must be on the same CUDA device as q"
        if initial_state.dtype != torch.float32:
            return "initial_state must be float32"
    return None


def k3_decay_gate(raw_gate: Tensor, A_log: Tensor, dt_bias: Tensor, lower_bound: float = -5.0) -> Tensor:
    """K3 lower-bounded log decay lb * sigmoid(exp(A) * (z + b)), computed by the CUDA gate kernel."""
    _gate_shapes(raw_gate, A_log, dt_bias)
    if lower_bound >= 0:
        raise ValueError("lower_bound must be negative")
    beta_dummy = raw_gate.new_zeros(raw_gate.shape[:3])
    g, _ = ops.GateFunction.apply(raw_gate, beta_dummy, A_log, dt_bias, float(lower_bound))
    return g


# ------------------------------------------------------------------------------------------
# operators
# ------------------------------------------------------------------------------------------

def chunk_kda(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, *, initial_state: Optional[Tensor] = None,
              output_final_state: bool = False, cu_seqlens: Optional[Tensor] = None, scale: Optional[float] = None,
              use_qk_l2norm: bool = True, lane: str = "auto") -> Tuple[Tensor, Optional[Tensor]]:
    """Exact chunked KDA on activated inputs with autograd.

    q, k, g [B,T,H,K]; v [B,T,H,V]; beta [B,T,H]; g is the per-channel log-decay (<= 0).
    initial_state / final state are V-first [N,H,V,K] float32 with N = B, or the number of
    packed segments when cu_seqlens (int32 [N+1], B must be 1) is given.
    q,k,v share one dtype (float32 or bfloat16); g, beta share one dtype.

    Range of g: the tensor-core lane (lane="tc", and "auto" for bfloat16 with K = V = 128) forms its decay factors
    exp(+-(G - c)) in bfloat16 around a reference c per 16-token block, which is in range for g in [-5, 0] per token -
    the range the reference's gate produces (k3_decay_gate with lower_bound >= -5).  Pass lane="fp32" for log-decays
    below -5 per token.

    When gradients are disabled, or no input requires one, the call is a prefill: the kernels skip every panel that
    only a backward would read and no workspace outlives the call.
    """
    n_states = None
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError("packed inputs (cu_seqlens) require batch size 1")
        if cu_seqlens.dtype != torch.int32 or cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
            raise ValueError("cu_seqlens must be int32 [N+1]")
        n_states = cu_seqlens.numel() - 1
    _validate_operator_inputs(q, k, v, g, beta, initial_state, n_states)
    reason = _backend_reason(q, k, v, g, beta, None, None, initial_state, lower_bound=-1.0, allow_fp32=True)
    if reason is None and g.dtype != beta.dtype:
        reason = "g and beta must share a dtype"
    if reason is not None:
        raise RuntimeError(f"project CUDA KDA backend unavailable: {reason}")
    sc = float(q.shape[-1] ** -0.5 if scale is None else scale)
    lane_id = _select_lane(lane, q, v)
    cu = None if cu_seqlens is None else cu_seqlens.contiguous()
    return _chunk_dispatch(q, k, v, g, beta, initial_state, bool(output_final_state), cu, sc, bool(use_qk_l2norm), lane_id)


def _chunk_dispatch(q, k, v, g, beta, initial_state, output_final_state, cu, scale, l2norm, lane_id):
    """Training calls go through the autograd Function (workspace kept for the backward); calls that cannot need a
    backward take the forward-only kernels' path (the reference sends those to its token loop, chunk.cu:1694-1698)."""
    tracked = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state))
    if tracked:
        return ops.ChunkKDAFunction.apply(q, k, v, g, beta, initial_state, output_final_state, cu, scale, l2norm, lane_id)
    q, k, v, g, beta = (t.detach().contiguous() for t in (q, k, v, g, beta))
    h0 = None if initial_state is None else initial_state.detach().contiguous()
    o, fs, _ = ops.chunk_kda_fwd(q, k, v, g, beta, h0, cu, scale, l2norm, output_final_state, lane_id, forward_only=True)
    return o, fs


def chunk_kda_norm(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, gate: Tensor, norm_weight: Tensor, *,
                   eps: float = 1e-5, initial_state: Optional[Tensor] = None, output_final_state: bool = False,
                   cu_seqlens: Optional[Tensor] = None, scale: Optional[float] = None,
                   use_qk_l2norm: bool = True) -> Tuple[Tensor, Optional[Tensor]]:
    """`RMSNormGated(chunk_kda(q, k, v, g, beta), gate)` with the norm applied inside the chunk-output kernel.

    Same results as the two operators in sequence (bit for bit in the forward), one launch and one read of the output
    less.  Needs the tensor-core lane: bfloat16 activations and K = V = 128; anything else raises.  gate [B,T,H,V];
    norm_weight [V]."""
    n_states = None
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError("packed inputs (cu_seqlens) require batch size 1")
        if cu_seqlens.dtype != torch.int32 or cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
            raise ValueError("cu_seqlens must be int32 [N+1]")
        n_states = cu_seqlens.numel() - 1
    _validate_operator_inputs(q, k, v, g, beta, initial_state, n_states)
    if gate.shape != v.shape:
        raise ValueError("gate must have the shape of v")
    if tuple(norm_weight.shape) != (v.shape[-1],):
        raise ValueError(f"norm_weight must have shape {(v.shape[-1],)}")
    reason = _backend_reason(q, k, v, g, beta, None, None, initial_state, lower_bound=-1.0, allow_fp32=True)
    if reason is None and g.dtype != beta.dtype:
        reason = "g and beta must share a dtype"
    if reason is None and not (q.dtype == torch.bfloat16 and q.shape[-1] == 128 and v.shape[-1] == 128):
        reason = "the fused output norm needs the tensor-core lane (bfloat16, K = V = 128)"
    if reason is None and (gate.device != q.device or norm_weight.device != q.device):
        reason = "all KDA tensors must be on the same CUDA device"
    if reason is not None:
        raise RuntimeError(f"project CUDA KDA backend unavailable: {reason}")
    sc = float(q.shape[-1] ** -0.5 if scale is None else scale)
    cu = None if cu_seqlens is None else cu_seqlens.contiguous()
    return ops.ChunkKDANormFunction.apply(q, k, v, g, beta, gate, norm_weight, initial_state, bool(output_final_state), cu, sc,
                                          bool(use_qk_l2norm), float(eps))


def _select_lane(lane: str, q: Tensor, v: Tensor) -> int:
    """"tc": tcgen05 tensor-core tiles (128-wide heads, bf16 activations); "fp32": CUDA-core float32
    arithmetic for any head size up to 256; "auto": tc whenever the shape allows it."""
    tc_ok = q.dtype == torch.bfloat16 and q.shape[-1] == 128 and v.shape[-1] == 128
    if lane == "auto":
        return _lib.LANE_TC if tc_ok else _lib.LANE_FP32
    if lane == "fp32":
        return _lib.LANE_FP32
    if lane == "tc":
        if not tc_ok:
            raise RuntimeError("project CUDA KDA backend unavailable: the tensor-core lane needs bfloat16 and K = V = 128")
        return _lib.LANE_TC
    raise ValueError(f"unknown lane: {lane}")


def recurrent_kda_step(q, k, v, g, beta, state, *, scale=None, use_qk_l2norm=True):
    """One decode token on activated inputs; returns (o, new_state); `state` is not modified."""
    sc = float(q.shape[-1] ** -0.5 if scale is None else scale)
    return ops.decode_step(q, k, v, g, beta, state, sc, use_qk_l2norm)


def kda(q: Tensor, k: Tensor, v: Tensor, raw_gate: Tensor, beta_logits: Tensor, A_log: Tensor, dt_bias: Tensor, *,
        initial_state: Optional[Tensor] = None, output_final_state: bool = False, mode: str = "project_chunk",
        lower_bound: float = -5.0, scale: Optional[float] = None, allow_fallback: bool = False,
        cu_seqlens: Optional[Tensor] = None, lane: str = "auto") -> Tuple[Tensor, Optional[Tensor]]:
    """Raw-input KDA operator (L2 norm, gate and beta sigmoid fused), reference signature.

    Only the project modes exist here; anything else raises (fail closed)."""
    if mode not in MODES:
        raise ValueError(f"unknown KDA mode: {mode}")
    n_states = None if cu_seqlens is None else cu_seqlens.numel() - 1
    _validate_operator_inputs(q, k, v, raw_gate, beta_logits, initial_state, n_states)
    _gate_shapes(raw_gate, A_log, dt_bias)
    reason = _backend_reason(q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state, lower_bound=lower_bound)
    if mode == "project_recurrent" and torch.is_grad_enabled() and any(
            t.requires_grad for t in (q, k, v, raw_gate, beta_logits, A_log, dt_bias)):
        reason = "project recurrent KDA is inference-only"
    if reason is not None:
        raise RuntimeError(f"project CUDA KDA backend unavailable: {reason}")
    sc = float(scale if scale is not None else q.shape[-1] ** -0.5)
    g, beta = ops.GateFunction.apply(raw_gate, beta_logits, A_log, dt_bias, float(lower_bound))
    if mode == "project_recurrent":
        if q.shape[1] != 1:
            raise RuntimeError("project CUDA KDA backend unavailable: recurrent decode takes one token per call")
        state = initial_state
        if state is None:
            state = torch.zeros(q.shape[0], q.shape[2], v.shape[3], q.shape[3], dtype=torch.float32, device=q.device)
        o, new_state = ops.decode_step(q, k, v, g, beta, state.contiguous(), sc, True)
        return o, (new_state if output_final_state else None)
    cu = None if cu_seqlens is None else cu_seqlens.contiguous()
    return _chunk_dispatch(q, k, v, g, beta, initial_state, bool(output_final_state), cu, sc, True, _select_lane(lane, q, v))


# ------------------------------------------------------------------------------------------
# modules
# ------------------------------------------------------------------------------------------

class Linear(nn.Linear):
    """FP32 master weights, matmul in the activation dtype (cuBLAS; not part of this package's kernels)."""

    def forward(self, x: Tensor) -> Tensor:
        bias = None if self.bias is None else self.bias.to(dtype=x.dtype)
        return F.linear(x, self.weight.to(dtype=x.dtype), bias)


class RMSNormGated(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: Tensor, gate: Tensor) -> Tensor:
        if not x.is_cuda:
            raise RuntimeError("project CUDA gated RMSNorm cannot fall back on CPU")
        return ops.RMSNormGateFunction.apply(x, gate, self.weight, self.eps)


class ShortConvolution(nn.Conv1d):
    """Depthwise causal convolution + SiLU with explicit, non-mutating cache state."""

    def __init__(self, hidden_size: int, kernel_size: int = 4):
        super().__init__(hidden_size, hidden_size, kernel_size, groups=hidden_size, bias=False, padding=kernel_size - 1)

    def forward(self, x: Tensor, state: Optional[Tensor] = None, *, output_final_state: bool = False,
                backend: str = "project_cuda") -> Tuple[Tensor, Optional[Tensor]]:
        if x.ndim != 3 or x.shape[-1] != self.in_channels:
            raise ValueError(f"x must have shape [B,T,{self.in_channels}]")
        batch, length, channels = x.shape
        width = self.kernel_size[0]
        if state is not None:
            expected = (batch, channels, width)
            if tuple(state.shape) != expected:
                raise ValueError(f"convolution state must have shape {expected}")
        if backend != "project_cuda":
            raise ValueError(f"unknown CUDA short-convolution backend: {backend}")
        if not x.is_cuda:
            raise RuntimeError("project CUDA causal convolution cannot fall back on CPU")
        if length == 0:
            cur = x.new_zeros(batch, channels, width) if state is None else state.to(x.dtype).clone()
            return x.new_empty(batch, 0, channels), (cur if output_final_state else None)
        return ops.ConvFunction.apply(x, self.weight.squeeze(1), state, output_final_state, True)


def short_convolutions(convs, xs):
    """Run several same-shaped `ShortConvolution`s (the q, k and v branches of a layer) as one launch each way.

    Training path only: no cache in, no final state out.  Returns the list of outputs; results are identical to calling
    the modules one by one (the same kernel runs over an extra grid dimension)."""
    convs, xs = list(convs), list(xs)
    if len(convs) != len(xs) or not convs:
        raise ValueError("short_convolutions needs one input per convolution")
    for conv, x in zip(convs, xs):
        if x.ndim != 3 or x.shape[-1] != conv.in_channels:
            raise ValueError(f"x must have shape [B,T,{conv.in_channels}]")
        if not x.is_cuda:
            raise RuntimeError("project CUDA causal convolution cannot fall back on CPU")
    if len(convs) > 4 or xs[0].shape[1] == 0:
        return [conv(x)[0] for conv, x in zip(convs, xs)]
    return list(ops.ConvMultiFunction.apply(True, len(convs), *xs, *[c.weight.squeeze(1) for c in convs]))


class KimiDeltaAttention(nn.Module):
    """K3-compatible KDA mixer: q/k/v projections -> short conv -> KDA -> gated RMSNorm -> o_proj."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, conv_size: int = 4,
                 layer_idx: Optional[int] = None, mode: str = "project_chunk", norm_eps: float = 1e-5,
                 lower_bound: float = -5.0, allow_fallback: bool = False):
        super().__init__()
        if hidden_size != num_heads * head_dim:
            raise ValueError("initial KDA implementation requires hidden_size = num_heads * head_dim")
        if conv_size <= 0:
            raise ValueError("conv_size must be positive")
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.conv_size, self.layer_idx, self.mode = conv_size, layer_idx, mode
        self.fuse_prefill_conv = False      # see forward(): convolutions inside the intra-chunk kernel for no-grad prefill
        self.lower_bound, self.allow_fallback = lower_bound, allow_fallback
        self.q_proj = Linear(hidden_size, hidden_size, bias=False)
        self.k_proj = Linear(hidden_size, hidden_size, bias=False)
        self.v_proj = Linear(hidden_size, hidden_size, bias=False)
        self.q_conv1d = ShortConvolution(hidden_size, conv_size)
        self.k_conv1d = ShortConvolution(hidden_size, conv_size)
        self.v_conv1d = ShortConvolution(hidden_size, conv_size)
        self.A_log = nn.Parameter(torch.zeros(num_heads, dtype=torch.float32))
        self.f_a_proj = Linear(hidden_size, head_dim, bias=False)
        self.f_b_proj = Linear(head_dim, hidden_size, bias=False)
        self.dt_bias = nn.Parameter(torch.zeros(hidden_size, dtype=torch.float32))
        self.b_proj = Linear(hidden_size, num_heads, bias=False)
        self.g_proj = Linear(hidden_size, hidden_size, bias=False)
        self.o_norm = RMSNormGated(head_dim, eps=norm_eps)
        self.o_proj = Linear(hidden_size, hidden_size, bias=False)

    def forward(self, hidden_states: Tensor, state: Optional[KDAState] = None, output_final_state: bool = False,
                mode: Optional[str] = None, allow_fallback: Optional[bool] = None):
        if hidden_states.ndim != 3 or hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(f"hidden_states must have shape [B,T,{self.hidden_size}]")
        batch, length, _ = hidden_states.shape
        requested_mode = self.mode if mode is None else mode
        want_state = output_final_state
        q_state = None if state is None else state.q_conv
        k_state = None if state is None else state.k_conv
        v_state = None if state is None else state.v_conv
        memory = None if state is None else state.memory
        if (self.fuse_prefill_conv and state is None and length > 0 and requested_mode == "project_chunk"
                and not torch.is_grad_enabled() and hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16
                and self.head_dim == 128 and self.conv_size == 4):
            # opt-in no-grad prefill at the tensor-core lane's shape: the three convolutions run inside the intra-chunk
            # kernel, so q, k, v are never written to memory (3 x T x hidden_size x 2 bytes less per layer); identical
            # results.  Measured 3 % slower than the separate convolution launch (the intra-chunk kernel is bound by
            # instruction issue, the convolution by bandwidth), hence off by default.
            return self._prefill_fused(hidden_states, want_state)
        if state is None and not want_state and length > 0:
            # training path: the three branches share one launch each way
            q, k, v = short_convolutions((self.q_conv1d, self.k_conv1d, self.v_conv1d),
                                         (self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)))
            q_final = k_final = v_final = None
        else:
            q, q_final = self.q_conv1d(self.q_proj(hidden_states), q_state, output_final_state=want_state)
            k, k_final = self.k_conv1d(self.k_proj(hidden_states), k_state, output_final_state=want_state)
            v, v_final = self.v_conv1d(self.v_proj(hidden_states), v_state, output_final_state=want_state)
        shape4 = (batch, length, self.num_heads, self.head_dim)
        q, k, v = q.reshape(shape4), k.reshape(shape4), v.reshape(shape4)
        raw_gate = self.f_b_proj(self.f_a_proj(hidden_states)).reshape(shape4)
        beta_logits = self.b_proj(hidden_states)
        output_gate = self.g_proj(hidden_states).reshape(shape4)
        fuse_norm = (requested_mode == "project_chunk" and length > 0 and q.is_cuda and q.dtype == torch.bfloat16
                     and self.head_dim == 128 and torch.is_grad_enabled())
        if fuse_norm:
            # training path at the tensor-core lane's shape: gate activations, then chunked KDA with the output norm in
            # the chunk-output kernel's epilogue
            _validate_operator_inputs(q, k, v, raw_gate, beta_logits, memory)
            g, beta = ops.GateFunction.apply(raw_gate, beta_logits, self.A_log, self.dt_bias, float(self.lower_bound))
            mixed, final_memory = chunk_kda_norm(q, k, v, g, beta, output_gate, self.o_norm.weight, eps=self.o_norm.eps,
                                                 initial_state=memory, output_final_state=want_state)
        else:
            mixed, final_memory = kda(q, k, v, raw_gate, beta_logits, self.A_log, self.dt_bias, initial_state=memory,
                                      output_final_state=want_state, mode=requested_mode, lower_bound=self.lower_bound)
            mixed = self.o_norm(mixed, output_gate)
        output = self.o_proj(mixed.reshape(batch, length, self.hidden_size))
        final_state = KDAState(final_memory, q_final, k_final, v_final) if want_state else None
        return output, final_state

    def _prefill_fused(self, hidden_states: Tensor, want_state: bool):
        batch, length, _ = hidden_states.shape
        shape4 = (batch, length, self.num_heads, self.head_dim)
        xq, xk, xv = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
        raw_gate = self.f_b_proj(self.f_a_proj(hidden_states)).reshape(shape4)
        beta_logits = self.b_proj(hidden_states)
        g, beta = ops.GateFunction.apply(raw_gate, beta_logits, self.A_log, self.dt_bias, float(self.lower_bound))
        conv_w = [c.weight.squeeze(1) for c in (self.q_conv1d, self.k_conv1d, self.v_conv1d)]
        mixed, memory = ops.chunk_kda_conv_fwd(xq.reshape(shape4), xk.reshape(shape4), xv.reshape(shape4), *conv_w, g, beta, None, None,
                                               self.head_dim ** -0.5, True, want_state)
        mixed = self.o_norm(mixed, self.g_proj(hidden_states).reshape(shape4))
        output = self.o_proj(mixed.reshape(batch, length, self.hidden_size))
        if not want_state:
            return output, None

        def cache(x):      # [B, C, W]: the last W inputs, the current token included, zero-padded on the left
            tail = x[:, max(0, length - self.conv_size):, :]
            if length < self.conv_size:
                tail = torch.nn.functional.pad(tail, (0, 0, self.conv_size - length, 0))
            return tail.transpose(1, 2).contiguous()

        return output, KDAState(memory, cache(xq), cache(xk), cache(xv))

    @torch.no_grad()
    def decode_token(self, hidden_states: Tensor, state: KDAState) -> Tensor:
        """One decode token with the state updated IN PLACE (inference only).

        The non-mutating contract of `forward(..., state, output_final_state=True, mode="project_recurrent")` costs a
        serving loop six library launches and four freshly allocated state tensors per layer and token (the reference's
        cache plumbing: nanochat/engine.py:83-226, get/set_kda_state :160-170).  Here the caller owns one `KDAState`
        (see `KDAState.zeros`); the three convolution caches are advanced by one fused launch, the gate and beta
        activations run inside the decode kernel, and the memory is rewritten where it lies: three library launches, no
        state allocation.  Same arithmetic, same results as the non-mutating path."""
        if hidden_states.ndim != 3 or hidden_states.shape[1] != 1 or hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(f"hidden_states must have shape [B,1,{self.hidden_size}]")
        if not hidden_states.is_cuda:
            raise RuntimeError("project CUDA KDA backend unavailable: project KDA requires CUDA")
        batch = hidden_states.shape[0]
        x = hidden_states
        conv_w = [c.weight.squeeze(1) for c in (self.q_conv1d, self.k_conv1d, self.v_conv1d)]
        q, k, v = ops.conv_step_multi((self.q_proj(x), self.k_proj(x), self.v_proj(x)), conv_w,
                                      (state.q_conv, state.k_conv, state.v_conv))
        shape4 = (batch, 1, self.num_heads, self.head_dim)
        raw_gate = self.f_b_proj(self.f_a_proj(x)).reshape(shape4)
        beta_logits = self.b_proj(x)
        o, _ = ops.decode_step_raw(q.reshape(shape4), k.reshape(shape4), v.reshape(shape4), raw_gate, beta_logits, self.A_log,
                                   self.dt_bias, self.lower_bound, state.memory, self.head_dim ** -0.5, out_state=state.memory)
        mixed = self.o_norm(o, self.g_proj(x).reshape(shape4))
        return self.o_proj(mixed.reshape(batch, 1, self.hidden_size))


__all__ = ["KDAState", "KimiDeltaAttention", "RMSNormGated", "ShortConvolution", "chunk_kda", "chunk_kda_norm", "k3_decay_gate", "kda",
           "kda_backend_provenance", "prepare_kda_backend", "recurrent_kda_step", "short_convolutions"]
