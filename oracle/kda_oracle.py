"""CPU oracle for the Kimi Delta Attention (KDA) hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
it is the checker used by the tests, by the smoke entry and by the CPU-baseline
leg of the benchmark.  It is a from-scratch restatement, in plain PyTorch on
the CPU, of the algorithm that the reference pins in its own independent oracle:

* gate parameterisation ............ reference tests/kda_oracle.py:31-47
* token recurrence (decay first) .... reference tests/kda_oracle.py:50-127
* causal depthwise conv + cache ..... reference tests/kda_oracle.py:130-161
* gated RMSNorm .................... reference tests/kda_oracle.py:164-173

Parity pin: tests/golden/*.npz were produced by running the reference's own
oracle (imported by path) and the reference's CPU production loop
(nanochat/mixers/kda.py:269-327) on seeded inputs; tests/test_oracle_golden.py
checks this restatement against those vectors and against the reference's
closed-form known answers (tests/test_kda_operator.py:62-137).

Conventions
-----------
q, k, g : [B, T, H, K]      v, o : [B, T, H, V]      beta : [B, T, H]
memory state (public)  : V-first  [B, H, V, K], float32
packed / varlen        : B == 1 with cu_seqlens int [N+1]; state [N, H, V, K]
Per token:  S <- S * exp(g_t)[:, None];  r = v_t - k_t^T S;
            S <- S + (beta_t k_t) r^T;   o_t = (scale * q_t)^T S
with q_t, k_t L2-normalised over K when ``l2norm`` is set (the reference always
normalises, tests/kda_oracle.py:83-84).
"""

from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------

def decay_gate(raw_gate: Tensor, A_log: Tensor, dt_bias: Tensor, lower_bound: float = -5.0) -> Tensor:
    """g = lower_bound * sigmoid(exp(A_log)[h] * (raw + dt_bias[h, k])).

    Follows reference tests/kda_oracle.py:31-47 (same formula as
    nanochat/mixers/kda.py:230-243).
    """
    if raw_gate.dim() != 4:
        raise ValueError("raw_gate must have shape [B, T, H, K]")
    H, K = raw_gate.shape[2], raw_gate.shape[3]
    if tuple(A_log.shape) != (H,):
        raise ValueError(f"A_log must have shape {(H,)}")
    if dt_bias.numel() != H * K:
        raise ValueError(f"dt_bias must contain {H * K} values")
    rate = torch.exp(A_log).view(1, 1, H, 1)
    return lower_bound * torch.sigmoid(rate * (raw_gate + dt_bias.reshape(1, 1, H, K)))


def invert_decay_gate(g: Tensor, lower_bound: float = -5.0) -> Tensor:
    """raw_gate such that decay_gate(raw, A_log=0, dt_bias=0) == g (test helper)."""
    p = (g / lower_bound).clamp(1e-7, 1 - 1e-7)
    return torch.log(p) - torch.log1p(-p)


def _unit(x: Tensor, eps: float = 1e-12) -> Tensor:
    # same guard as torch.nn.functional.normalize: x / max(||x||, eps)
    return x / x.norm(dim=-1, keepdim=True).clamp_min(eps)


# --------------------------------------------------------------------------
# core recurrence on activated inputs
# --------------------------------------------------------------------------

def kda_recurrence(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    g: Tensor,
    beta: Tensor,
    *,
    initial_state: Optional[Tensor] = None,
    scale: Optional[float] = None,
    l2norm: bool = True,
    compute_dtype: torch.dtype = torch.float32,
) -> Tuple[Tensor, Tensor]:
    """Token-by-token KDA on activated inputs (g = log-decay <= 0, beta in (0,1)).

    Returns (o [B,T,H,V] in v.dtype, final state [B,H,V,K] in compute_dtype).
    Follows the loop body of reference tests/kda_oracle.py:113-124.
    """
    if q.shape != k.shape or q.shape != g.shape or q.dim() != 4:
        raise ValueError("q, k and g must share shape [B, T, H, K]")
    if v.dim() != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError("v must have shape [B, T, H, V]")
    if beta.shape != q.shape[:3]:
        raise ValueError("beta must have shape [B, T, H]")
    B, T, H, K = q.shape
    V = v.shape[-1]
    sc = K ** -0.5 if scale is None else float(scale)
    cd = compute_dtype

    qh = q.to(cd).permute(0, 2, 1, 3)          # [B,H,T,K]
    kh = k.to(cd).permute(0, 2, 1, 3)
    if l2norm:
        qh, kh = _unit(qh), _unit(kh)
    qh = qh * sc
    vh = v.to(cd).permute(0, 2, 1, 3)          # [B,H,T,V]
    wh = torch.exp(g.to(cd)).permute(0, 2, 1, 3)  # per-channel decay factor
    bh = beta.to(cd).permute(0, 2, 1)          # [B,H,T]

    if initial_state is None:
        S = torch.zeros(B, H, K, V, dtype=cd, device=q.device)
    else:
        if tuple(initial_state.shape) != (B, H, V, K):
            raise ValueError(f"initial_state must be V-first [B, H, V, K] with shape {(B, H, V, K)}")
        S = initial_state.to(cd).transpose(-1, -2)

    rows = []
    for t in range(T):
        kt = kh[:, :, t, :, None]                      # [B,H,K,1]
        S = S * wh[:, :, t, :, None]                   # decay before the delta
        resid = vh[:, :, t, None, :] - (kt * S).sum(dim=2, keepdim=True)   # [B,H,1,V]
        S = S + (bh[:, :, t, None, None] * kt) * resid
        rows.append((qh[:, :, t, :, None] * S).sum(dim=2))                 # [B,H,V]
    if rows:
        o = torch.stack(rows, dim=2).permute(0, 2, 1, 3)
    else:
        o = vh.new_empty(B, 0, H, V)
    return o.to(v.dtype), S.transpose(-1, -2).contiguous()


def kda_recurrence_varlen(
    q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, cu_seqlens: Sequence[int],
    *, initial_state: Optional[Tensor] = None, scale: Optional[float] = None,
    l2norm: bool = True, compute_dtype: torch.dtype = torch.float32,
) -> Tuple[Tensor, Tensor]:
    """Packed sequences: run every [cu[n], cu[n+1]) segment on its own.

    The reference has no packed-sequence path; by construction the answer for a
    packed batch is the answer of each segment alone with its own state.
    """
    cu = [int(c) for c in cu_seqlens]
    if q.shape[0] != 1:
        raise ValueError("packed inputs must have batch size 1")
    outs, finals = [], []
    for n in range(len(cu) - 1):
        a, b = cu[n], cu[n + 1]
        h0 = None if initial_state is None else initial_state[n:n + 1]
        o, s = kda_recurrence(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b],
                              initial_state=h0, scale=scale, l2norm=l2norm, compute_dtype=compute_dtype)
        outs.append(o)
        finals.append(s)
    return torch.cat(outs, dim=1), torch.cat(finals, dim=0)


def kda_raw(
    q: Tensor, k: Tensor, v: Tensor, raw_gate: Tensor, beta_logits: Tensor, A_log: Tensor, dt_bias: Tensor,
    *, initial_state: Optional[Tensor] = None, lower_bound: float = -5.0, scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
) -> Tuple[Tensor, Tensor]:
    """Raw operator surface (activations fused): reference tests/kda_oracle.py:50-127."""
    cd = compute_dtype
    g = decay_gate(raw_gate.to(cd), A_log.to(cd), dt_bias.to(cd), lower_bound)
    beta = torch.sigmoid(beta_logits.to(cd))
    return kda_recurrence(q, k, v, g, beta, initial_state=initial_state, scale=scale,
                          l2norm=True, compute_dtype=cd)


def decode_step(q, k, v, g, beta, state, *, scale=None, l2norm=True):
    """One-token step: T == 1 recurrence on a given V-first state."""
    return kda_recurrence(q, k, v, g, beta, initial_state=state, scale=scale, l2norm=l2norm)


# --------------------------------------------------------------------------
# short causal depthwise convolution (+ SiLU) with an explicit cache
# --------------------------------------------------------------------------

def causal_conv(x: Tensor, weight: Tensor, *, initial_state: Optional[Tensor] = None,
                activation: bool = True) -> Tuple[Tensor, Tensor]:
    """y[b,t,c] = act(sum_j w[c,j] * xx[b, t+j, c]) with xx = [cache[..., 1:], x].

    x [B,T,C]; weight [C,W]; cache [B,C,W] holds the last W inputs *including*
    the current token, zeros on the left at sequence start.  Follows reference
    tests/kda_oracle.py:130-161 (written here as one windowed gather instead of
    a token loop).
    """
    if x.dim() != 3 or weight.dim() != 2 or x.shape[-1] != weight.shape[0]:
        raise ValueError("expected x [B,T,C] and weight [C,W]")
    B, T, C = x.shape
    W = weight.shape[1]
    if initial_state is None:
        cache = x.new_zeros(B, C, W)
    else:
        if tuple(initial_state.shape) != (B, C, W):
            raise ValueError("invalid convolution state shape")
        cache = initial_state
    xx = torch.cat([cache.transpose(1, 2), x], dim=1)       # [B, W+T, C]; row W+t is token t
    final = xx[:, -W:, :].transpose(1, 2).contiguous()
    if T == 0:
        return x.new_empty(B, 0, C), final
    win = xx[:, 1:, :].unfold(1, W, 1)                      # [B, T, C, W]; window ending at token t
    y = (win * weight.view(1, 1, C, W)).sum(dim=-1)
    if activation:
        y = y * torch.sigmoid(y)
    return y, final


# --------------------------------------------------------------------------
# gated RMSNorm
# --------------------------------------------------------------------------

def rmsnorm_gated(x: Tensor, gate: Tensor, weight: Tensor, eps: float) -> Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate) over the last dim.

    Follows reference tests/kda_oracle.py:164-173.
    """
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * inv * weight.to(x.dtype) * torch.sigmoid(gate)


# --------------------------------------------------------------------------
# helpers shared by tests and the benchmark's CPU leg
# --------------------------------------------------------------------------

def rel_l2(actual: Tensor, expected: Tensor) -> float:
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    den = e.norm().item()
    num = (a - e).norm().item()
    if den == 0.0:
        return num
    return num / den


def make_inputs(B, T, H, K, V, *, seed=0, dtype=torch.float32, with_state=False, n_states=None):
    """Seeded synthetic activations with the distributions the benchmark configs name:
    q,k ~ N(0,1) L2-normalised; v ~ N(0,1); beta = sigmoid(N(0,1));
    g = clamp(-softplus(N(0,1)) * 0.1, -5, 0); optional state ~ N(0, 0.02)."""
    gen = torch.Generator().manual_seed(seed)
    q = _unit(torch.randn(B, T, H, K, generator=gen))
    k = _unit(torch.randn(B, T, H, K, generator=gen))
    v = torch.randn(B, T, H, V, generator=gen)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen))
    g = (-torch.nn.functional.softplus(torch.randn(B, T, H, K, generator=gen)) * 0.1).clamp(-5.0, 0.0)
    out = {"q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "g": g.to(dtype), "beta": beta.to(dtype)}
    if with_state:
        n = B if n_states is None else n_states
        out["h0"] = torch.randn(n, H, V, K, generator=gen) * 0.02
    return out


def default_scale(K: int) -> float:
    return 1.0 / math.sqrt(K)
