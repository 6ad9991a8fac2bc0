"""Tensor-level operators over the C ABI: allocation, stream and autograd plumbing only.

PyTorch is used for device memory, the current CUDA stream and autograd bookkeeping;
every arithmetic step runs in libkda_b200.so.  Nothing here falls back to PyTorch math.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

Tensor = torch.Tensor

_DT = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16}


def _dt(t: Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise RuntimeError(f"KDA kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _ptr(t: Optional[Tensor]):
    return None if t is None else t.data_ptr()


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _need_cuda(*ts):
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("KDA CUDA operators cannot run on CPU tensors (there is no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("all KDA tensors must be on the same CUDA device")
    return dev


def _bytes(n: int, dev) -> Tensor:
    return torch.empty(max(int(n), 256), dtype=torch.uint8, device=dev)


# --------------------------------------------------------------------------------------------
# chunked KDA on activated inputs
# --------------------------------------------------------------------------------------------

def _shape(q, v, g, n_seq, seq_len, scale, l2norm, lane, forward_only=False) -> "_lib.ChunkShape":
    tokens = q.shape[0] * q.shape[1]
    return _lib.ChunkShape(n_seq, seq_len, tokens, q.shape[2], q.shape[3], v.shape[3], _dt(q), _dt(g), lane,
                           1 if l2norm else 0, float(scale), 1 if forward_only else 0)


# ---- device status word without a hot-path synchronisation ------------------------------------
# Every chunk forward / backward queues a 4-byte copy of its workspace's status word into a page-locked ring with an
# event behind it.  The next call on that device reads the words whose events have completed (host memory, no wait) and
# raises if one is non-zero, so an expired bounded wait or an inconsistent cu_seqlens cannot pass silently.  Nothing is
# queued or polled while the stream is being captured into a CUDA graph.
_STATUS_SLOTS = 64
_status = {}      # device index -> [pinned int32 words, deque of (event, slot), next slot]


def _capturing() -> bool:
    return torch.cuda.is_current_stream_capturing()


def poll_status(dev) -> None:
    ring = _status.get(dev.index)
    if ring is None or _capturing():
        return
    words, pending, _ = ring
    bad = 0
    while pending and pending[0][0].query():
        _, slot = pending.popleft()
        w = int(words[slot])
        words[slot] = 0
        bad = bad or w
    if bad:
        code = _lib.load().kda_status_word_code(bad)
        msg = _lib.load().kda_error_string(code).decode()
        raise RuntimeError(f"an earlier KDA call on {dev} reported device status {bad}: {msg} ({code}); its results are undefined")


def _queue_status(sh, ws, dev) -> None:
    if _capturing():
        return
    ring = _status.get(dev.index)
    if ring is None:
        import collections
        ring = _status[dev.index] = [torch.zeros(_STATUS_SLOTS, dtype=torch.int32).pin_memory(), collections.deque(), 0]
    words, pending, nxt = ring
    if len(pending) >= _STATUS_SLOTS:      # the host is far ahead of the device: skip this sample
        return
    slot = nxt % _STATUS_SLOTS
    ring[2] = nxt + 1
    rc = _lib.load().kda_chunk_status_async(sh, _ptr(ws), words.data_ptr() + 4 * slot, _stream(dev))
    if rc == _lib.OK:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(dev))
        pending.append((ev, slot))


def chunk_kda_fwd(q, k, v, g, beta, h0, cu_seqlens, scale, l2norm, want_final, lane=_lib.LANE_FP32, forward_only=False, norm=None):
    """Returns (o, final_state or None, saved) where saved = (shape, workspace) for the backward.
    forward_only: inference / prefill - the panels only a backward reads are neither stored nor allocated.
    norm = (gate, weight float32 [V], eps): also apply the gated RMSNorm in the output kernel's epilogue (tensor-core lane
    only); the return value then is (o, final_state, saved, y, inv_rms)."""
    lib = _lib.load()
    dev = _need_cuda(q, k, v, g, beta, h0, cu_seqlens)
    poll_status(dev)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if cu_seqlens is not None:
        n_seq, seq_len = cu_seqlens.numel() - 1, 0
    else:
        n_seq, seq_len = B, T
    sh = _shape(q, v, g, n_seq, seq_len, scale, l2norm, lane, forward_only)
    o = torch.empty(B, T, H, V, dtype=v.dtype, device=dev)
    fs = torch.empty(n_seq, H, V, K, dtype=torch.float32, device=dev) if want_final else None
    nbytes = lib.kda_chunk_workspace_bytes(sh)
    ws = _bytes(nbytes, dev)
    with torch.cuda.device(dev):
        if norm is None:
            rc = lib.kda_chunk_fwd(sh, _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(h0), _ptr(cu_seqlens), _ptr(o),
                                   _ptr(fs), _ptr(ws), ws.numel(), _stream(dev))
            _lib.check(rc, "kda_chunk_fwd")
        else:
            gate, nw, eps = norm
            y = torch.empty_like(o)
            inv = torch.empty(B * T * H, dtype=torch.float32, device=dev)
            rc = lib.kda_chunk_fwd_norm(sh, _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(h0), _ptr(cu_seqlens), _ptr(o),
                                        _ptr(fs), _ptr(ws), ws.numel(), _ptr(gate), _ptr(nw), float(eps), _ptr(y), _ptr(inv),
                                        _stream(dev))
            _lib.check(rc, "kda_chunk_fwd_norm")
        _queue_status(sh, ws, dev)
    if norm is not None:
        return o, fs, (sh, ws), y, inv
    return o, fs, (sh, ws)


def chunk_kda_conv_fwd(xq, xk, xv, wq, wk, wv, g, beta, h0, cu_seqlens, scale, l2norm, want_final):
    """No-grad forward with the three short convolutions (width 4, SiLU, zero padding at every sequence start) folded
    into the intra-chunk kernel: xq, xk, xv [B,T,H,128] bf16 are the convolutions' inputs, wq, wk, wv [H*128,4] their
    weights (float32 or bf16).  Tensor-core lane only.  Returns (o, final_state or None), bit-identical to
    conv_fwd x3 followed by chunk_kda_fwd(forward_only=True)."""
    lib = _lib.load()
    dev = _need_cuda(xq, xk, xv, wq, wk, wv, g, beta, h0, cu_seqlens)
    poll_status(dev)
    B, T, H, K = xq.shape
    if cu_seqlens is not None:
        n_seq, seq_len = cu_seqlens.numel() - 1, 0
    else:
        n_seq, seq_len = B, T
    sh = _shape(xq, xv, g, n_seq, seq_len, scale, l2norm, _lib.LANE_TC, True)
    ws_ = [w.contiguous() for w in (wq, wk, wv)]
    if len({w.dtype for w in ws_}) != 1 or ws_[0].dtype not in (torch.float32, torch.bfloat16) or any(w.shape != (H * K, 4) for w in ws_):
        raise ValueError("convolution weights must share one dtype (float32 or bfloat16) and have shape [H*K, 4]")
    o = torch.empty(B, T, H, K, dtype=xv.dtype, device=dev)
    fs = torch.empty(n_seq, H, K, K, dtype=torch.float32, device=dev) if want_final else None
    ws = _bytes(lib.kda_chunk_workspace_bytes(sh), dev)
    with torch.cuda.device(dev):
        rc = lib.kda_chunk_fwd_conv(sh, _ptr(xq), _ptr(xk), _ptr(xv), _ptr(ws_[0]), _ptr(ws_[1]), _ptr(ws_[2]), 4,
                                    _lib.DTYPE_F32 if ws_[0].dtype == torch.float32 else _lib.DTYPE_BF16, _ptr(g), _ptr(beta),
                                    _ptr(h0), _ptr(cu_seqlens), _ptr(o), _ptr(fs), _ptr(ws), ws.numel(), _stream(dev))
        _lib.check(rc, "kda_chunk_fwd_conv")
        _queue_status(sh, ws, dev)
    return o, fs


def chunk_kda_bwd(q, k, v, g, beta, cu_seqlens, do, dfs, saved, want_dh0):
    lib = _lib.load()
    sh, ws = saved
    dev = q.device
    poll_status(dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dg, db = torch.empty_like(g), torch.empty_like(beta)
    n_seq = sh.n_seq
    dh0 = torch.empty(n_seq, sh.heads, sh.value_dim, sh.key_dim, dtype=torch.float32, device=dev) if want_dh0 else None
    scr = _bytes(lib.kda_chunk_bwd_scratch_bytes(sh), dev)
    with torch.cuda.device(dev):
        rc = lib.kda_chunk_bwd(sh, _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(cu_seqlens), _ptr(do), _ptr(dfs),
                               _ptr(ws), ws.numel(), _ptr(scr), scr.numel(), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dg),
                               _ptr(db), _ptr(dh0), _stream(dev))
        _lib.check(rc, "kda_chunk_bwd")
        _queue_status(sh, ws, dev)
    return dq, dk, dv, dg, db, dh0


def chunk_status(saved, dev) -> None:
    """Raise if a bounded device-side wait expired in the kernels that used this workspace (synchronises the stream)."""
    sh, ws = saved
    with torch.cuda.device(dev):
        rc = _lib.load().kda_chunk_status(sh, _ptr(ws), _stream(dev))
    _lib.check(rc, "kda_chunk_status")


class ChunkKDAFunction(torch.autograd.Function):
    """Autograd boundary of the chunked operator on activated inputs.

    Argument list of the operator surface: (q, k, v, g, beta, initial_state,
    output_final_state, cu_seqlens) plus scale / l2norm / lane.  Mirrors the role of
    the reference's _ProjectKDAAutograd (nanochat/mixers/kda.py:383-415).
    """

    @staticmethod
    def forward(ctx, q, k, v, g, beta, initial_state, output_final_state, cu_seqlens, scale, l2norm, lane):
        q, k, v, g, beta = (t.contiguous() for t in (q, k, v, g, beta))
        h0 = None if initial_state is None else initial_state.contiguous()
        o, fs, (sh, ws) = chunk_kda_fwd(q, k, v, g, beta, h0, cu_seqlens, scale, l2norm, output_final_state, lane)
        ctx.shape = sh
        ctx.cu = cu_seqlens
        ctx.has_h0 = initial_state is not None
        # The workspace rides with the saved tensors: it lives exactly as long as the graph does, and a second backward
        # through a retained graph finds it intact (the backward kernels only read it).
        ctx.save_for_backward(q, k, v, g, beta, ws)
        ctx.set_materialize_grads(False)
        return o, fs

    @staticmethod
    def backward(ctx, do, dfs):
        q, k, v, g, beta, ws = ctx.saved_tensors
        do = torch.zeros_like(v) if do is None else do.contiguous()
        if dfs is not None:
            dfs = dfs.contiguous().float()
        dq, dk, dv, dg, db, dh0 = chunk_kda_bwd(q, k, v, g, beta, ctx.cu, do, dfs, (ctx.shape, ws), ctx.has_h0)
        return dq, dk, dv, dg, db, dh0, None, None, None, None, None


class ChunkKDANormFunction(torch.autograd.Function):
    """Chunked KDA followed by the layer's gated RMSNorm, the norm applied in the output kernel's epilogue (one launch and
    one pass over the output less than the two operators in sequence; the reference layer crosses an operator boundary
    here, nanochat/mixers/kda.py:768-795).  Tensor-core lane only.  The backward is the two existing backwards in sequence."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, gate, norm_weight, initial_state, output_final_state, cu_seqlens, scale, l2norm, eps):
        q, k, v, g, beta = (t.contiguous() for t in (q, k, v, g, beta))
        gate = gate.contiguous().to(v.dtype)
        w32 = norm_weight.contiguous().float()
        h0 = None if initial_state is None else initial_state.contiguous()
        o, fs, (sh, ws), y, inv = chunk_kda_fwd(q, k, v, g, beta, h0, cu_seqlens, scale, l2norm, output_final_state,
                                                _lib.LANE_TC, norm=(gate, w32, eps))
        ctx.shape, ctx.cu, ctx.has_h0, ctx.wdtype = sh, cu_seqlens, initial_state is not None, norm_weight.dtype
        ctx.save_for_backward(q, k, v, g, beta, ws, o, gate, w32, inv)
        ctx.set_materialize_grads(False)
        return y, fs

    @staticmethod
    def backward(ctx, dy, dfs):
        q, k, v, g, beta, ws, o, gate, w32, inv = ctx.saved_tensors
        dy = torch.zeros_like(o) if dy is None else dy.contiguous().to(o.dtype)
        do, dgate, dw = rmsnorm_gate_bwd(o, gate, w32, inv, dy)
        if dfs is not None:
            dfs = dfs.contiguous().float()
        dq, dk, dv, dg, db, dh0 = chunk_kda_bwd(q, k, v, g, beta, ctx.cu, do, dfs, (ctx.shape, ws), ctx.has_h0)
        return dq, dk, dv, dg, db, dgate, dw.to(ctx.wdtype), dh0, None, None, None, None, None


# --------------------------------------------------------------------------------------------
# gate activations
# --------------------------------------------------------------------------------------------

class GateFunction(torch.autograd.Function):
    """(raw_gate, beta_logits, A_log, dt_bias) -> (g, beta) in float32, with the parameter
    gradients reduced deterministically (reference chunk_wy_backward.cu:3881-3987)."""

    @staticmethod
    def forward(ctx, raw_gate, beta_logits, A_log, dt_bias, lower_bound):
        lib = _lib.load()
        dev = _need_cuda(raw_gate, beta_logits, A_log, dt_bias)
        raw_gate, beta_logits = raw_gate.contiguous(), beta_logits.contiguous()
        A32, b32 = A_log.contiguous().float(), dt_bias.contiguous().float().reshape(-1)
        B, T, H, K = raw_gate.shape
        if beta_logits.dtype != raw_gate.dtype:
            beta_logits = beta_logits.to(raw_gate.dtype)
        g = torch.empty(B, T, H, K, dtype=torch.float32, device=dev)
        beta = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = lib.kda_gate_fwd(B * T, H, K, _dt(raw_gate), _ptr(raw_gate), _ptr(beta_logits), _ptr(A32), _ptr(b32),
                                  float(lower_bound), _ptr(g), _ptr(beta), _stream(dev))
        _lib.check(rc, "kda_gate_fwd")
        ctx.save_for_backward(raw_gate, beta_logits, A32, b32)
        ctx.lb = float(lower_bound)
        ctx.bias_shape = dt_bias.shape
        ctx.out_dtypes = (A_log.dtype, dt_bias.dtype)
        return g, beta

    @staticmethod
    def backward(ctx, dg, dbeta):
        lib = _lib.load()
        raw_gate, beta_logits, A32, b32 = ctx.saved_tensors
        dev = raw_gate.device
        B, T, H, K = raw_gate.shape
        dg = dg.contiguous().float()
        dbeta = dbeta.contiguous().float()
        d_raw = torch.empty_like(raw_gate)
        d_bl = torch.empty_like(beta_logits)
        dA = torch.empty(H, dtype=torch.float32, device=dev)
        dbias = torch.empty(H * K, dtype=torch.float32, device=dev)
        scr = _bytes(lib.kda_gate_bwd_scratch_bytes(B * T, H, K), dev)
        with torch.cuda.device(dev):
            rc = lib.kda_gate_bwd(B * T, H, K, _dt(raw_gate), _ptr(raw_gate), _ptr(beta_logits), _ptr(A32), _ptr(b32),
                                  ctx.lb, _ptr(dg), _ptr(dbeta), _ptr(d_raw), _ptr(d_bl), _ptr(dA), _ptr(dbias),
                                  _ptr(scr), scr.numel(), _stream(dev))
        _lib.check(rc, "kda_gate_bwd")
        return d_raw, d_bl, dA.to(ctx.out_dtypes[0]), dbias.reshape(ctx.bias_shape).to(ctx.out_dtypes[1]), None


# --------------------------------------------------------------------------------------------
# decode
# --------------------------------------------------------------------------------------------

def decode_step(q, k, v, g, beta, state, scale, l2norm=True, out_state: Optional[Tensor] = None):
    """One token per sequence.  q,k,g [B,1,H,K] (or [B,H,K]); state [B,H,V,K] float32.
    Returns (o shaped like v, new state).  The input state is left untouched unless
    out_state aliases it."""
    lib = _lib.load()
    dev = _need_cuda(q, k, v, g, beta, state)
    q, k, v, g, beta = (t.contiguous() for t in (q, k, v, g, beta))
    if g.dtype != beta.dtype:
        beta = beta.to(g.dtype)
    H, K = q.shape[-2], q.shape[-1]
    V = v.shape[-1]
    n = q.numel() // (H * K)
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape) != (n, H, V, K):
        raise ValueError(f"state must be contiguous float32 V-first [B, H, V, K] with shape {(n, H, V, K)}")
    new_state = torch.empty_like(state) if out_state is None else out_state
    o = torch.empty_like(v)
    with torch.cuda.device(dev):
        rc = lib.kda_decode_step(n, H, K, V, _dt(q), _dt(g), 1 if l2norm else 0, float(scale), _ptr(q), _ptr(k), _ptr(v),
                                 _ptr(g), _ptr(beta), _ptr(state), _ptr(new_state), _ptr(o), _stream(dev))
    _lib.check(rc, "kda_decode_step")
    return o, new_state


def decode_step_raw(q, k, v, raw_gate, beta_logits, A_log, dt_bias, lower_bound, state, scale, out_state: Optional[Tensor] = None):
    """One decode token on RAW inputs (gate and beta activations fused into the kernel, q and k L2-normalised): the
    signature of the reference's recurrent_decode operator in a single launch.  `out_state` may be `state` itself."""
    lib = _lib.load()
    dev = _need_cuda(q, k, v, raw_gate, beta_logits, A_log, dt_bias, state)
    q, k, v, raw_gate, beta_logits = (t.contiguous() for t in (q, k, v, raw_gate, beta_logits))
    if not (q.dtype == k.dtype == v.dtype == raw_gate.dtype == beta_logits.dtype):
        raise RuntimeError("decode_step_raw takes q, k, v, raw_gate and beta_logits in one dtype")
    H, K = q.shape[-2], q.shape[-1]
    V = v.shape[-1]
    n = q.numel() // (H * K)
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape) != (n, H, V, K):
        raise ValueError(f"state must be contiguous float32 V-first [B, H, V, K] with shape {(n, H, V, K)}")
    if A_log.dtype != torch.float32 or dt_bias.dtype != torch.float32 or A_log.numel() != H or dt_bias.numel() != H * K:
        raise ValueError("A_log [H] and dt_bias [H*K] must be float32")
    new_state = torch.empty_like(state) if out_state is None else out_state
    o = torch.empty_like(v)
    with torch.cuda.device(dev):
        rc = lib.kda_decode_step_raw(n, H, K, V, _dt(q), float(scale), _ptr(q), _ptr(k), _ptr(v), _ptr(raw_gate), _ptr(beta_logits),
                                     _ptr(A_log.contiguous()), _ptr(dt_bias.contiguous()), float(lower_bound), _ptr(state),
                                     _ptr(new_state), _ptr(o), _stream(dev))
    _lib.check(rc, "kda_decode_step_raw")
    return o, new_state


def conv_step_multi(xs, weights, caches, silu=True):
    """One decode token through several same-shaped convolutions in one launch; `caches` ([B,C,W] each) are updated IN
    PLACE.  xs: [B,C] (or [B,1,C]) tensors.  Returns the outputs, shaped like xs."""
    import ctypes as C
    lib = _lib.load()
    xs = [x.contiguous() for x in xs]
    ws = [w.contiguous() for w in weights]
    dev = _need_cuda(*xs, *ws, *caches)
    Bn, Cc, W = caches[0].shape
    for x, w, c in zip(xs, ws, caches):
        if x.numel() != Bn * Cc or tuple(c.shape) != (Bn, Cc, W) or tuple(w.shape) != (Cc, W) or not c.is_contiguous() or c.dtype != x.dtype:
            raise ValueError("conv_step_multi needs x [B,C], weight [C,W] and a contiguous cache [B,C,W] of the activation dtype per branch")
    ys = [torch.empty_like(x) for x in xs]
    with torch.cuda.device(dev):
        rc = lib.kda_conv_step_multi(len(xs), Bn, Cc, W, _dt(xs[0]) | _wflag(xs[0], ws[0]), 1 if silu else 0,
                                     C.cast(_ptr_array(xs), C.c_void_p), C.cast(_ptr_array(ws), C.c_void_p),
                                     C.cast(_ptr_array(caches), C.c_void_p), C.cast(_ptr_array(ys), C.c_void_p), _stream(dev))
    _lib.check(rc, "kda_conv_step_multi")
    return ys


def decode_steps(q, k, v, g, beta, state, scale, l2norm=True):
    """n consecutive decode steps in one library call.  q,k,g [n,B,H,K]; v [n,B,H,V]; beta [n,B,H]; `state` [B,H,V,K]
    float32 is UPDATED IN PLACE.  Returns o [n,B,H,V].  One kernel launch per step, issued from C without a host round
    trip per token (the serving loop of the reference makes one operator call per token: nanochat/engine.py:83-226)."""
    lib = _lib.load()
    dev = _need_cuda(q, k, v, g, beta, state)
    q, k, v, g, beta = (t.contiguous() for t in (q, k, v, g, beta))
    if g.dtype != beta.dtype:
        beta = beta.to(g.dtype)
    n, B, H, K = q.shape
    V = v.shape[-1]
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape) != (B, H, V, K):
        raise ValueError(f"state must be contiguous float32 V-first [B, H, V, K] with shape {(B, H, V, K)}")
    o = torch.empty_like(v)
    with torch.cuda.device(dev):
        rc = lib.kda_decode_steps(n, B, H, K, V, _dt(q), _dt(g), 1 if l2norm else 0, float(scale), _ptr(q), _ptr(k), _ptr(v),
                                  _ptr(g), _ptr(beta), _ptr(state), _ptr(o), _stream(dev))
    _lib.check(rc, "kda_decode_steps")
    return o


# --------------------------------------------------------------------------------------------
# short convolution
# --------------------------------------------------------------------------------------------

KDA_WEIGHT_F32 = 0x100


def _wflag(x, weight):
    """float32 weights next to lower-precision activations are read as they are (rounded on load by the kernel)."""
    return KDA_WEIGHT_F32 if (weight.dtype == torch.float32 and x.dtype != torch.float32) else 0


def conv_fwd(x, weight, initial_state, want_final, silu=True):
    lib = _lib.load()
    dev = _need_cuda(x, weight, initial_state)
    B, T, Cc = x.shape
    W = weight.shape[-1]
    y = torch.empty_like(x)
    fin = torch.empty(B, Cc, W, dtype=x.dtype, device=dev) if want_final else None
    with torch.cuda.device(dev):
        rc = lib.kda_conv_fwd(B, T, Cc, W, _dt(x) | _wflag(x, weight), 1 if silu else 0, _ptr(x), _ptr(weight), _ptr(initial_state), _ptr(y),
                              _ptr(fin), _stream(dev))
    _lib.check(rc, "kda_conv_fwd")
    return y, fin


def conv_bwd(x, weight, initial_state, dy, dfin, silu=True):
    lib = _lib.load()
    dev = x.device
    B, T, Cc = x.shape
    W = weight.shape[-1]
    dx = torch.empty_like(x)
    dw = torch.empty(Cc, W, dtype=torch.float32, device=dev)
    dinit = torch.empty_like(initial_state) if initial_state is not None else None
    scr = _bytes(lib.kda_conv_bwd_scratch_bytes(B, T, Cc, W), dev)
    with torch.cuda.device(dev):
        rc = lib.kda_conv_bwd(B, T, Cc, W, _dt(x) | _wflag(x, weight), 1 if silu else 0, _ptr(x), _ptr(weight), _ptr(initial_state), _ptr(dy),
                              _ptr(dfin), _ptr(dx), _ptr(dw), _ptr(dinit), _ptr(scr), scr.numel(), _stream(dev))
    _lib.check(rc, "kda_conv_bwd")
    return dx, dw, dinit


class ConvFunction(torch.autograd.Function):
    """Causal depthwise convolution + SiLU with an explicit cache
    (role of the reference's _ProjectConvolutionAutograd, nanochat/mixers/kda.py:439-466)."""

    @staticmethod
    def forward(ctx, x, weight, initial_state, output_final_state, silu):
        x = x.contiguous()
        w = weight.contiguous()
        if w.dtype != torch.float32:
            w = w.to(x.dtype)
        s0 = None if initial_state is None else initial_state.contiguous().to(x.dtype)
        y, fin = conv_fwd(x, w, s0, output_final_state, silu)
        ctx.save_for_backward(x, w, s0)
        ctx.silu = silu
        ctx.wdtype = weight.dtype
        return y, fin

    @staticmethod
    def backward(ctx, dy, dfin):
        x, w, s0 = ctx.saved_tensors
        dy = dy.contiguous().to(x.dtype)
        if dfin is not None:
            dfin = dfin.contiguous().to(x.dtype)
        dx, dw, dinit = conv_bwd(x, w, s0, dy, dfin, ctx.silu)
        return dx, dw.to(ctx.wdtype), dinit, None, None


def _ptr_array(ts):
    import ctypes as C
    arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    return arr


class ConvMultiFunction(torch.autograd.Function):
    """n same-shaped causal convolutions + SiLU (the q, k and v branches of a layer) in one launch each way.
    Training path only (no cache, no final state); falls back to the per-tensor operator when the library declines."""

    @staticmethod
    def forward(ctx, silu, n, *tensors):
        import ctypes as C
        xs = [t.contiguous() for t in tensors[:n]]
        ws = []
        for w in tensors[n:]:
            w = w.contiguous()
            ws.append(w if w.dtype == torch.float32 else w.to(xs[0].dtype))
        lib = _lib.load()
        dev = _need_cuda(*xs, *ws)
        B, T, Cc = xs[0].shape
        W = ws[0].shape[-1]
        same = all(x.shape == xs[0].shape and x.dtype == xs[0].dtype for x in xs) and \
            all(w.shape == ws[0].shape and w.dtype == ws[0].dtype for w in ws)
        ys = [torch.empty_like(x) for x in xs]
        rc = _lib.ERR_UNSUPPORTED
        if same:
            with torch.cuda.device(dev):
                rc = lib.kda_conv_fwd_multi(n, B, T, Cc, W, _dt(xs[0]) | _wflag(xs[0], ws[0]), 1 if silu else 0,
                                            C.cast(_ptr_array(xs), C.c_void_p), C.cast(_ptr_array(ws), C.c_void_p),
                                            C.cast(_ptr_array(ys), C.c_void_p), _stream(dev))
        if rc == _lib.ERR_UNSUPPORTED:
            ys = [conv_fwd(x, w, None, False, silu)[0] for x, w in zip(xs, ws)]
        else:
            _lib.check(rc, "kda_conv_fwd_multi")
        ctx.save_for_backward(*xs, *ws)
        ctx.n, ctx.silu, ctx.same = n, silu, same
        ctx.wdtypes = [w.dtype for w in tensors[n:]]
        return tuple(ys)

    @staticmethod
    def backward(ctx, *dys):
        import ctypes as C
        n = ctx.n
        saved = ctx.saved_tensors
        xs, ws = list(saved[:n]), list(saved[n:])
        dys = [(torch.zeros_like(x) if d is None else d.contiguous().to(x.dtype)) for d, x in zip(dys, xs)]
        lib = _lib.load()
        dev = xs[0].device
        B, T, Cc = xs[0].shape
        W = ws[0].shape[-1]
        dxs = [torch.empty_like(x) for x in xs]
        dws = [torch.empty(Cc, W, dtype=torch.float32, device=dev) for _ in xs]
        rc = _lib.ERR_UNSUPPORTED
        if ctx.same:
            scr = _bytes(lib.kda_conv_bwd_multi_scratch_bytes(n, B, T, Cc, W), dev)
            with torch.cuda.device(dev):
                rc = lib.kda_conv_bwd_multi(n, B, T, Cc, W, _dt(xs[0]) | _wflag(xs[0], ws[0]), 1 if ctx.silu else 0,
                                            C.cast(_ptr_array(xs), C.c_void_p), C.cast(_ptr_array(ws), C.c_void_p),
                                            C.cast(_ptr_array(dys), C.c_void_p), C.cast(_ptr_array(dxs), C.c_void_p),
                                            C.cast(_ptr_array(dws), C.c_void_p), _ptr(scr), scr.numel(), _stream(dev))
        if rc == _lib.ERR_UNSUPPORTED:
            res = [conv_bwd(x, w, None, d, None, ctx.silu) for x, w, d in zip(xs, ws, dys)]
            dxs, dws = [r[0] for r in res], [r[1] for r in res]
        else:
            _lib.check(rc, "kda_conv_bwd_multi")
        return (None, None, *dxs, *[dw.to(dt) for dw, dt in zip(dws, ctx.wdtypes)])


# --------------------------------------------------------------------------------------------
# gated RMSNorm
# --------------------------------------------------------------------------------------------

def rmsnorm_gate_fwd(x, gate, weight, eps):
    lib = _lib.load()
    dev = _need_cuda(x, gate, weight)
    D = x.shape[-1]
    rows = x.numel() // D
    y = torch.empty_like(x)
    inv = torch.empty(rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.kda_rmsnorm_gate_fwd(rows, D, _dt(x), float(eps), _ptr(x), _ptr(gate), _ptr(weight), _ptr(y), _ptr(inv),
                                      _stream(dev))
    _lib.check(rc, "kda_rmsnorm_gate_fwd")
    return y, inv


def rmsnorm_gate_bwd(x, gate, weight, inv, dy):
    lib = _lib.load()
    dev = x.device
    D = x.shape[-1]
    rows = x.numel() // D
    dx, dgate = torch.empty_like(x), torch.empty_like(gate)
    dw = torch.empty(D, dtype=torch.float32, device=dev)
    scr = _bytes(lib.kda_rmsnorm_gate_bwd_scratch_bytes(rows, D), dev)
    with torch.cuda.device(dev):
        rc = lib.kda_rmsnorm_gate_bwd(rows, D, _dt(x), _ptr(x), _ptr(gate), _ptr(weight), _ptr(inv), _ptr(dy), _ptr(dx),
                                      _ptr(dgate), _ptr(dw), _ptr(scr), scr.numel(), _stream(dev))
    _lib.check(rc, "kda_rmsnorm_gate_bwd")
    return dx, dgate, dw


class RMSNormGateFunction(torch.autograd.Function):
    """y = rms_norm(x; w, eps) * sigmoid(gate)
    (role of the reference's _ProjectRMSNormGateAutograd, nanochat/mixers/kda.py:418-436)."""

    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        x = x.contiguous()
        gate = gate.contiguous().to(x.dtype)
        w32 = weight.contiguous().float()
        y, inv = rmsnorm_gate_fwd(x, gate, w32, eps)
        ctx.save_for_backward(x, gate, w32, inv)
        ctx.wdtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gate, w32, inv = ctx.saved_tensors
        dx, dgate, dw = rmsnorm_gate_bwd(x, gate, w32, inv, dy.contiguous().to(x.dtype))
        return dx, dgate, dw.to(ctx.wdtype), None
