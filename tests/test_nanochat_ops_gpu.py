"""`torch.ops.nanochat_kda.*` driven the way the reference mixer drives them (positional calls from autograd
Functions that save only the inputs and the forward output: nanochat/mixers/kda.py:383-466), checked against the oracle."""

import pytest
import torch

import kda_oracle as O

pytestmark = pytest.mark.gpu
D0 = "cuda:0"


class _KDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state, output_final_state, lower_bound, scale):
        output, final_state = torch.ops.nanochat_kda.chunk_forward(q, k, v, raw_gate, beta_logits, A_log, dt_bias, initial_state,
                                                                  output_final_state, lower_bound, scale)
        ctx.initial_state, ctx.final_state, ctx.lb, ctx.scale = initial_state, final_state, lower_bound, scale
        ctx.save_for_backward(q, k, v, raw_gate, beta_logits, A_log, dt_bias, output)
        return output, final_state

    @staticmethod
    def backward(ctx, grad_output, grad_final_state):
        q, k, v, raw_gate, beta_logits, A_log, dt_bias, output = ctx.saved_tensors
        g = torch.ops.nanochat_kda.chunk_backward(q, k, v, raw_gate, beta_logits, A_log, dt_bias, ctx.initial_state, output,
                                                  ctx.final_state, grad_output, grad_final_state, ctx.lb, ctx.scale)
        assert len(g) == 8
        return (*g[:7], g[7] if ctx.initial_state is not None else None, None, None, None)


def _inputs(T, D, seed, grad):
    gen = torch.Generator().manual_seed(seed)
    act = lambda *s: torch.randn(*s, generator=gen).bfloat16().to(D0).requires_grad_(grad)
    q, k, v, g = (act(2, T, 2, D) for _ in range(4))
    beta = act(2, T, 2)
    A_log = (torch.randn(2, generator=gen) * 0.2).to(D0).requires_grad_(grad)
    dt_bias = (torch.randn(2, D, generator=gen) * 0.3).to(D0).requires_grad_(grad)
    h0 = (torch.randn(2, 2, D, D, generator=gen) * 0.05).to(D0).requires_grad_(grad)
    return q, k, v, g, beta, A_log, dt_bias, h0


@pytest.mark.parametrize("T,D", [(65, 128), (33, 64)])
def test_chunk_ops_forward_backward_match_oracle(T, D):
    from experiment_swa_kda_b200 import nanochat_ops
    nanochat_ops.register()
    t = _inputs(T, D, 5 + T, True)
    e = tuple(x.detach().float().cpu().clone().requires_grad_(True) for x in t)
    o, s = _KDA.apply(*t[:7], t[7], True, -5.0, D ** -0.5)
    eo, es = O.kda_raw(*e[:7], initial_state=e[7])
    gen = torch.Generator().manual_seed(1)
    co, cs = torch.randn(eo.shape, generator=gen).bfloat16(), torch.randn(es.shape, generator=gen)
    got = torch.autograd.grad((o, s), t, (co.to(D0), cs.to(D0)))
    want = torch.autograd.grad((eo, es), e, (co.float(), cs))
    assert O.rel_l2(o.float(), eo) <= 1e-2 and O.rel_l2(s, es) <= 1e-2
    for name, a, b in zip(("q", "k", "v", "raw_gate", "beta_logits", "A_log", "dt_bias", "initial_state"), got, want):
        if name in ("A_log", "dt_bias"):
            # parameter gradients are sums over all tokens of bf16-level terms that largely cancel: the reference's own
            # element-wise bar for them (configs/research/kda_cuda_ownership.toml:44-47) is the meaningful one
            torch.testing.assert_close(a.float().cpu(), b, atol=2e-2, rtol=2e-2)
        else:
            assert O.rel_l2(a.float(), b) <= 1e-2, name


def test_decode_conv_and_norm_ops():
    from experiment_swa_kda_b200 import nanochat_ops
    nanochat_ops.register()
    q, k, v, g, beta, A_log, dt_bias, h0 = _inputs(1, 128, 9, False)
    o, s = torch.ops.nanochat_kda.recurrent_decode(q, k, v, g, beta, A_log, dt_bias, h0, True, -5.0, 128 ** -0.5)
    eo, es = O.kda_raw(*(x.float().cpu() for x in (q, k, v, g, beta, A_log, dt_bias)), initial_state=h0.cpu())
    assert O.rel_l2(o.float(), eo) <= 1e-2 and O.rel_l2(s, es) <= 1e-4
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(2, 70, 256, generator=gen).bfloat16().to(D0)
    w = (torch.randn(256, 4, generator=gen) * 0.1).bfloat16().to(D0)
    s0 = torch.randn(2, 256, 4, generator=gen).bfloat16().to(D0)
    y, fs = torch.ops.nanochat_kda.causal_convolution_forward(x, w, s0, True)
    ey, efs = O.causal_conv(x.float().cpu(), w.float().cpu(), initial_state=s0.float().cpu())
    assert O.rel_l2(y.float(), ey) <= 1e-2 and torch.equal(fs.float().cpu(), efs)
    dy = torch.randn(2, 70, 256, generator=gen).bfloat16().to(D0)
    dx, dw, ds0 = torch.ops.nanochat_kda.causal_convolution_backward(x, w, s0, y, fs, dy, None)
    xe, we, se = (t.float().cpu().requires_grad_(True) for t in (x, w, s0))
    ye, _ = O.causal_conv(xe, we, initial_state=se)
    gx, gw, gs = torch.autograd.grad(ye, (xe, we, se), dy.float().cpu())
    assert O.rel_l2(dx.float(), gx) <= 1e-2 and O.rel_l2(dw.float(), gw) <= 1e-2 and O.rel_l2(ds0.float(), gs) <= 1e-2
    xn = torch.randn(300, 128, generator=gen).bfloat16().to(D0)
    gate = torch.randn(300, 128, generator=gen).bfloat16().to(D0)
    wn = (1 + 0.1 * torch.randn(128, generator=gen)).to(D0)
    yn, inv = torch.ops.nanochat_kda.rmsnorm_gate_forward(xn, gate, wn, 1e-5)
    assert O.rel_l2(yn.float(), O.rmsnorm_gated(xn.float().cpu(), gate.float().cpu(), wn.cpu(), 1e-5)) <= 1e-2
    cy = torch.randn(300, 128, generator=gen).bfloat16().to(D0)
    dxn, dgate, dwn = torch.ops.nanochat_kda.rmsnorm_gate_backward(xn, gate, wn, inv, cy, 1e-5)
    xe, ge, we = (t.float().cpu().requires_grad_(True) for t in (xn, gate, wn))
    want = torch.autograd.grad(O.rmsnorm_gated(xe, ge, we, 1e-5), (xe, ge, we), cy.float().cpu())
    assert dwn.shape == (128,) and dwn.dtype == torch.float32
    for a, b in zip((dxn, dgate, dwn), want):
        assert O.rel_l2(a.float(), b) <= 1e-2


def test_convolution_backward_with_a_final_state_cotangent():
    """Both cotangents at once (output and carried-out window), with and without a carried-in window."""
    from experiment_swa_kda_b200 import nanochat_ops
    nanochat_ops.register()
    gen = torch.Generator().manual_seed(12)
    for with_state, T in ((True, 70), (False, 2), (True, 3)):
        x = torch.randn(2, T, 256, generator=gen).bfloat16().to(D0)
        w = (torch.randn(256, 4, generator=gen) * 0.1).bfloat16().to(D0)
        s0 = torch.randn(2, 256, 4, generator=gen).bfloat16().to(D0) if with_state else None
        y, fs = torch.ops.nanochat_kda.causal_convolution_forward(x, w, s0, True)
        dy = torch.randn(2, T, 256, generator=gen).bfloat16().to(D0)
        dfs = torch.randn(2, 256, 4, generator=gen).bfloat16().to(D0)
        dx, dw, ds0 = torch.ops.nanochat_kda.causal_convolution_backward(x, w, s0, y, fs, dy, dfs)
        xe, we = x.float().cpu().requires_grad_(True), w.float().cpu().requires_grad_(True)
        se = s0.float().cpu().requires_grad_(True) if with_state else None
        ye, fse = O.causal_conv(xe, we, initial_state=se)
        leaves = [xe, we] + ([se] if with_state else [])
        want = torch.autograd.grad((ye, fse), leaves, (dy.float().cpu(), dfs.float().cpu()))
        assert O.rel_l2(dx.float(), want[0]) <= 1e-2 and O.rel_l2(dw.float(), want[1]) <= 1e-2
        if with_state:
            assert O.rel_l2(ds0.float(), want[2]) <= 1e-2
        else:
            assert ds0 is None


def test_chunk_backward_takes_a_non_contiguous_grad_output():
    """The reference contract lets grad_output arrive with any strides (it is made contiguous inside the operator,
    nanochat/mixers/cuda_kda/chunk.cu:1802)."""
    from experiment_swa_kda_b200 import nanochat_ops
    nanochat_ops.register()
    t = _inputs(65, 128, 77, False)
    o, s = torch.ops.nanochat_kda.chunk_forward(*t[:7], t[7], True, -5.0, 128 ** -0.5)
    gen = torch.Generator().manual_seed(3)
    wide = torch.randn(2, 65, 2, 256, generator=gen).bfloat16().to(D0)
    go_view = wide[..., ::2]                       # stride 2 in the last dimension
    assert not go_view.is_contiguous()
    a = torch.ops.nanochat_kda.chunk_backward(*t[:7], t[7], o, s, go_view, None, -5.0, 128 ** -0.5)
    b = torch.ops.nanochat_kda.chunk_backward(*t[:7], t[7], o, s, go_view.contiguous(), None, -5.0, 128 ** -0.5)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_chunk_backward_uses_the_forward_sidecar_instead_of_recomputing():
    """The forward that tracks gradients returns `output` as the head of a larger allocation; handed back to
    chunk_backward it supplies the gate and the workspace, so only the backward kernels run.  A copy of the output has
    no sidecar: the operator then recomputes the forward first and must give the same gradients."""
    from experiment_swa_kda_b200 import _lib, nanochat_ops
    nanochat_ops.register()
    t = _inputs(200, 128, 31, True)
    o, s = torch.ops.nanochat_kda.chunk_forward(*t[:7], t[7], True, -5.0, 128 ** -0.5)
    assert o.untyped_storage().nbytes() > o.numel() * 2 and o.is_contiguous() and o.shape == (2, 200, 2, 128)
    go = torch.randn(o.shape, generator=torch.Generator().manual_seed(4)).bfloat16().to(D0)
    gs = torch.randn(s.shape, generator=torch.Generator().manual_seed(5)).to(D0)
    n0 = _lib.launch_count()
    kept = torch.ops.nanochat_kda.chunk_backward(*t[:7], t[7], o, s, go, gs, -5.0, 128 ** -0.5)
    n1 = _lib.launch_count()
    redo = torch.ops.nanochat_kda.chunk_backward(*t[:7], t[7], o.clone(), s, go, gs, -5.0, 128 ** -0.5)
    n2 = _lib.launch_count()
    assert (n2 - n1) > (n1 - n0), "the copy should have cost a forward recompute, the original should not"
    for a, b in zip(kept, redo):
        assert torch.equal(a, b)
    # a forward without gradients keeps nothing: smaller allocation, same visible result
    with torch.no_grad():
        td = [x.detach() for x in t]
        o2, s2 = torch.ops.nanochat_kda.chunk_forward(*td[:7], td[7], True, -5.0, 128 ** -0.5)
    assert torch.equal(o2, o) and torch.equal(s2, s)
    assert o2.untyped_storage().nbytes() < o.untyped_storage().nbytes()


def test_packed_batch_through_the_registered_operators():
    """cu_seqlens is the trailing, defaulted argument of chunk_forward / chunk_backward: a packed batch with ragged tails
    and an empty segment, forward and backward through torch.ops, against the per-segment oracle."""
    from experiment_swa_kda_b200 import nanochat_ops
    nanochat_ops.register()
    cu = [0, 130, 131, 131, 400]
    gen = torch.Generator().manual_seed(55)
    act = lambda *s: torch.randn(*s, generator=gen).bfloat16().to(D0)
    q, k, v, g = (act(1, 400, 2, 128) for _ in range(4))
    beta = act(1, 400, 2)
    A_log = (torch.randn(2, generator=gen) * 0.2).to(D0)
    dt_bias = (torch.randn(2, 128, generator=gen) * 0.3).to(D0)
    h0 = (torch.randn(4, 2, 128, 128, generator=gen) * 0.05).to(D0)
    cu_dev = torch.tensor(cu, dtype=torch.int32, device=D0)
    t = [x.requires_grad_(True) for x in (q, k, v, g, beta, A_log, dt_bias, h0)]
    o, s = torch.ops.nanochat_kda.chunk_forward(*t[:7], t[7], True, -5.0, 128 ** -0.5, cu_dev)
    co = torch.randn(o.shape, generator=gen).bfloat16()
    cs = torch.randn(s.shape, generator=gen)
    got = torch.ops.nanochat_kda.chunk_backward(*t[:7], t[7], o, s, co.to(D0), cs.to(D0), -5.0, 128 ** -0.5, cu_dev)
    e = [x.detach().float().cpu().clone().requires_grad_(True) for x in t]
    ge = O.decay_gate(e[3], e[5], e[6], -5.0)
    eo, es = O.kda_recurrence_varlen(e[0], e[1], e[2], ge, torch.sigmoid(e[4]), cu, initial_state=e[7])
    want = torch.autograd.grad((eo, es), e, (co.float(), cs))
    assert s.shape == (4, 2, 128, 128)
    assert O.rel_l2(o.float(), eo) <= 1e-2 and O.rel_l2(s, es) <= 1e-2
    for name, a, b in zip(("q", "k", "v", "raw_gate", "beta_logits", "A_log", "dt_bias", "initial_state"), got, want):
        if name in ("A_log", "dt_bias"):
            torch.testing.assert_close(a.float().cpu(), b, atol=2e-2, rtol=2e-2)
        else:
            assert O.rel_l2(a.float(), b) <= 1e-2, name


def test_operator_rejects_bad_inputs_before_launching():
    from experiment_swa_kda_b200 import _lib, nanochat_ops
    nanochat_ops.register()
    t = list(_inputs(65, 128, 5, False))
    n0 = _lib.launch_count()
    with pytest.raises(RuntimeError, match="A_log must be a CUDA tensor"):
        torch.ops.nanochat_kda.chunk_forward(*t[:5], t[5].cpu(), t[6], t[7], True, -5.0, 128 ** -0.5)
    with pytest.raises(RuntimeError, match="initial_state must be a CUDA tensor"):
        torch.ops.nanochat_kda.chunk_forward(*t[:7], t[7].cpu(), True, -5.0, 128 ** -0.5)
    with pytest.raises(RuntimeError, match="dt_bias must be contiguous CUDA float32 with H\\*K elements"):
        torch.ops.nanochat_kda.chunk_forward(*t[:6], t[6][:, :64], t[7], True, -5.0, 128 ** -0.5)
    with pytest.raises(RuntimeError, match="lower_bound must be in"):
        torch.ops.nanochat_kda.recurrent_decode(*(x[:, :1] for x in t[:5]), t[5], t[6], t[7], True, -7.0, 128 ** -0.5)
    with pytest.raises(RuntimeError, match="weight must be on the same device"):
        torch.ops.nanochat_kda.rmsnorm_gate_forward(t[0].reshape(-1, 128), t[0].reshape(-1, 128), torch.ones(128), 1e-5)
    with pytest.raises(RuntimeError, match=r"initial_state must have shape \[B, C, W\]"):
        torch.ops.nanochat_kda.causal_convolution_forward(t[0].reshape(2, 65, 256), torch.ones(256, 4, device=D0).bfloat16(),
                                                          torch.zeros(2, 256, 3, device=D0).bfloat16(), False)
    assert _lib.launch_count() == n0


def test_inconsistent_cu_seqlens_is_clamped_and_reported_not_followed():
    """cu_seqlens is read on the device.  A table that reaches past the token count, runs backwards, or needs more
    chunk slots than the workspace holds, or stops short of the token count, is cut back to what the tensors cover (bad segments count as empty) and the
    status word reports it: synchronously through kda_chunk_status, and at the next call through the status ring."""
    import experiment_swa_kda_b200 as m
    from experiment_swa_kda_b200 import _lib, ops
    for bad_cu in ([0, 100, 90, 200], [0, 150, 260], [5, 100, 200], [0, 100, 150]):
        d = O.make_inputs(1, 200, 2, 128, 128, seed=1, with_state=False)
        x = {n: t.bfloat16().to(D0) for n, t in d.items()}
        cu = torch.tensor(bad_cu, dtype=torch.int32, device=D0)
        o, fs, saved = ops.chunk_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], None, cu, 128 ** -0.5, True, True, _lib.LANE_TC)
        with pytest.raises(RuntimeError, match="cu_seqlens is inconsistent"):
            ops.chunk_status(saved, o.device)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="an earlier KDA call .* cu_seqlens is inconsistent"):
            m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"])
        m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"])      # reported once; the device is usable
    torch.cuda.synchronize()
    ops.poll_status(torch.device(D0))


def test_a_bounded_wait_that_runs_out_returns_and_raises_the_status_word():
    """A one-warp kernel waits 2000 polls on a barrier nothing arrives at: it must come back (no trap, no hang), leave
    its wait code in the status word, and the host must turn that word into KDA_ERR_DEVICE_STATUS."""
    from experiment_swa_kda_b200 import _lib
    lib = _lib.load()
    words = torch.full((2,), -1, dtype=torch.int32, device=D0)
    rc = lib.kda_selftest_bounded_wait(words.data_ptr(), 2000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    status, returned = (int(x) for x in words.cpu())
    assert returned == 2 and status == 99
    code = lib.kda_status_word_code(status)
    assert code == -6 and b"bounded wait expired" in lib.kda_error_string(code)
    assert lib.kda_selftest_bounded_wait(words.data_ptr(), 0, None) == -1
    # the context is intact: an ordinary call still works
    assert int((words + 1).sum().item()) == 99 + 2 + 2
