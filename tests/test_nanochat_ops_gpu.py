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
    dxn, dgate, dwn = torch.ops.nanochat_kda.rmsnorm_gate_backward(xn, gate, wn, inv, yn, 1e-5)
    assert torch.isfinite(dxn.float()).all() and torch.isfinite(dgate.float()).all() and dwn.shape == (128,)
