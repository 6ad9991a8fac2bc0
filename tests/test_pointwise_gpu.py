"""GPU parity for the bandwidth kernels: convolution, gated RMSNorm, gate activations."""

import os

import numpy as np
import pytest
import torch

import kda_oracle as O

pytestmark = pytest.mark.gpu
D0 = "cuda:0"

CONV_TAGS = ["t9", "t9s", "t2s", "t4", "t70s", "t5w3"]


def _conv_mod(C, W, w):
    from experiment_swa_kda_b200 import ShortConvolution
    mod = ShortConvolution(C, W).to(D0)
    with torch.no_grad():
        mod.weight.copy_(w.unsqueeze(1))
    return mod


@pytest.mark.parametrize("tag", CONV_TAGS)
def test_conv_fp32_matches_reference_vectors(golden_dir, tag):
    z = np.load(os.path.join(golden_dir, "conv.npz"))
    g = lambda n: torch.from_numpy(z[f"{tag}_{n}"])
    x = g("x").to(D0).requires_grad_(True)
    w = g("w")
    has_state = f"{tag}_s0" in z.files
    s0 = g("s0").to(D0).requires_grad_(True) if has_state else None
    mod = _conv_mod(w.shape[0], w.shape[1], w.to(D0))
    y, fs = mod(x, s0, output_final_state=True)
    torch.testing.assert_close(y.cpu(), g("y"), atol=2e-6, rtol=1e-5)
    assert torch.equal(fs.cpu(), g("fs"))
    leaves = [x, mod.weight] + ([s0] if has_state else [])
    grads = torch.autograd.grad((y, fs), leaves, (g("cy").to(D0), g("cs").to(D0)))
    torch.testing.assert_close(grads[0].cpu(), g("dx"), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(grads[1].squeeze(1).cpu(), g("dw"), atol=1e-4, rtol=1e-5)
    if has_state:
        torch.testing.assert_close(grads[2].cpu(), g("ds0"), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("B,T,C,state", [(2, 4096, 384, False), (2, 257, 384, True), (1, 3, 384, True), (3, 100, 20, True)])
def test_conv_bf16_matches_oracle(B, T, C, state):
    gen = torch.Generator().manual_seed(T + C)
    x = torch.randn(B, T, C, generator=gen).bfloat16()
    w = (torch.rand(C, 4, generator=gen) * 2 - 1) * (3 ** 0.5) * C ** -0.5
    s0 = torch.randn(B, C, 4, generator=gen).bfloat16() if state else None
    mod = _conv_mod(C, 4, w.to(D0))
    xd = x.to(D0).requires_grad_(True)
    sd = s0.to(D0).requires_grad_(True) if state else None
    y, fs = mod(xd, sd, output_final_state=True)
    xe = x.float().requires_grad_(True)
    we = w.bfloat16().float().requires_grad_(True)     # the module casts its weight to the activation dtype
    se = s0.float().requires_grad_(True) if state else None
    ye, fse = O.causal_conv(xe, we, initial_state=se)
    cy = torch.randn(ye.shape, generator=gen).bfloat16()
    cs = torch.randn(fse.shape, generator=gen).bfloat16()
    assert O.rel_l2(y.float(), ye) <= 1e-2 and torch.equal(fs.float().cpu(), fse.detach())
    leaves = [xd, mod.weight] + ([sd] if state else [])
    got = torch.autograd.grad((y, fs), leaves, (cy.to(D0), cs.to(D0)))
    want = torch.autograd.grad((ye, fse), [xe, we] + ([se] if state else []), (cy.float(), cs.float()))
    assert O.rel_l2(got[0].float(), want[0]) <= 1e-2
    assert O.rel_l2(got[1].squeeze(1).float(), want[1]) <= 1e-2
    if state:
        assert O.rel_l2(got[2].float(), want[2]) <= 1e-2


@pytest.mark.parametrize("B,T,C,dtype", [(2, 4096, 384, torch.bfloat16), (1, 100, 20, torch.bfloat16), (2, 67, 384, torch.float32),
                                         (3, 1, 64, torch.float32), (1, 5, 130, torch.bfloat16), (2, 129, 72, torch.float32),
                                         # bf16 with C % 128 == 0: small sizes stay on the tile kernel, large ones take the
                                         # streaming backward (32 and 64 tokens per thread run), all with ragged ends
                                         (1, 1, 128, torch.bfloat16), (2, 3, 256, torch.bfloat16), (3, 67, 128, torch.bfloat16),
                                         (2, 1031, 1024, torch.bfloat16), (2, 4099, 2048, torch.bfloat16),
                                         (1, 30001, 2048, torch.bfloat16)])
def test_conv_training_path_matches_oracle(B, T, C, dtype):
    """No carried-in window, no final state: the tiled forward / backward kernels (ragged T and C tails included)."""
    gen = torch.Generator().manual_seed(T * 7 + C)
    x = torch.randn(B, T, C, generator=gen).to(dtype)
    w = (torch.rand(C, 4, generator=gen) * 2 - 1) * (3 ** 0.5) * C ** -0.5
    mod = _conv_mod(C, 4, w.to(D0))
    xd = x.to(D0).requires_grad_(True)
    y, fs = mod(xd)
    assert fs is None
    xe = x.float().requires_grad_(True)
    we = (w.to(dtype).float() if dtype == torch.bfloat16 else w.clone()).requires_grad_(True)
    ye, _ = O.causal_conv(xe, we)
    cy = torch.randn(ye.shape, generator=gen).to(dtype)
    got = torch.autograd.grad(y, [xd, mod.weight], cy.to(D0))
    want = torch.autograd.grad(ye, [xe, we], cy.float())
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert O.rel_l2(y.float(), ye) <= tol
    assert O.rel_l2(got[0].float(), want[0]) <= tol
    assert O.rel_l2(got[1].squeeze(1).float(), want[1]) <= tol


@pytest.mark.parametrize("B,T,C,dtype", [(2, 300, 384, torch.bfloat16), (1, 67, 20, torch.float32)])
def test_short_convolutions_one_launch_equals_per_tensor_calls(B, T, C, dtype):
    """The batched q/k/v convolution entry points give bit-identical outputs and gradients to three separate calls."""
    gen = torch.Generator().manual_seed(T + C)
    mods = [_conv_mod(C, 4, ((torch.rand(C, 4, generator=gen) * 2 - 1) * 0.1).to(D0)) for _ in range(3)]
    xs = [torch.randn(B, T, C, generator=gen).to(dtype).to(D0).requires_grad_(True) for _ in range(3)]
    cys = [torch.randn(B, T, C, generator=gen).to(dtype).to(D0) for _ in range(3)]
    import experiment_swa_kda_b200 as M
    ys = M.short_convolutions(mods, xs)
    got = torch.autograd.grad(ys, xs + [m.weight for m in mods], cys)
    ys1 = [m(x)[0] for m, x in zip(mods, xs)]
    want = torch.autograd.grad(ys1, xs + [m.weight for m in mods], cys)
    for a, b in zip(ys, ys1):
        assert torch.equal(a, b)
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_conv_full_sequence_equals_token_decode():
    gen = torch.Generator().manual_seed(99)
    x = torch.randn(2, 9, 8, generator=gen).to(D0)
    mod = _conv_mod(8, 4, torch.randn(8, 4, generator=gen).to(D0))
    with torch.no_grad():
        full, full_state = mod(x, output_final_state=True)
        state, pieces = None, []
        for t in range(9):
            y, state = mod(x[:, t:t + 1], state, output_final_state=True)
            pieces.append(y)
    torch.testing.assert_close(torch.cat(pieces, 1), full, atol=1e-6, rtol=1e-6)
    assert torch.equal(state, full_state)


@pytest.mark.parametrize("eps", [1e-5, 1e-6])
def test_rmsnorm_fp32_matches_reference_vectors(golden_dir, eps):
    from experiment_swa_kda_b200 import RMSNormGated
    z = np.load(os.path.join(golden_dir, "rmsnorm_gated.npz"))
    x = torch.from_numpy(z["x"]).to(D0).requires_grad_(True)
    gate = torch.from_numpy(z["gate"]).to(D0).requires_grad_(True)
    mod = RMSNormGated(16, eps=eps).to(D0)
    with torch.no_grad():
        mod.weight.copy_(torch.from_numpy(z["w"]))
    y = mod(x, gate)
    tag = f"eps{eps:g}"
    torch.testing.assert_close(y.cpu(), torch.from_numpy(z[f"{tag}_y"]), atol=1e-6, rtol=1e-5)
    got = torch.autograd.grad(y, (x, gate, mod.weight), torch.from_numpy(z[f"{tag}_cy"]).to(D0))
    for a, n in zip(got, ("dx", "dgate", "dw")):
        torch.testing.assert_close(a.cpu(), torch.from_numpy(z[f"{tag}_{n}"]), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("rows,D,dtype", [(24576, 128, torch.bfloat16), (1000, 128, torch.float32), (77, 96, torch.bfloat16),
                                         (33, 256, torch.bfloat16)])
def test_rmsnorm_matches_oracle(rows, D, dtype):
    from experiment_swa_kda_b200 import RMSNormGated
    gen = torch.Generator().manual_seed(rows + D)
    x = torch.randn(rows, D, generator=gen).to(dtype)
    gate = torch.randn(rows, D, generator=gen).to(dtype)
    w = 1 + 0.1 * torch.randn(D, generator=gen)
    cy = torch.randn(rows, D, generator=gen).to(dtype)
    mod = RMSNormGated(D, eps=1e-6).to(D0)
    with torch.no_grad():
        mod.weight.copy_(w)
    xd, gd = x.to(D0).requires_grad_(True), gate.to(D0).requires_grad_(True)
    y = mod(xd, gd)
    got = torch.autograd.grad(y, (xd, gd, mod.weight), cy.to(D0))
    xe, ge, we = x.float().requires_grad_(True), gate.float().requires_grad_(True), w.clone().requires_grad_(True)
    ye = O.rmsnorm_gated(xe, ge, we, 1e-6)
    want = torch.autograd.grad(ye, (xe, ge, we), cy.float())
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert O.rel_l2(y.float(), ye) <= tol
    for a, b in zip(got, want):
        assert O.rel_l2(a.float(), b) <= tol


def test_gate_matches_reference_vectors_and_gradients(golden_dir):
    from experiment_swa_kda_b200 import k3_decay_gate
    z = np.load(os.path.join(golden_dir, "gate.npz"))
    raw = torch.from_numpy(z["raw"]).float().to(D0).requires_grad_(True)
    A = torch.from_numpy(z["A_log"]).float().to(D0).requires_grad_(True)
    bias = torch.from_numpy(z["dt_bias"]).float().to(D0).requires_grad_(True)
    g = k3_decay_gate(raw, A, bias)
    torch.testing.assert_close(g.cpu().double(), torch.from_numpy(z["g"]), atol=2e-6, rtol=1e-5)
    g2 = k3_decay_gate(raw, A, bias, lower_bound=-2.0)
    torch.testing.assert_close(g2.cpu().double(), torch.from_numpy(z["g_lb2"]), atol=2e-6, rtol=1e-5)
    cot = torch.randn(g.shape, generator=torch.Generator().manual_seed(0)).to(D0)
    got = torch.autograd.grad(g, (raw, A, bias), cot)
    r64, A64, b64 = (t.detach().double().cpu().requires_grad_(True) for t in (raw, A, bias))
    want = torch.autograd.grad(O.decay_gate(r64, A64, b64), (r64, A64, b64), cot.double().cpu())
    for a, b in zip(got, want):
        torch.testing.assert_close(a.double().cpu(), b, atol=1e-5, rtol=1e-4)


def test_layer_forward_backward_finite_and_matches_composed_oracle():
    from experiment_swa_kda_b200 import KimiDeltaAttention
    torch.manual_seed(0)
    layer = KimiDeltaAttention(256, 2, 128, norm_eps=1e-6).to(D0)
    with torch.no_grad():
        layer.A_log.normal_(std=0.2)
        layer.dt_bias.normal_(std=0.3)
    x = torch.randn(2, 70, 256, device=D0, dtype=torch.bfloat16, requires_grad=True)
    y, st = layer(x, output_final_state=True)
    y.float().square().mean().backward()
    assert torch.isfinite(y).all() and torch.isfinite(x.grad).all()
    for n, p in layer.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), n
    # compose the same layer from the oracle pieces on the CPU, float32
    with torch.no_grad():
        P = {n: p.detach().float().cpu() for n, p in layer.named_parameters()}
        xc = x.detach().float().cpu()
        lin = lambda name, inp: inp @ P[name + ".weight"].bfloat16().float().t()
        q, _ = O.causal_conv(lin("q_proj", xc), P["q_conv1d.weight"].squeeze(1).bfloat16().float())
        k, _ = O.causal_conv(lin("k_proj", xc), P["k_conv1d.weight"].squeeze(1).bfloat16().float())
        v, _ = O.causal_conv(lin("v_proj", xc), P["v_conv1d.weight"].squeeze(1).bfloat16().float())
        sh = (2, 70, 2, 128)
        raw = lin("f_b_proj", lin("f_a_proj", xc)).reshape(sh)
        bl = lin("b_proj", xc)
        o, mem = O.kda_raw(q.reshape(sh), k.reshape(sh), v.reshape(sh), raw, bl, P["A_log"], P["dt_bias"])
        o = O.rmsnorm_gated(o, lin("g_proj", xc).reshape(sh), P["o_norm.weight"], 1e-6)
        ye = lin("o_proj", o.reshape(2, 70, 256))
    assert O.rel_l2(y.float(), ye) <= 3e-2      # several bf16 GEMMs in series
    assert O.rel_l2(st.memory, mem) <= 3e-2
