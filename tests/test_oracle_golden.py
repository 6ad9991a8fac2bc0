"""Pins oracle/kda_oracle.py to the reference: golden vectors produced by the
reference's own oracle and CPU production loop (tests/golden/make_golden.py)
and the reference's closed-form known answers (its tests/test_kda_operator.py:62-180)."""

import math
import os

import numpy as np
import pytest
import torch

import kda_oracle as O

NAMES = ("q", "k", "v", "raw_gate", "beta_logits", "A_log", "dt_bias", "initial_state")
RAW_CASES = ["raw_b2_t7_h2_k4_v3", "raw_b1_t64_h2_k16_v11", "raw_b2_t65_h2_k16_v24", "raw_b1_t130_h2_k32_v32"]


def _load(golden_dir, tag):
    z = np.load(os.path.join(golden_dir, tag + ".npz"))
    return {n: torch.from_numpy(z[n]) for n in z.files}


@pytest.mark.parametrize("tag", RAW_CASES)
@pytest.mark.parametrize("which", ["oracle", "prod"])
def test_raw_surface_matches_reference_vectors(golden_dir, tag, which):
    d = _load(golden_dir, tag)
    leaf = {n: d[n].clone().requires_grad_(True) for n in NAMES}
    o, s = O.kda_raw(*(leaf[n] for n in NAMES[:7]), initial_state=leaf["initial_state"])
    grads = torch.autograd.grad((o, s), [leaf[n] for n in NAMES], (d["cot_o"], d["cot_s"]))
    # both sides are float32 token loops; they differ only by summation order
    assert O.rel_l2(o, d[f"{which}_o"]) < 2e-6
    assert O.rel_l2(s, d[f"{which}_s"]) < 2e-6
    for n, gr in zip(NAMES, grads):
        assert O.rel_l2(gr, d[f"{which}_d_{n}"]) < 2e-5, n


def test_float64_vector(golden_dir):
    d = _load(golden_dir, "raw_f64_b1_t70_h2_k8_v8")
    o, s = O.kda_raw(*(d[n].double() for n in NAMES[:7]), initial_state=d["initial_state"].double(),
                     compute_dtype=torch.float64)
    assert O.rel_l2(o, d["oracle_o"]) < 1e-13
    assert O.rel_l2(s, d["oracle_s"]) < 1e-13


def test_gate_vectors_and_bounds(golden_dir):
    d = _load(golden_dir, "gate")
    assert torch.allclose(O.decay_gate(d["raw"], d["A_log"], d["dt_bias"]), d["g"], atol=1e-12, rtol=1e-12)
    assert torch.allclose(O.decay_gate(d["raw"], d["A_log"], d["dt_bias"], -2.0), d["g_lb2"], atol=1e-12, rtol=1e-12)
    raw = torch.tensor([-100.0, -2.0, 0.0, 2.0, 100.0], dtype=torch.float64).view(1, 1, 1, 5)
    g = O.decay_gate(raw, torch.tensor([0.3], dtype=torch.float64), torch.zeros(1, 5, dtype=torch.float64))
    assert torch.all(g <= 0) and torch.all(g >= -5)
    assert torch.all(g[..., 1:] < g[..., :-1])
    assert g[..., 0].item() == pytest.approx(0.0, abs=1e-12)
    assert g[..., -1].item() == pytest.approx(-5.0, abs=1e-12)


def test_gate_inversion_round_trip():
    d = O.make_inputs(1, 64, 2, 16, 16, seed=0)
    raw = O.invert_decay_gate(d["g"])
    back = O.decay_gate(raw, torch.zeros(2), torch.zeros(2, 16))
    assert (back - d["g"]).abs().max().item() < 1e-6


def test_one_token_zero_state_closed_form():
    gen = torch.Generator().manual_seed(1729)
    q = torch.randn(1, 1, 2, 4, generator=gen, dtype=torch.float64)
    k = torch.randn(1, 1, 2, 4, generator=gen, dtype=torch.float64)
    v = torch.randn(1, 1, 2, 3, generator=gen, dtype=torch.float64)
    g = -torch.rand(1, 1, 2, 4, generator=gen, dtype=torch.float64)
    beta = torch.rand(1, 1, 2, generator=gen, dtype=torch.float64)
    o, s = O.kda_recurrence(q, k, v, g, beta, compute_dtype=torch.float64)
    kn = k[0, 0] / k[0, 0].norm(dim=-1, keepdim=True)
    qn = q[0, 0] / q[0, 0].norm(dim=-1, keepdim=True) * 0.5
    want_s = beta[0, 0][:, None, None] * v[0, 0][:, :, None] * kn[:, None, :]     # [H,V,K]
    want_o = (want_s * qn[:, None, :]).sum(-1)
    assert torch.allclose(s[0], want_s, atol=1e-10, rtol=1e-10)
    assert torch.allclose(o[0, 0], want_o, atol=1e-10, rtol=1e-10)


def test_exact_key_overwrites_and_orthogonal_key_survives():
    state = torch.zeros(1, 1, 2, 2, dtype=torch.float64)
    state[0, 0, :, 0] = torch.tensor([3.0, -1.0])
    q = torch.tensor([[[[1.0, 0.0]], [[0.0, 1.0]]]], dtype=torch.float64)
    v = torch.tensor([[[[5.0, 7.0]], [[11.0, 13.0]]]], dtype=torch.float64)
    o, fs = O.kda_raw(q, q.clone(), v, torch.full_like(q, -100.0), torch.full((1, 2, 1), 100.0, dtype=torch.float64),
                      torch.zeros(1, dtype=torch.float64), torch.zeros(1, 2, dtype=torch.float64),
                      initial_state=state, compute_dtype=torch.float64)
    assert torch.allclose(fs[0, 0, :, 0], v[0, 0, 0], atol=1e-8)
    assert torch.allclose(fs[0, 0, :, 1], v[0, 1, 0], atol=1e-8)
    assert torch.isfinite(o).all()


def test_decay_is_applied_before_the_delta_correction():
    one = torch.ones(1, 1, 1, 1, dtype=torch.float64)
    o, fs = O.kda_raw(one, one.clone(), 10 * one, torch.zeros_like(one), torch.zeros(1, 1, 1, dtype=torch.float64),
                      torch.zeros(1, dtype=torch.float64), torch.zeros(1, 1, dtype=torch.float64),
                      initial_state=2 * one, compute_dtype=torch.float64)
    decayed = 2.0 * math.exp(-2.5)
    want = decayed + 0.5 * (10.0 - decayed)
    assert fs.item() == pytest.approx(want, rel=1e-12)
    assert o.item() == pytest.approx(want, rel=1e-12)


def test_causal_prefix_batch_independence_and_varlen():
    d = O.make_inputs(2, 9, 2, 4, 3, seed=11)
    full, _ = O.kda_recurrence(d["q"], d["k"], d["v"], d["g"], d["beta"])
    short, _ = O.kda_recurrence(*(d[n][:, :4] for n in ("q", "k", "v", "g", "beta")))
    assert torch.equal(full[:, :4], short)
    one, _ = O.kda_recurrence(*(d[n][1:2] for n in ("q", "k", "v", "g", "beta")))
    assert torch.allclose(full[1:2], one, atol=1e-7)
    # packed layout: two sequences of 9 tokens in one row
    packed = {n: d[n].reshape(1, 18, *d[n].shape[2:]) for n in d}
    po, ps = O.kda_recurrence_varlen(packed["q"], packed["k"], packed["v"], packed["g"], packed["beta"], [0, 9, 18])
    assert torch.allclose(po.reshape(2, 9, 2, 3), full, atol=1e-7)
    assert ps.shape == (2, 2, 3, 4)


CONV_TAGS = ["t9", "t9s", "t2s", "t4", "t70s", "t5w3"]


@pytest.mark.parametrize("tag", CONV_TAGS)
def test_conv_matches_reference_vectors(golden_dir, tag):
    d = _load(golden_dir, "conv")
    x = d[f"{tag}_x"].clone().requires_grad_(True)
    w = d[f"{tag}_w"].clone().requires_grad_(True)
    s0 = d[f"{tag}_s0"].clone().requires_grad_(True) if f"{tag}_s0" in d else None
    y, fs = O.causal_conv(x, w, initial_state=s0)
    assert torch.allclose(y, d[f"{tag}_y"], atol=2e-6, rtol=1e-5)
    assert torch.equal(fs, d[f"{tag}_fs"])
    assert torch.allclose(y, d[f"{tag}_prod_y"], atol=2e-6, rtol=1e-5)
    assert torch.allclose(fs, d[f"{tag}_prod_fs"])
    leaves = [x, w] + ([s0] if s0 is not None else [])
    gr = torch.autograd.grad((y, fs), leaves, (d[f"{tag}_cy"], d[f"{tag}_cs"]))
    assert torch.allclose(gr[0], d[f"{tag}_dx"], atol=1e-5, rtol=1e-5)
    assert torch.allclose(gr[1], d[f"{tag}_dw"], atol=1e-4, rtol=1e-5)
    if s0 is not None:
        assert torch.allclose(gr[2], d[f"{tag}_ds0"], atol=1e-5, rtol=1e-5)


def test_conv_full_sequence_equals_token_decode():
    gen = torch.Generator().manual_seed(99)
    x = torch.randn(2, 9, 6, generator=gen)
    w = torch.randn(6, 4, generator=gen)
    full, full_state = O.causal_conv(x, w)
    state, pieces = None, []
    for t in range(9):
        y, state = O.causal_conv(x[:, t:t + 1], w, initial_state=state)
        pieces.append(y)
    assert torch.allclose(torch.cat(pieces, 1), full, atol=1e-6)
    assert torch.equal(state, full_state)


@pytest.mark.parametrize("eps", [1e-5, 1e-6])
def test_rmsnorm_gated_matches_reference_vectors(golden_dir, eps):
    d = _load(golden_dir, "rmsnorm_gated")
    x = d["x"].clone().requires_grad_(True)
    gate = d["gate"].clone().requires_grad_(True)
    w = d["w"].clone().requires_grad_(True)
    y = O.rmsnorm_gated(x, gate, w, eps)
    tag = f"eps{eps:g}"
    assert torch.allclose(y, d[f"{tag}_y"], atol=1e-6, rtol=1e-5)
    gr = torch.autograd.grad(y, (x, gate, w), d[f"{tag}_cy"])
    for a, n in zip(gr, ("dx", "dgate", "dw")):
        assert torch.allclose(a, d[f"{tag}_{n}"], atol=1e-5, rtol=1e-5), n
    if eps == 1e-5:
        assert torch.allclose(y, d["prod_eps1e-05_y"], atol=1e-6, rtol=1e-5)
