"""GPU parity of the tensor-core lane (K = V = 128, bf16 I/O) at the corners of its documented range.

The cases are the reference's own stress cases moved to the head size that selects the tcgen05 kernels: the
fixed-length boundary set (reference nanochat/research/cuda_worker.py:302-311), gates saturated at the lower bound
and raw logits of +-100 / +-30 (cuda_worker.py:324-329, tests/test_kda_cuda.py:176-190), and the campaign-shape
chain conv -> KDA -> gated RMSNorm with every gradient including the convolution and norm weights.
Tolerance: relative L2 <= 1e-2 against the float32 CPU oracle on the same (bf16-rounded) inputs.
"""

import pytest
import torch

import kda_oracle as O

pytestmark = pytest.mark.gpu
D0 = "cuda:0"
BF16_TOL = 1e-2


def _kda_mod():
    import experiment_swa_kda_b200 as m
    return m


def _run_activated(d, tol=BF16_TOL, cu=None):
    """chunk_kda(lane='tc') forward + backward against the oracle on the same rounded inputs."""
    m = _kda_mod()
    x = {n: (t.float() if n == "h0" else t.bfloat16()).to(D0).requires_grad_(True) for n, t in d.items()}
    cu_dev = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=D0)
    o, s = m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x.get("h0"), output_final_state=True,
                       cu_seqlens=cu_dev, lane="tc")
    gen = torch.Generator().manual_seed(17)
    do = torch.randn(o.shape, generator=gen).bfloat16().to(D0)
    ds = torch.randn(s.shape, generator=gen).to(D0)
    names = [n for n in ("q", "k", "v", "g", "beta", "h0") if n in x]
    grads = torch.autograd.grad((o, s), [x[n] for n in names], (do, ds))
    leaf = {n: x[n].detach().float().cpu().clone().requires_grad_(True) for n in names}
    if cu is None:
        eo, es = O.kda_recurrence(leaf["q"], leaf["k"], leaf["v"], leaf["g"], leaf["beta"], initial_state=leaf.get("h0"))
    else:
        eo, es = O.kda_recurrence_varlen(leaf["q"], leaf["k"], leaf["v"], leaf["g"], leaf["beta"], cu, initial_state=leaf.get("h0"))
    want = torch.autograd.grad((eo, es), [leaf[n] for n in names], (do.float().cpu(), ds.cpu()))
    assert torch.isfinite(o.float()).all() and torch.isfinite(s).all()
    errs = {"o": O.rel_l2(o.float(), eo), "s": O.rel_l2(s, es)}
    for n, a, b in zip(names, grads, want):
        assert torch.isfinite(a.float()).all(), n
        errs["d" + n] = O.rel_l2(a.float(), b)
    bad = {n: e for n, e in errs.items() if not e <= tol}
    assert not bad, f"rel-L2 above {tol}: {bad} (all: {errs})"
    return errs


@pytest.mark.parametrize("T", [1, 2, 3, 4, 63, 64, 65, 127, 128, 129, 257])
def test_boundary_lengths_tensor_core_lane(T):
    _run_activated(O.make_inputs(2, T, 2, 128, 128, seed=400 + T, with_state=True))


@pytest.mark.parametrize("pattern", ["all_saturated", "alternating_channels", "saturated_blocks"])
def test_saturated_gates_tensor_core_lane(pattern):
    """Log-decay at the lower bound g = -5 for whole chunks: 80 nats of decay inside one 16-row block, 320 inside a chunk.
    The per-block decay centre must keep both bf16 factors of every masked product in range."""
    d = O.make_inputs(1, 257, 2, 128, 128, seed=31, with_state=True)
    g = d["g"]
    if pattern == "all_saturated":
        g = torch.full_like(g, -5.0)
    elif pattern == "alternating_channels":
        g = g.clone()
        g[..., ::2] = -5.0                      # every other channel saturated, the rest mild
    else:
        g = g.clone()
        g[:, 64:128] = -5.0                     # one whole chunk saturated between mild chunks
        g[:, 200:216, :, :64] = -5.0            # one 16-row block of half the channels
    d["g"] = g
    _run_activated(d)


def test_scaled_gates_clamped_to_range_tensor_core_lane():
    """The usual gate distribution scaled by 40 and clamped to [-5, 0]: most channels at or near the bound."""
    d = O.make_inputs(2, 200, 2, 128, 128, seed=33, with_state=True)
    d["g"] = (d["g"] * 40.0).clamp(-5.0, 0.0)
    _run_activated(d)


def test_default_initialisation_gate_regime_keeps_the_decay_gradient_accurate():
    """g around -2.5 per token (raw gate logits near zero, where a freshly initialised layer sits): contexts are a few
    tokens long, so dg is a local quantity while the chunked pull-back builds it from row and column parts that must
    cancel over up to 64 rows.  Both parts are formed from the same bf16-rounded factors, which keeps dg - and its sum
    over tokens, the bias gradient of the gate - inside the bar instead of growing a random walk of rounding errors."""
    d = O.make_inputs(2, 256, 2, 128, 128, seed=5, with_state=True)
    d["g"] = (-5 * torch.sigmoid(torch.randn(d["g"].shape, generator=torch.Generator().manual_seed(9)) * 0.5)).clamp(-5, 0)
    m = _kda_mod()
    x = {n: (t.float() if n == "h0" else t.bfloat16()).to(D0).requires_grad_(True) for n, t in d.items()}
    o, s = m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True, lane="tc")
    do = torch.randn(o.shape, generator=torch.Generator().manual_seed(1)).bfloat16().to(D0)
    dg, = torch.autograd.grad(o, [x["g"]], do)
    leaf = {n: t.detach().float().cpu().requires_grad_(True) for n, t in x.items()}
    eo, _ = O.kda_recurrence(leaf["q"], leaf["k"], leaf["v"], leaf["g"], leaf["beta"], initial_state=leaf["h0"])
    want, = torch.autograd.grad(eo, [leaf["g"]], do.float().cpu())
    assert O.rel_l2(dg.float(), want) <= BF16_TOL
    assert O.rel_l2(dg.float().sum((0, 1)), want.sum((0, 1))) <= BF16_TOL      # what the gate's bias gradient sums


def _raw_inputs(T, D, seed, heads=2, batch=1, grad=True):
    gen = torch.Generator().manual_seed(seed)
    act = lambda *shape: torch.randn(*shape, generator=gen).to(torch.bfloat16).to(D0).requires_grad_(grad)
    q, k, v, g = (act(batch, T, heads, D) for _ in range(4))
    beta = act(batch, T, heads)
    A_log = (torch.randn(heads, generator=gen) * 0.2).to(D0).requires_grad_(grad)
    dt_bias = (torch.randn(heads, D, generator=gen) * 0.3).to(D0).requires_grad_(grad)
    h0 = (torch.randn(batch, heads, D, D, generator=gen) * 0.05).to(D0).requires_grad_(grad)
    return [q, k, v, g, beta, A_log, dt_bias, h0]


@pytest.mark.parametrize("magnitude", [100.0, 30.0])
def test_extreme_raw_gate_logits_tensor_core_lane(magnitude):
    """Raw gate logits of -m / +m on alternating channels (g = 0 and g = lower bound) through the raw surface at the
    head size that selects the tcgen05 kernels: forward and every gradient finite and inside the bf16 bar."""
    m = _kda_mod()
    t = _raw_inputs(257, 128, 3)
    with torch.no_grad():
        t[3][..., ::2].fill_(-magnitude)
        t[3][..., 1::2].fill_(magnitude)
    o, s = m.kda(*t[:7], initial_state=t[7], output_final_state=True, mode="project_chunk", lane="tc")
    gen = torch.Generator().manual_seed(5)
    co = torch.randn(o.shape, generator=gen).bfloat16()
    cs = torch.randn(s.shape, generator=gen)
    got = torch.autograd.grad((o, s), t, (co.to(D0), cs.to(D0)))
    e = [x.detach().float().cpu().clone().requires_grad_(True) for x in t]
    eo, es = O.kda_raw(*e[:7], initial_state=e[7])
    want = torch.autograd.grad((eo, es), e, (co.float(), cs))
    assert torch.isfinite(o.float()).all() and torch.isfinite(s).all()
    assert O.rel_l2(o.float(), eo) <= BF16_TOL and O.rel_l2(s, es) <= BF16_TOL
    names = ("q", "k", "v", "raw_gate", "beta_logits", "A_log", "dt_bias", "initial_state")
    for n, a, b in zip(names, got, want):
        assert torch.isfinite(a.float()).all(), n
        if n in ("raw_gate", "A_log", "dt_bias"):
            # the sigmoid is saturated: these gradients are ~0 on both sides; compare absolutely at the reference's bar
            torch.testing.assert_close(a.float().cpu(), b, atol=2e-2, rtol=2e-2)
        else:
            assert O.rel_l2(a.float(), b) <= BF16_TOL, n


def test_backward_twice_with_retained_graph_gives_identical_gradients():
    m = _kda_mod()
    d = O.make_inputs(1, 130, 2, 128, 128, seed=8, with_state=True)
    x = {n: (t.float() if n == "h0" else t.bfloat16()).to(D0).requires_grad_(True) for n, t in d.items()}
    o, s = m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True)
    loss = o.float().sum() + s.sum()
    first = torch.autograd.grad(loss, list(x.values()), retain_graph=True)
    second = torch.autograd.grad(loss, list(x.values()))
    for a, b in zip(first, second):
        assert torch.equal(a, b)


def test_non_finite_tokens_of_the_next_packed_sequence_do_not_leak_into_a_ragged_tail():
    """Two packed sequences; the second one is all NaN.  The first sequence's outputs and gradients (its ragged last
    chunk shares 64-row tiles with the second sequence's tokens) must equal those of the first sequence run alone."""
    m = _kda_mod()
    d = O.make_inputs(1, 100 + 60, 2, 128, 128, seed=41)
    x = {n: t.bfloat16().to(D0) for n, t in d.items()}
    for n in x:
        x[n][:, 100:] = float("nan")
    cu = torch.tensor([0, 100, 160], dtype=torch.int32, device=D0)
    xs = {n: t.clone().requires_grad_(True) for n, t in x.items()}
    o, _ = m.chunk_kda(xs["q"], xs["k"], xs["v"], xs["g"], xs["beta"], cu_seqlens=cu, lane="tc")
    do = torch.ones_like(o)
    do[:, 100:] = 0
    grads = torch.autograd.grad(o, list(xs.values()), do)
    alone = {n: t[:, :100].clone().requires_grad_(True) for n, t in x.items()}
    oa, _ = m.chunk_kda(alone["q"], alone["k"], alone["v"], alone["g"], alone["beta"], lane="tc")
    ga = torch.autograd.grad(oa, list(alone.values()), torch.ones_like(oa))
    assert torch.equal(o[:, :100], oa)
    for a, b in zip(grads, ga):
        assert torch.equal(a[:, :100], b)


@pytest.mark.parametrize("T", [2048 + 64 * 3 + 17, 1024 + 64 * 4 + 5])      # 36 chunks -> 4 segments, 21 chunks -> 2 segments
def test_split_scans_agree_with_the_single_chain_and_the_oracle(T):
    """A long fixed-length batch with few (sequence, head) recurrences runs every state scan as 2 nseg - 1 units side by
    side (segment 0 from the true state; every later segment once from zero and once as composite maps) plus a
    chunk-parallel fix-up that walks the short chain of segment-start states itself; the same tokens handed over as a
    packed batch (cu_seqlens) take the single chain.  Both must agree with each other closely and with the oracle inside
    the bar: outputs, final state (non-zero initial state, ragged tail) and every gradient."""
    m = _kda_mod()
    d = O.make_inputs(1, T, 2, 128, 128, seed=91, with_state=True)
    gen = torch.Generator().manual_seed(4)
    do = torch.randn(1, T, 2, 128, generator=gen).bfloat16().to(D0)
    ds = torch.randn(1, 2, 128, 128, generator=gen).to(D0)
    res = []
    for packed in (False, True):
        x = {n: (t.float() if n == "h0" else t.bfloat16()).to(D0).requires_grad_(True) for n, t in d.items()}
        cu = torch.tensor([0, T], dtype=torch.int32, device=D0) if packed else None
        o, s = m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True,
                           cu_seqlens=cu, lane="tc")
        res.append((o, s, torch.autograd.grad((o, s), list(x.values()), (do, ds))))
    (o1, s1, g1), (o2, s2, g2) = res
    assert O.rel_l2(o1.float(), o2.float()) <= 4e-3 and O.rel_l2(s1, s2) <= 4e-3
    for a, b in zip(g1, g2):
        assert O.rel_l2(a.float(), b.float()) <= 6e-3
    _run_activated(d)                           # the split path against the oracle


@pytest.mark.parametrize("lens,H", [([64 * 40 + 5, 30, 64 * 70 + 1], 2),          # 6 recurrences, mean 37 chunks -> 4 segments
                                    ([64 * 60 + 3, 0, 64 * 99, 1], 3),             # 12 recurrences, mean 39 chunks -> 4 segments
                                    ([64 * 50, 64 * 3 + 9, 0, 64 * 19 + 63], 4)])  # 16 recurrences, mean 18 chunks -> 2 segments
def test_split_scans_on_packed_batches_with_short_and_empty_sequences(lens, H):
    """Packed batches with few sequences split their scans too (the decision uses the mean length), so a batch mixes long
    sequences with ones of a single chunk or none: segments of one chunk or zero chunks, composite maps that stay the
    identity, local states that stay zero.  Outputs, final states (non-zero initial states) and every gradient against
    the oracle, sequence by sequence."""
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    d = O.make_inputs(1, cu[-1], H, 128, 128, seed=300 + H, with_state=True, n_states=len(lens))
    _run_activated(d, cu=cu)


@pytest.mark.parametrize("lens,H,wdtype", [([300], 2, torch.float32), ([1], 1, torch.float32), ([3, 64, 65, 130, 2], 3, torch.bfloat16),
                                           ([64 * 34 + 7, 5], 2, torch.float32)])
def test_convolutions_inside_the_forward_kernel_equal_convolutions_then_forward(lens, H, wdtype):
    """kda_chunk_fwd_conv (q, k, v never written to memory: the intra-chunk kernel forms them from the convolutions'
    inputs, reading the three rows before a chunk from the previous chunk of the same sequence and zeros at a sequence
    start) against the three stand-alone convolutions followed by the forward-only chunk forward: identical output and
    final state, bit for bit, over one-token, sub-chunk, chunk-boundary, multi-chunk and split-scan lengths, fixed and
    packed layouts, float32 and bf16 weights."""
    from experiment_swa_kda_b200 import ops, _lib
    gen = torch.Generator().manual_seed(sum(lens) + H)
    T, C = sum(lens), H * 128
    edges = [0]
    for n in lens:
        edges.append(edges[-1] + n)
    cu = torch.tensor(edges, dtype=torch.int32, device=D0) if len(lens) > 1 else None
    d = O.make_inputs(1, T, H, 128, 128, seed=7 + T, with_state=True, n_states=len(lens))
    g, beta, h0 = d["g"].bfloat16().to(D0), d["beta"].bfloat16().to(D0), d["h0"].float().to(D0)
    xs = [torch.randn(1, T, C, generator=gen).bfloat16().to(D0) for _ in range(3)]
    ws = [((torch.rand(C, 4, generator=gen) * 2 - 1) * 0.5).to(wdtype).to(D0) for _ in range(3)]
    # reference: each sequence convolved on its own (zero padding at its start), then the forward-only chunk forward
    acts = []
    for x, w in zip(xs, ws):
        parts = [ops.conv_fwd(x[:, a:b].contiguous(), w, None, False)[0] for a, b in zip(edges[:-1], edges[1:]) if b > a]
        acts.append(torch.cat(parts, 1).reshape(1, T, H, 128))
    want_o, want_s, _ = ops.chunk_kda_fwd(acts[0], acts[1], acts[2], g, beta, h0, cu, 128 ** -0.5, True, True, _lib.LANE_TC, forward_only=True)
    got_o, got_s = ops.chunk_kda_conv_fwd(xs[0].reshape(1, T, H, 128), xs[1].reshape(1, T, H, 128), xs[2].reshape(1, T, H, 128), *ws, g, beta,
                                          h0, cu, 128 ** -0.5, True, True)
    assert torch.equal(got_o, want_o) and torch.equal(got_s, want_s)


def test_output_norm_in_the_chunk_output_epilogue_equals_the_two_operators_in_sequence():
    """chunk_kda_norm (gated RMSNorm applied to the output tile inside the chunk-output kernel) against chunk_kda followed
    by RMSNormGated: identical y, final state and gradients (the epilogue repeats the stand-alone kernel's arithmetic),
    one library launch less; ragged packed batch with states."""
    from experiment_swa_kda_b200 import _lib
    m = _kda_mod()
    cu = [0, 70, 199, 200, 333]
    d = O.make_inputs(1, 333, 2, 128, 128, seed=77, with_state=True, n_states=4)
    gen = torch.Generator().manual_seed(2)
    gate = torch.randn(1, 333, 2, 128, generator=gen).bfloat16().to(D0)
    nw = (1 + 0.1 * torch.randn(128, generator=gen)).to(D0)
    cy = torch.randn(1, 333, 2, 128, generator=gen).bfloat16().to(D0)
    cu_dev = torch.tensor(cu, dtype=torch.int32, device=D0)
    outs, counts = [], []
    for fused in (True, False):
        x = {n: (t.float() if n == "h0" else t.bfloat16()).to(D0).requires_grad_(True) for n, t in d.items()}
        gt, w = gate.clone().requires_grad_(True), nw.clone().requires_grad_(True)
        n0 = _lib.launch_count()
        if fused:
            y, s = m.chunk_kda_norm(x["q"], x["k"], x["v"], x["g"], x["beta"], gt, w, eps=1e-6, initial_state=x["h0"],
                                    output_final_state=True, cu_seqlens=cu_dev)
        else:
            o, s = m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True,
                               cu_seqlens=cu_dev)
            norm = m.RMSNormGated(128, eps=1e-6).to(D0)
            norm.weight = torch.nn.Parameter(w.detach().clone())
            y = norm(o, gt)
            w = norm.weight
        counts.append(_lib.launch_count() - n0)
        grads = torch.autograd.grad((y, s), list(x.values()) + [gt, w], (cy, torch.ones_like(s)))
        outs.append((y, s, grads))
    assert counts[0] == counts[1] - 1
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    for a, b in zip(outs[0][2], outs[1][2]):
        assert torch.equal(a, b)
    # and against the oracle
    leaf = {n: (t.float() if n == "h0" else t.bfloat16().float()) for n, t in d.items()}
    eo, _ = O.kda_recurrence_varlen(leaf["q"], leaf["k"], leaf["v"], leaf["g"], leaf["beta"], cu, initial_state=leaf["h0"])
    ey = O.rmsnorm_gated(eo, gate.float().cpu(), nw.cpu(), 1e-6)
    assert O.rel_l2(outs[0][0].float(), ey) <= BF16_TOL


# ---------------------------------------------------------------------------------- the campaign chain, full size
def test_config1_chain_full_shape_every_gradient():
    """B2 T4096 H3 D128 bf16: short conv (width 4, SiLU) on q/k/v -> chunked KDA -> gated RMSNorm (eps 1e-6) through the
    public modules, forward and backward, against the composed float32 oracle: y and the gradients of the three conv
    inputs, g, beta, the norm gate, the three convolution weights and the norm weight."""
    m = _kda_mod()
    B, T, H, D, W = 2, 4096, 3, 128, 4
    C = H * D
    gen = torch.Generator().manual_seed(1234)
    bf = torch.bfloat16
    host = {
        "xq": torch.randn(B, T, C, generator=gen).to(bf), "xk": torch.randn(B, T, C, generator=gen).to(bf),
        "xv": torch.randn(B, T, C, generator=gen).to(bf),
        "g": (-torch.nn.functional.softplus(torch.randn(B, T, H, D, generator=gen)) * 0.1).clamp(-5, 0).to(bf),
        "beta": torch.sigmoid(torch.randn(B, T, H, generator=gen)).to(bf),
        "gate": torch.randn(B, T, H, D, generator=gen).to(bf),
    }
    probe = torch.randn(B, T, H, D, generator=gen).to(bf)
    bound = (3 ** 0.5) * C ** -0.5
    ws = [((torch.rand(C, W, generator=gen) * 2 - 1) * bound) for _ in range(3)]
    nw = 1 + 0.1 * torch.randn(D, generator=gen)
    convs = [m.ShortConvolution(C, W).to(D0) for _ in range(3)]
    for c, w in zip(convs, ws):
        with torch.no_grad():
            c.weight.copy_(w.unsqueeze(1))
    norm = m.RMSNormGated(D, eps=1e-6).to(D0)
    with torch.no_grad():
        norm.weight.copy_(nw)
    x = {n: t.to(D0).requires_grad_(True) for n, t in host.items()}
    q, k, v = (t.view(B, T, H, D) for t in m.short_convolutions(convs, (x["xq"], x["xk"], x["xv"])))
    o, _ = m.chunk_kda(q, k, v, x["g"], x["beta"])
    y = norm(o, x["gate"])
    leaves = [x[n] for n in host] + [c.weight for c in convs] + [norm.weight]
    got = torch.autograd.grad(y, leaves, probe.to(D0))

    e = {n: t.float().clone().requires_grad_(True) for n, t in host.items()}
    ew = [w.to(bf).float().requires_grad_(True) for w in ws]       # the modules round their weights to the activation dtype
    enw = nw.clone().requires_grad_(True)
    eq, ek, ev = (O.causal_conv(e[n], w)[0].view(B, T, H, D) for n, w in zip(("xq", "xk", "xv"), ew))
    eo, _ = O.kda_recurrence(eq, ek, ev, e["g"], e["beta"])
    ey = O.rmsnorm_gated(eo, e["gate"], enw, 1e-6)
    want = torch.autograd.grad(ey, [e[n] for n in host] + ew + [enw], probe.float())
    assert O.rel_l2(y.float(), ey) <= BF16_TOL
    names = list(host) + ["wq", "wk", "wv", "norm_weight"]
    errs = {}
    for n, a, b in zip(names, got, want):
        a = a.float().cpu()
        errs[n] = O.rel_l2(a.reshape(b.shape), b)
    bad = {n: v_ for n, v_ in errs.items() if not v_ <= BF16_TOL}
    assert not bad, f"chain gradients above {BF16_TOL}: {bad} (all: {errs})"
