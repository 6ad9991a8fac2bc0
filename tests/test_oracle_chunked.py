"""The chunked WY restatement (forward and hand-derived backward) agrees with
autograd through the token recurrence; this is the algebra the CUDA kernels follow."""

import pytest
import torch

import kda_chunked as C
import kda_oracle as O


@pytest.mark.parametrize("T,K,V,chunk", [(150, 8, 6, 64), (64, 16, 16, 64), (37, 4, 5, 16), (1, 4, 3, 64)])
def test_chunked_forward_backward_float64(T, K, V, chunk):
    d = O.make_inputs(2, T, 2, K, V, seed=3, dtype=torch.float64, with_state=True)
    d["q"] = d["q"] * 2.5          # non-unit rows exercise the normalisation VJP
    d["k"] = d["k"] * 0.7
    d["g"] = d["g"] * 8
    d["h0"] = d["h0"].double() * 10
    leaf = {n: t.clone().requires_grad_(True) for n, t in d.items()}
    o, s = O.kda_recurrence(leaf["q"], leaf["k"], leaf["v"], leaf["g"], leaf["beta"], initial_state=leaf["h0"],
                            compute_dtype=torch.float64)
    gen = torch.Generator().manual_seed(1)
    do = torch.randn(o.shape, generator=gen, dtype=torch.float64)
    ds = torch.randn(s.shape, generator=gen, dtype=torch.float64)
    want = torch.autograd.grad((o, s), [leaf[n] for n in ("q", "k", "v", "g", "beta", "h0")], (do, ds))
    oc, sc, aux = C.chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], C=chunk)
    assert O.rel_l2(oc, o) < 1e-12 and O.rel_l2(sc, s) < 1e-12
    got = C.chunk_kda_backward(d["q"], d["k"], d["v"], d["g"], d["beta"], aux, do, ds)
    for n, a, e in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), got, want):
        assert O.rel_l2(a, e) < 1e-11, n
