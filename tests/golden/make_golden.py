"""Regenerate tests/golden/*.npz from the reference's own CPU code.

Run only where a checkout of the reference project is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's independent oracle (tests/kda_oracle.py) and its CPU
production loop (nanochat/mixers/kda.py, mode="reference") by path, feeds them
seeded inputs and stores inputs, outputs and gradients.  The fixtures are what
pins oracle/kda_oracle.py to the reference; the tests never need the reference
checkout themselves.
"""

from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def raw_inputs(seed, B, T, H, K, V, state=True):
    gen = torch.Generator().manual_seed(seed)
    d = {
        "q": torch.randn(B, T, H, K, generator=gen),
        "k": torch.randn(B, T, H, K, generator=gen),
        "v": torch.randn(B, T, H, V, generator=gen),
        "raw_gate": torch.randn(B, T, H, K, generator=gen),
        "beta_logits": torch.randn(B, T, H, generator=gen),
        "A_log": torch.randn(H, generator=gen) * 0.2,
        "dt_bias": torch.randn(H, K, generator=gen) * 0.3,
    }
    if state:
        d["initial_state"] = torch.randn(B, H, V, K, generator=gen) * 0.1
    d["cot_o"] = torch.randn(B, T, H, V, generator=gen)
    d["cot_s"] = torch.randn(B, H, V, K, generator=gen)
    return d


def main(ref_root):
    ref_oracle = _load(os.path.join(ref_root, "tests", "kda_oracle.py"), "ref_kda_oracle")
    sys.path.insert(0, ref_root)
    os.environ.setdefault("TORCH_COMPILE_DISABLE", "1")
    import importlib
    ref_kda = importlib.import_module("nanochat.mixers.kda")

    names = ("q", "k", "v", "raw_gate", "beta_logits", "A_log", "dt_bias", "initial_state")
    cases = [
        ("raw_b2_t7_h2_k4_v3", 1729, 2, 7, 2, 4, 3),
        ("raw_b1_t64_h2_k16_v11", 1730, 1, 64, 2, 16, 11),
        ("raw_b2_t65_h2_k16_v24", 1731, 2, 65, 2, 16, 24),
        ("raw_b1_t130_h2_k32_v32", 1732, 1, 130, 2, 32, 32),
    ]
    for tag, seed, B, T, H, K, V in cases:
        d = raw_inputs(seed, B, T, H, K, V)
        out = {n: t.numpy() for n, t in d.items()}
        for label, fn in (("oracle", None), ("prod", None)):
            leaf = {n: d[n].clone().requires_grad_(True) for n in names}
            if label == "oracle":
                o, s = ref_oracle.recurrent_kda(*(leaf[n] for n in names[:7]), initial_state=leaf["initial_state"])
            else:
                o, s = ref_kda.kda(*(leaf[n] for n in names[:7]), initial_state=leaf["initial_state"],
                                   output_final_state=True, mode="reference")
            grads = torch.autograd.grad((o, s), [leaf[n] for n in names], (d["cot_o"], d["cot_s"]))
            out[f"{label}_o"] = o.detach().numpy()
            out[f"{label}_s"] = s.detach().numpy()
            for n, gr in zip(names, grads):
                out[f"{label}_d_{n}"] = gr.numpy()
        np.savez_compressed(os.path.join(HERE, tag + ".npz"), **out)
        print("wrote", tag)

    # float64 run of one case: separates oracle rounding from implementation error
    d = raw_inputs(1733, 1, 70, 2, 8, 8)
    o, s = ref_oracle.recurrent_kda(*(d[n].double() for n in names[:7]), initial_state=d["initial_state"].double(),
                                    compute_dtype=torch.float64)
    out = {n: t.numpy() for n, t in d.items()}
    out["oracle_o"] = o.numpy(); out["oracle_s"] = s.numpy()
    np.savez_compressed(os.path.join(HERE, "raw_f64_b1_t70_h2_k8_v8.npz"), **out)

    # gate
    gen = torch.Generator().manual_seed(7)
    raw = torch.randn(2, 3, 2, 4, generator=gen, dtype=torch.float64)
    A = torch.randn(2, generator=gen, dtype=torch.float64)
    bias = torch.randn(2, 4, generator=gen, dtype=torch.float64)
    np.savez_compressed(os.path.join(HERE, "gate.npz"), raw=raw.numpy(), A_log=A.numpy(), dt_bias=bias.numpy(),
                        g=ref_oracle.k3_decay_gate(raw, A, bias).numpy(),
                        g_lb2=ref_oracle.k3_decay_gate(raw, A, bias, -2.0).numpy())

    # convolution: with / without cache, T < W, T == W, T > W
    conv = {}
    gen = torch.Generator().manual_seed(99)
    for tag, B, T, C, W, st in (("t9", 2, 9, 6, 4, False), ("t9s", 2, 9, 6, 4, True), ("t2s", 1, 2, 5, 4, True),
                                ("t4", 1, 4, 5, 4, False), ("t70s", 2, 70, 12, 4, True), ("t5w3", 1, 5, 4, 3, True)):
        x = torch.randn(B, T, C, generator=gen, requires_grad=True)
        w = torch.randn(C, W, generator=gen, requires_grad=True)
        s0 = torch.randn(B, C, W, generator=gen, requires_grad=True) if st else None
        y, fs = ref_oracle.causal_depthwise_conv(x, w, initial_state=s0)
        cy = torch.randn(y.shape, generator=gen)
        cs = torch.randn(fs.shape, generator=gen)
        leaves = [x, w] + ([s0] if st else [])
        grads = torch.autograd.grad((y, fs), leaves, (cy, cs))
        conv.update({f"{tag}_x": x.detach().numpy(), f"{tag}_w": w.detach().numpy(), f"{tag}_y": y.detach().numpy(),
                     f"{tag}_fs": fs.detach().numpy(), f"{tag}_cy": cy.numpy(), f"{tag}_cs": cs.numpy(),
                     f"{tag}_dx": grads[0].numpy(), f"{tag}_dw": grads[1].numpy()})
        if st:
            conv[f"{tag}_s0"] = s0.detach().numpy()
            conv[f"{tag}_ds0"] = grads[2].numpy()
        # the production module's CPU path (nn.Conv1d weights are [C,1,W])
        mod = ref_kda.ShortConvolution(C, W)
        with torch.no_grad():
            mod.weight.copy_(w.detach().unsqueeze(1))
        yp, fsp = mod(x.detach(), None if s0 is None else s0.detach(), output_final_state=True)
        conv[f"{tag}_prod_y"] = yp.detach().numpy()
        conv[f"{tag}_prod_fs"] = fsp.detach().numpy()
    np.savez_compressed(os.path.join(HERE, "conv.npz"), **conv)

    # gated RMSNorm
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(3, 5, 2, 16, generator=gen, requires_grad=True)
    gt = torch.randn(3, 5, 2, 16, generator=gen, requires_grad=True)
    w = (1 + 0.1 * torch.randn(16, generator=gen)).requires_grad_(True)
    norm = {}
    for eps in (1e-5, 1e-6):
        y = ref_oracle.rmsnorm_gated(x, gt, w, eps)
        cy = torch.randn(y.shape, generator=gen)
        gr = torch.autograd.grad(y, (x, gt, w), cy)
        tag = f"eps{eps:g}"
        norm.update({f"{tag}_y": y.detach().numpy(), f"{tag}_cy": cy.numpy(), f"{tag}_dx": gr[0].numpy(),
                     f"{tag}_dgate": gr[1].numpy(), f"{tag}_dw": gr[2].numpy()})
    mod = ref_kda.RMSNormGated(16, eps=1e-5)
    with torch.no_grad():
        mod.weight.copy_(w.detach())
    norm["prod_eps1e-05_y"] = mod(x.detach(), gt.detach()).detach().numpy()
    norm.update(x=x.detach().numpy(), gate=gt.detach().numpy(), w=w.detach().numpy())
    np.savez_compressed(os.path.join(HERE, "rmsnorm_gated.npz"), **norm)
    print("done")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
