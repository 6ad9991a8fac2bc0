"""Layer-level equivalences of KimiDeltaAttention on the GPU, mirroring the reference's layer tests
(tests/test_kda_layer.py:148-169 full sequence == token-by-token decode with conv caches, :172-193 non-zero incoming
KDAState and non-mutation, :231-248 gradients of the input and of every parameter), here against the composed CPU
oracle instead of "finite only".  The layer runs in bf16 with several cuBLAS GEMMs in series, so the bar is 3e-2
relative L2 (each stage alone is held to 1e-2 by the operator tests).
"""

import pytest
import torch

import kda_oracle as O

pytestmark = pytest.mark.gpu
D0 = "cuda:0"
LAYER_TOL = 3e-2
HID, HEADS, DIM = 256, 2, 128


def _layer(seed=0, eps=1e-6):
    from experiment_swa_kda_b200 import KimiDeltaAttention
    torch.manual_seed(seed)
    layer = KimiDeltaAttention(HID, HEADS, DIM, norm_eps=eps).to(D0)
    with torch.no_grad():
        layer.A_log.normal_(std=0.2)
        layer.dt_bias.normal_(std=0.3)
        layer.o_norm.weight.add_(0.1 * torch.randn_like(layer.o_norm.weight))
    return layer


def _oracle_layer(P, x, state=None, eps=1e-6):
    """The layer composed from the oracle pieces in float32 on the CPU, rounded to bf16 wherever the layer hands a
    bf16 tensor from one stage to the next.  P: name -> float32 tensors from _params_cpu (weights of
    the Linear and convolution modules already rounded to bf16, as the modules do).  Returns (y, (memory, q_conv, k_conv, v_conv))."""
    B, T, _ = x.shape
    rnd = lambda t: t.bfloat16().float()      # the layer hands bf16 tensors from stage to stage (identity for autograd)
    lin = lambda name, inp: rnd(inp @ P[name + ".weight"].t())
    sq, sk, sv, mem = (None, None, None, None) if state is None else (state[1], state[2], state[3], state[0])
    q, fq = O.causal_conv(lin("q_proj", x), P["q_conv1d.weight"].squeeze(1), initial_state=sq)
    k, fk = O.causal_conv(lin("k_proj", x), P["k_conv1d.weight"].squeeze(1), initial_state=sk)
    v, fv = O.causal_conv(lin("v_proj", x), P["v_conv1d.weight"].squeeze(1), initial_state=sv)
    sh = (B, T, HEADS, DIM)
    raw = lin("f_b_proj", lin("f_a_proj", x)).reshape(sh)
    bl = lin("b_proj", x)
    o, fm = O.kda_raw(rnd(q).reshape(sh), rnd(k).reshape(sh), rnd(v).reshape(sh), raw, bl, P["A_log"], P["dt_bias"], initial_state=mem)
    o = rnd(O.rmsnorm_gated(rnd(o), lin("g_proj", x).reshape(sh), P["o_norm.weight"], eps))
    return lin("o_proj", o.reshape(B, T, HID)), (fm, fq, fk, fv)


def _params_cpu(layer, grad=False):
    P = {}
    for n, p in layer.named_parameters():
        t = p.detach().float().cpu()
        if n.endswith("proj.weight") or n.endswith("conv1d.weight"):
            t = t.bfloat16().float()
        P[n] = t.clone().requires_grad_(grad)
    return P


def test_layer_full_sequence_equals_token_by_token_decode_with_conv_caches():
    layer = _layer(1).eval()
    x = torch.randn(2, 11, HID, generator=torch.Generator().manual_seed(19)).bfloat16().to(D0)
    with torch.no_grad():
        full, full_state = layer(x, state=None, output_final_state=True, mode="project_chunk")
        state, pieces = None, []
        for i in range(x.shape[1]):
            piece, state = layer(x[:, i:i + 1], state=state, output_final_state=True, mode="project_recurrent")
            pieces.append(piece)
    decoded = torch.cat(pieces, dim=1)
    assert O.rel_l2(decoded.float(), full.float()) <= 1e-2
    assert O.rel_l2(state.memory, full_state.memory) <= 1e-2
    # the conv caches hold the same projected inputs either way: bit-identical
    for a, b in ((state.q_conv, full_state.q_conv), (state.k_conv, full_state.k_conv), (state.v_conv, full_state.v_conv)):
        assert a.shape == (2, HID, 4) and torch.equal(a, b)


def test_layer_nonzero_incoming_state_matches_oracle_and_is_not_mutated():
    from experiment_swa_kda_b200 import KDAState
    layer = _layer(2)
    gen = torch.Generator().manual_seed(23)
    x = torch.randn(2, 70, HID, generator=gen).bfloat16().to(D0)
    state = KDAState(memory=(torch.randn(2, HEADS, DIM, DIM, generator=gen) * 0.1).to(D0),
                     q_conv=torch.randn(2, HID, 4, generator=gen).bfloat16().to(D0),
                     k_conv=torch.randn(2, HID, 4, generator=gen).bfloat16().to(D0),
                     v_conv=torch.randn(2, HID, 4, generator=gen).bfloat16().to(D0))
    keep = [t.clone() for t in (state.memory, state.q_conv, state.k_conv, state.v_conv)]
    with torch.no_grad():
        y, new = layer(x, state=state, output_final_state=True, mode="project_chunk")
        ye, (em, eq, ek, ev) = _oracle_layer(_params_cpu(layer), x.float().cpu(), tuple(t.float().cpu() for t in keep))
    for a, b in zip((state.memory, state.q_conv, state.k_conv, state.v_conv), keep):
        assert torch.equal(a, b)
    assert O.rel_l2(y.float(), ye) <= LAYER_TOL
    assert O.rel_l2(new.memory, em) <= LAYER_TOL
    for a, b in ((new.q_conv, eq), (new.k_conv, ek), (new.v_conv, ev)):
        assert O.rel_l2(a.float(), b) <= 1e-2


def test_layer_gradients_of_input_and_every_parameter_match_the_oracle_layer():
    layer = _layer(3)
    gen = torch.Generator().manual_seed(41)
    x = torch.randn(2, 130, HID, generator=gen).bfloat16().to(D0).requires_grad_(True)
    cot = torch.randn(2, 130, HID, generator=gen).bfloat16()
    y, _ = layer(x, state=None, output_final_state=False, mode="project_chunk")
    y.backward(cot.to(D0))
    P = _params_cpu(layer, grad=True)
    xe = x.detach().float().cpu().requires_grad_(True)
    ye, _ = _oracle_layer(P, xe)
    ye.backward(cot.float())
    assert O.rel_l2(y.float(), ye) <= LAYER_TOL
    errs = {"x": O.rel_l2(x.grad.float(), xe.grad)}
    for n, p in layer.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), n
        if n in ("A_log", "dt_bias"):
            # sums over every token and channel of signed bf16-level terms that largely cancel (the sum is ~1 % of the
            # summed magnitudes), so the bar is element-wise: the reference's 2e-2 for gate parameters
            # (configs/research/kda_cuda_ownership.toml:44-47) plus 5 % of the largest entry
            ref = P[n].grad
            assert (p.grad.float().cpu() - ref).abs().max() <= 5e-2 * ref.abs().max() + 2e-2, n
            continue
        errs[n] = O.rel_l2(p.grad.float(), P[n].grad)
    bad = {n: e for n, e in errs.items() if not e <= LAYER_TOL}
    assert not bad, f"layer gradients above {LAYER_TOL}: {bad} (all: {errs})"


def test_in_place_decode_token_equals_the_non_mutating_recurrent_path():
    """`decode_token` (one fused convolution-cache step, gate activations inside the decode kernel, memory rewritten in
    place: three library launches per token) against `forward(mode="project_recurrent")` (six launches, every state tensor
    reallocated): identical outputs and identical states after every token, starting from a non-trivial prefilled state."""
    from experiment_swa_kda_b200 import _lib
    layer = _layer(5).eval()
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(3, 40, HID, generator=gen).bfloat16().to(D0)
    with torch.no_grad():
        _, prefilled = layer(x[:, :33], state=None, output_final_state=True, mode="project_chunk")
        owned = prefilled.clone()
        ref_state = prefilled
        for i in range(33, 40):
            n0 = _lib.launch_count()
            want, ref_state = layer(x[:, i:i + 1], state=ref_state, output_final_state=True, mode="project_recurrent")
            n1 = _lib.launch_count()
            got = layer.decode_token(x[:, i:i + 1], owned)
            n2 = _lib.launch_count()
            assert (n2 - n1, n1 - n0) == (3, 6)
            assert torch.equal(got, want)
            for a, b in ((owned.memory, ref_state.memory), (owned.q_conv, ref_state.q_conv), (owned.k_conv, ref_state.k_conv),
                         (owned.v_conv, ref_state.v_conv)):
                assert torch.equal(a, b)


def test_no_grad_prefill_with_convolutions_inside_the_forward_kernel_equals_the_training_forward():
    """With `fuse_prefill_conv` set, a no_grad forward with no incoming state takes the fused prefill path (convolutions
    inside the intra-chunk kernel): output, memory and the three convolution caches equal those of the
    gradient-tracking forward, and decoding on from either state gives the same tokens."""
    layer = _layer(7).eval()
    x = torch.randn(2, 150, HID, generator=torch.Generator().manual_seed(5)).bfloat16().to(D0)
    from experiment_swa_kda_b200 import _lib
    with torch.no_grad():
        n0 = _lib.launch_count()
        layer(x[:, :143], state=None, output_final_state=True, mode="project_chunk")
        n1 = _lib.launch_count()
        layer.fuse_prefill_conv = True
        y_fused, st_fused = layer(x[:, :143], state=None, output_final_state=True, mode="project_chunk")
        n2 = _lib.launch_count()
        layer.fuse_prefill_conv = False
    assert n2 - n1 == (n1 - n0) - 3          # the three convolution launches are gone
    y_train, st_train = layer(x[:, :143].clone().requires_grad_(True), state=None, output_final_state=True, mode="project_chunk")
    assert torch.equal(y_fused, y_train.detach())
    for a, b in ((st_fused.memory, st_train.memory), (st_fused.q_conv, st_train.q_conv), (st_fused.k_conv, st_train.k_conv),
                 (st_fused.v_conv, st_train.v_conv)):
        assert torch.equal(a, b.detach())
    with torch.no_grad():
        a, _ = layer(x[:, 143:144], state=st_fused, output_final_state=True, mode="project_recurrent")
        b, _ = layer(x[:, 143:144], state=KDAStateDetach(st_train), output_final_state=True, mode="project_recurrent")
    assert torch.equal(a, b)


def KDAStateDetach(s):
    from experiment_swa_kda_b200 import KDAState
    return KDAState(s.memory.detach(), s.q_conv.detach(), s.k_conv.detach(), s.v_conv.detach())
