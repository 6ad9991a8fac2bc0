"""CPU-only checks of the drop-in boundary: the C-ABI library builds, loads and exports
every symbol include/kda_b200.h declares; host-side validation mirrors the reference's
error contract; no compute call is made (no GPU here)."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "kda_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from experiment_swa_kda_b200 import _lib
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/kda_b200.h but not exported"
    assert set(_lib.EXPORTED_SYMBOLS) == set(names)
    assert lib.kda_build_arch() == b"sm_100a"


def test_workspace_queries_and_error_strings():
    from experiment_swa_kda_b200 import _lib
    lib = _lib.load()
    sh = _lib.ChunkShape(2, 4096, 8192, 3, 128, 128, 1, 0, 0, 1, 0.0884)
    ws, scr = lib.kda_chunk_workspace_bytes(sh), lib.kda_chunk_bwd_scratch_bytes(sh)
    assert ws % 256 == 0 and scr % 256 == 0 and ws > 384 * 128 * 128 * 4
    packed = _lib.ChunkShape(5, 0, 263, 2, 32, 48, 0, 0, 0, 1, 0.1)
    assert lib.kda_chunk_workspace_bytes(packed) > 0
    assert b"workspace" in lib.kda_error_string(-3)
    # argument checks run before any CUDA call
    assert lib.kda_chunk_fwd(sh, *([None] * 10), 0, None) == -5
    bad = _lib.ChunkShape(2, 4096, 8192, 3, 512, 128, 1, 0, 0, 1, 0.1)
    assert lib.kda_chunk_fwd(bad, *([None] * 10), 0, None) == -1
    assert lib.kda_conv_fwd(1, 8, 4, 9, 0, 1, *([None] * 6)) in (-2, -5)
    assert lib.kda_rmsnorm_gate_bwd_scratch_bytes(24576, 128) > 0
    assert lib.kda_gate_bwd_scratch_bytes(8192, 3, 128) >= 2 * 128 * 384 * 4


def test_host_validation_matches_reference_contract():
    import experiment_swa_kda_b200 as m
    q = torch.randn(1, 2, 2, 4)
    v = torch.randn(1, 2, 2, 3)
    b = torch.randn(1, 2, 2)
    A, dt = torch.zeros(2), torch.zeros(2, 4)
    with pytest.raises(ValueError, match="unknown KDA mode"):
        m.kda(q, q, v, q, b, A, dt, mode="chunk")
    with pytest.raises(ValueError, match=r"V-first|\[B, H, V, K\]"):
        m.kda(q, q, v, q, b, A, dt, initial_state=torch.zeros(1, 2, 4, 3), mode="project_chunk")
    with pytest.raises(ValueError, match="A_log must have shape"):
        m.kda(q, q, v, q, b, torch.zeros(3), dt, mode="project_chunk")
    with pytest.raises(RuntimeError, match="project CUDA KDA backend unavailable: project KDA requires CUDA"):
        m.kda(q, q, v, q, b, A, dt, mode="project_chunk")          # fail closed: no CPU fallback
    with pytest.raises(RuntimeError, match="cannot fall back on CPU"):
        m.ShortConvolution(8, 4)(torch.randn(1, 3, 8))
    with pytest.raises(ValueError, match="convolution state must have shape"):
        m.ShortConvolution(8, 4)(torch.randn(1, 3, 8), torch.zeros(1, 8, 3))
    with pytest.raises(RuntimeError, match="cannot fall back on CPU"):
        m.RMSNormGated(8)(torch.randn(2, 8), torch.randn(2, 8))
    with pytest.raises(ValueError, match="hidden_size = num_heads"):
        m.KimiDeltaAttention(100, 3, 32)
    prov = m.kda_backend_provenance()
    assert prov["components"]["chunk_forward"]["torch_operator"] == "nanochat_kda::chunk_forward"
    assert all(c["owner"] == "project" for c in prov["components"].values())


def test_nanochat_kda_namespace_registers_the_reference_schemas():
    from experiment_swa_kda_b200 import nanochat_ops
    nanochat_ops.register()
    nanochat_ops.register()        # idempotent
    for name in ("chunk_forward", "chunk_backward", "recurrent_decode", "causal_convolution_forward",
                 "causal_convolution_backward", "rmsnorm_gate_forward", "rmsnorm_gate_backward"):
        op = getattr(torch.ops.nanochat_kda, name)
        assert op is not None
    schema = str(torch.ops.nanochat_kda.chunk_forward.default._schema)
    assert "Tensor? initial_state" in schema and "float lower_bound, float scale" in schema
    # no CPU kernel is registered: a CPU call fails closed instead of falling back
    x = torch.randn(1, 4, 8)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.nanochat_kda.causal_convolution_forward(x, torch.randn(8, 4), None, False)


def test_registered_schemas_carry_the_reference_return_names_and_the_trailing_cu_seqlens():
    from experiment_swa_kda_b200 import nanochat_ops
    s = nanochat_ops.schemas()
    assert s["chunk_forward"].endswith("float scale, Tensor? cu_seqlens=None) -> (Tensor output, Tensor? final_state)")
    assert "Tensor? cu_seqlens=None) -> (Tensor dq, Tensor dk, Tensor dv, Tensor draw_gate, Tensor dbeta_logits, " \
           "Tensor dA_log, Tensor ddt_bias, Tensor? dinitial_state)" in s["chunk_backward"]
    assert s["rmsnorm_gate_forward"].endswith("-> (Tensor output, Tensor inverse_rms)")
    assert s["causal_convolution_backward"].endswith("-> (Tensor dx, Tensor dweight, Tensor? dinitial_state)")


def test_operator_input_checks_run_before_any_launch():
    """The checks chunk_forward / chunk_backward / recurrent_decode apply before they touch the GPU
    (the role of the reference's validate_chunk_inputs, nanochat/mixers/cuda_kda/chunk.cu:1622-1663), driven through
    nanochat_kda::_validate_chunk_inputs, which is the same function and runs on tensors of any device."""
    from experiment_swa_kda_b200 import nanochat_ops
    nanochat_ops.register()
    check = torch.ops.nanochat_kda._validate_chunk_inputs
    B, T, H, K, V = 1, 5, 2, 8, 6
    bf = torch.bfloat16
    q, v, beta = torch.zeros(B, T, H, K, dtype=bf), torch.zeros(B, T, H, V, dtype=bf), torch.zeros(B, T, H, dtype=bf)
    A, bias = torch.zeros(H), torch.zeros(H, K)
    cases = {
        "shapes must match": (q, q[:, :4], v, q, beta, A, bias, None, -5.0),
        "v must match q": (q, q, v[:, :, :1], q, beta, A, bias, None, -5.0),
        r"beta_logits must have shape \[B, T, H\]": (q, q, v, q, beta[..., :1], A, bias, None, -5.0),
        r"A_log must be contiguous CUDA float32 \[H\]": (q, q, v, q, beta, torch.zeros(3), bias, None, -5.0),
        r"dt_bias must be contiguous CUDA float32 with H\*K elements": (q, q, v, q, beta, A, torch.zeros(H, K + 1), None, -5.0),
        r"initial_state must have shape \[B, H, V, K\]": (q, q, v, q, beta, A, bias, torch.zeros(B, H, K, V), -5.0),
        r"lower_bound must be in \[-5, 0\)": (q, q, v, q, beta, A, bias, None, -6.0),
        "activation tensors must be bfloat16": (q.float(), q.float(), v, q.float(), beta, A, bias, None, -5.0),
        "A_log and dt_bias must be float32": (q, q, v, q, beta, A.double(), bias, None, -5.0),
        "head dimensions must be in": (torch.zeros(B, T, H, 300, dtype=bf),) * 2 + (v, torch.zeros(B, T, H, 300, dtype=bf), beta, A,
                                                                                torch.zeros(H, 300), None, -5.0),
        # everything consistent, but nothing lives on a GPU: rejected, not handed to a kernel
        "q must be a CUDA tensor": (q, q, v, q, beta, A, bias, torch.zeros(B, H, V, K), -5.0),
    }
    for pattern, args in cases.items():
        with pytest.raises(RuntimeError, match=pattern):
            check(*args)
    with pytest.raises(RuntimeError, match=r"cu_seqlens must be int32 \[N\+1\]"):
        check(q, q, v, q, beta, A, bias, None, -5.0, torch.zeros(3, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="require batch size 1"):
        q2, v2, b2 = (t.repeat(2, *([1] * (t.dim() - 1))) for t in (q, v, beta))
        check(q2, q2, v2, q2, b2, A, bias, None, -5.0, torch.zeros(3, dtype=torch.int32))


def test_forward_only_shapes_need_less_workspace_and_refuse_a_backward():
    from experiment_swa_kda_b200 import _lib
    lib = _lib.load()
    train = _lib.ChunkShape(2, 4096, 8192, 3, 128, 128, 1, 0, 1, 1, 0.0884, 0)
    infer = _lib.ChunkShape(2, 4096, 8192, 3, 128, 128, 1, 0, 1, 1, 0.0884, 1)
    assert 0 < lib.kda_chunk_workspace_bytes(infer) < lib.kda_chunk_workspace_bytes(train)
    assert lib.kda_chunk_bwd(infer, *([None] * 9), 0, None, 0, *([None] * 7)) == -2
    bad = _lib.ChunkShape(2, 4096, 8192, 3, 128, 128, 1, 0, 1, 1, 0.0884, 7)
    assert lib.kda_chunk_fwd(bad, *([None] * 10), 0, None) == -1
    assert lib.kda_status_word_code(0) == 0 and lib.kda_status_word_code(10) == -7 and lib.kda_status_word_code(53) == -6
