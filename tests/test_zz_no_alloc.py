"""The scratch-free gated-RMSNorm backward (kda_rmsnorm_gate_bwd_static) against the regular entry point.

Meant for callers that cannot hand the library any scratch memory (fixed memory plans, plugins without an
allocator, paths that must not call cudaMalloc).  Called straight through the C ABI, twice in a row, because
the built-in scratch array keeps whatever the previous call left in it.  Collected last on purpose.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return t.data_ptr()


@pytest.mark.parametrize("rows,dim,dtype", [(24576, 128, torch.bfloat16), (301, 256, torch.float32), (50, 96, torch.bfloat16)])
def test_static_scratch_backward_matches_regular_entry_point(rows, dim, dtype):
    from experiment_swa_kda_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    io = _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_F32
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call in range(2):          # second call sees the first call's leftovers in the shared array
        gen = torch.Generator().manual_seed(100 * call + dim)
        x = torch.randn(rows, dim, generator=gen).to(dtype).to(dev)
        gate = torch.randn(rows, dim, generator=gen).to(dtype).to(dev)
        dy = torch.randn(rows, dim, generator=gen).to(dtype).to(dev)
        w = (1 + 0.1 * torch.randn(dim, generator=gen)).to(dev)
        y = torch.empty_like(x)
        inv = torch.empty(rows, dtype=torch.float32, device=dev)
        _lib.check(lib.kda_rmsnorm_gate_fwd(rows, dim, io, 1e-6, _ptr(x), _ptr(gate), _ptr(w), _ptr(y), _ptr(inv), stream),
                   "kda_rmsnorm_gate_fwd")
        ref = [torch.empty_like(x), torch.empty_like(x), torch.empty(dim, dtype=torch.float32, device=dev)]
        scr = torch.empty(lib.kda_rmsnorm_gate_bwd_scratch_bytes(rows, dim), dtype=torch.uint8, device=dev)
        _lib.check(lib.kda_rmsnorm_gate_bwd(rows, dim, io, _ptr(x), _ptr(gate), _ptr(w), _ptr(inv), _ptr(dy), _ptr(ref[0]),
                                            _ptr(ref[1]), _ptr(ref[2]), _ptr(scr), scr.numel(), stream), "kda_rmsnorm_gate_bwd")
        got = [torch.empty_like(x), torch.empty_like(x), torch.empty(dim, dtype=torch.float32, device=dev)]
        _lib.check(lib.kda_rmsnorm_gate_bwd_static(rows, dim, io, _ptr(x), _ptr(gate), _ptr(w), _ptr(inv), _ptr(dy),
                                                   _ptr(got[0]), _ptr(got[1]), _ptr(got[2]), stream),
                   "kda_rmsnorm_gate_bwd_static")
        torch.cuda.synchronize(dev)
        for a, b, name in zip(got, ref, ("dx", "dgate", "dweight")):
            assert torch.isfinite(a.float()).all(), name
            # same kernels, same summation order: identical bits
            assert torch.equal(a, b), name


def test_static_scratch_rejects_rows_wider_than_its_array():
    from experiment_swa_kda_b200 import _lib
    lib = _lib.load()
    rc = lib.kda_rmsnorm_gate_bwd_static(4, 512, _lib.DTYPE_F32, *([None] * 8), None)
    assert rc == -2
    assert b"unsupported" in lib.kda_error_string(rc)
