"""`torch.ops.nanochat_kda.*`: the seven operators the reference mixer calls, registered natively.

The reference's loader compiles its sources into a shared library whose static initialisers register the operator
namespace with the dispatcher (nanochat/mixers/cuda_kda/__init__.py:33-46, TORCH_LIBRARY in recurrent_decode.cu:185-190
and the TORCH_LIBRARY_FRAGMENTs of the other files); `_project_operator` (nanochat/mixers/kda.py:374-380) then looks
the operators up by the names in the provenance table.  `register()` does the same for the B200 kernels: it builds
(when stale) and loads `lib/libkda_b200_torch.so` - `torch_shim/nanochat_kda_ops.cpp`, a TORCH_LIBRARY /
TORCH_LIBRARY_IMPL(CUDA) translation unit over the C ABI - with `torch.ops.load_library`.  Nothing is registered from
Python, and there is no CPU implementation: a CPU tensor fails in the dispatcher.

Schemas are the reference's, verbatim (chunk.cu:2118-2128, recurrent_decode.cu:186-189,
causal_convolution_forward.cu:242-243, causal_convolution_backward.cu:456-459, rmsnorm_gate.cu:278-282).
"""

from __future__ import annotations

import torch

from . import _lib, build

OPERATORS = ("chunk_forward", "chunk_backward", "recurrent_decode", "causal_convolution_forward",
             "causal_convolution_backward", "rmsnorm_gate_forward", "rmsnorm_gate_backward")
_LOADED = None


def register(build_if_missing: bool = True) -> str:
    """Load the operator library (once per process); returns its path."""
    global _LOADED
    if _LOADED is not None:
        return _LOADED
    _lib.load(build_if_missing=build_if_missing)       # libkda_b200.so first: the operator library links against it
    path = build.build_torch_ops() if build_if_missing else build.SHIM_LIB
    torch.ops.load_library(path)
    _LOADED = path
    return path


def schemas() -> dict:
    """Operator name -> schema string as the dispatcher holds it."""
    register()
    return {name: str(getattr(torch.ops.nanochat_kda, name).default._schema) for name in OPERATORS}
