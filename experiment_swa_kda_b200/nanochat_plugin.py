"""Plug the B200 kernels into the reference mixer as its `project_cuda` backend, leaving the reference's code untouched.

The reference resolves its protected backend through one module, `nanochat.mixers.cuda_kda`, of which it uses two
functions (nanochat/mixers/kda.py:366-380, 469-488): `prepare()`, which must leave `torch.ops.nanochat_kda.*`
registered natively, and `provenance()`, whose `components[name]` entries (`owner == "project"`, `torch_operator`)
tell `_project_operator` which operator to call.  `install()` puts a module with exactly those two functions in the
reference loader's place (reference nanochat/mixers/cuda_kda/__init__.py:33-132 builds the sm_121 sources there), so
that `GPT(GPTConfig(kda_backend="project_cuda"))`, `KimiDeltaAttention(mode="project_chunk")` and the decode path run on
this library while every line of nanochat/mixers/kda.py stays as it is.
"""

from __future__ import annotations

import sys
import types

MODULE = "nanochat.mixers.cuda_kda"


def _prepare() -> None:
    from . import nanochat_ops
    nanochat_ops.register()


def _provenance() -> dict:
    from .kda import kda_backend_provenance
    prov = kda_backend_provenance()
    prov.setdefault("schema_version", 1)
    return prov


def install() -> types.ModuleType:
    """Register the stand-in loader module (idempotent) and return it.  Call before the reference's
    `prepare_kda_backend("project_cuda")`; the reference package itself may be imported before or after."""
    mod = sys.modules.get(MODULE)
    if mod is not None and getattr(mod, "__kda_b200__", False):
        return mod
    mod = types.ModuleType(MODULE)
    mod.__doc__ = "libkda_b200 stand-in for the reference's CUDA build loader"
    mod.__kda_b200__ = True
    mod.prepare = _prepare
    mod.provenance = _provenance
    sys.modules[MODULE] = mod
    parent = sys.modules.get("nanochat.mixers")
    if parent is not None:
        setattr(parent, "cuda_kda", mod)
    return mod
