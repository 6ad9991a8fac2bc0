"""ctypes binding of libkda_b200.so (the C ABI declared in include/kda_b200.h).

There is no fallback: if the library is missing, or an entry point returns an error
code, a RuntimeError is raised.
"""

from __future__ import annotations

import ctypes as C
import os

from . import build as _build

OK = 0
ERR_UNSUPPORTED = -2      # KDA_ERR_UNSUPPORTED
DTYPE_F32, DTYPE_BF16 = 0, 1
LANE_FP32, LANE_TC = 0, 1


class ChunkShape(C.Structure):
    _fields_ = [("n_seq", C.c_int32), ("seq_len", C.c_int32), ("tokens", C.c_int32), ("heads", C.c_int32),
                ("key_dim", C.c_int32), ("value_dim", C.c_int32), ("io_dtype", C.c_int32), ("gate_dtype", C.c_int32),
                ("lane", C.c_int32), ("l2norm", C.c_int32), ("scale", C.c_float), ("forward_only", C.c_int32)]


_P = C.c_void_p
_SIGNATURES = {
    "kda_error_string": (C.c_char_p, [C.c_int]),
    "kda_build_arch": (C.c_char_p, []),
    "kda_chunk_workspace_bytes": (C.c_size_t, [C.POINTER(ChunkShape)]),
    "kda_chunk_bwd_scratch_bytes": (C.c_size_t, [C.POINTER(ChunkShape)]),
    "kda_chunk_fwd": (C.c_int, [C.POINTER(ChunkShape)] + [_P] * 10 + [C.c_size_t, _P]),
    "kda_chunk_fwd_conv": (C.c_int, [C.POINTER(ChunkShape)] + [_P] * 6 + [C.c_int32, C.c_int32] + [_P] * 7 + [C.c_size_t, _P]),
    "kda_chunk_fwd_norm": (C.c_int, [C.POINTER(ChunkShape)] + [_P] * 10 + [C.c_size_t, _P, _P, C.c_float, _P, _P, _P]),
    "kda_chunk_bwd": (C.c_int, [C.POINTER(ChunkShape)] + [_P] * 9 + [C.c_size_t, _P, C.c_size_t] + [_P] * 7),
    "kda_chunk_status": (C.c_int, [C.POINTER(ChunkShape), _P, _P]),
    "kda_chunk_status_async": (C.c_int, [C.POINTER(ChunkShape), _P, _P, _P]),
    "kda_status_word_code": (C.c_int, [C.c_int32]),
    "kda_selftest_bounded_wait": (C.c_int, [_P, C.c_uint32, _P]),
    "kda_gate_fwd": (C.c_int, [C.c_int32] * 4 + [_P] * 4 + [C.c_float] + [_P] * 3),
    "kda_gate_bwd_scratch_bytes": (C.c_size_t, [C.c_int32] * 3),
    "kda_gate_bwd": (C.c_int, [C.c_int32] * 4 + [_P] * 4 + [C.c_float] + [_P] * 7 + [C.c_size_t, _P]),
    "kda_decode_step": (C.c_int, [C.c_int32] * 7 + [C.c_float] + [_P] * 9),
    "kda_decode_step_raw": (C.c_int, [C.c_int32] * 5 + [C.c_float] + [_P] * 7 + [C.c_float] + [_P] * 4),
    "kda_conv_step_multi": (C.c_int, [C.c_int32] * 6 + [_P] * 5),
    "kda_decode_steps": (C.c_int, [C.c_int32] * 8 + [C.c_float] + [_P] * 8),
    "kda_conv_fwd": (C.c_int, [C.c_int32] * 6 + [_P] * 6),
    "kda_conv_bwd_scratch_bytes": (C.c_size_t, [C.c_int32] * 4),
    "kda_conv_bwd": (C.c_int, [C.c_int32] * 6 + [_P] * 9 + [C.c_size_t, _P]),
    "kda_conv_fwd_multi": (C.c_int, [C.c_int32] * 7 + [_P] * 4),
    "kda_conv_bwd_multi_scratch_bytes": (C.c_size_t, [C.c_int32] * 5),
    "kda_conv_bwd_multi": (C.c_int, [C.c_int32] * 7 + [_P] * 6 + [C.c_size_t, _P]),
    "kda_rmsnorm_gate_fwd": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.c_float] + [_P] * 6),
    "kda_rmsnorm_gate_bwd_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "kda_rmsnorm_gate_bwd": (C.c_int, [C.c_int64, C.c_int32, C.c_int32] + [_P] * 9 + [C.c_size_t, _P]),
    "kda_rmsnorm_gate_bwd_static": (C.c_int, [C.c_int64, C.c_int32, C.c_int32] + [_P] * 9),
    "kda_launch_count": (C.c_ulonglong, []),
    "kda_profile_enable": (None, [C.c_int]),
    "kda_profile_report": (C.c_int, [C.c_char_p, C.c_size_t]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def library_path() -> str:
    return _build.LIB


def load(build_if_missing: bool = True):
    """Load (building first when sources are newer and nvcc is present) and return the CDLL."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("KDA_B200_LIB") or _build.LIB      # explicit library override (diagnostic builds)
    if path == _build.LIB and build_if_missing and _build.is_stale():
        try:
            _build.build()
        except RuntimeError:
            if not os.path.exists(path):
                raise
    if not os.path.exists(path):
        raise RuntimeError(f"KDA CUDA library not found at {path}; run `python -m experiment_swa_kda_b200.build`")
    lib = C.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError here means the library is stale
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != OK:
        msg = load().kda_error_string(code).decode()
        raise RuntimeError(f"{what} failed ({code}): {msg}")


def launch_count() -> int:
    return int(load().kda_launch_count())


def profile(on: bool) -> None:
    load().kda_profile_enable(1 if on else 0)


def profile_report() -> dict:
    """{kernel: (launches, total_ms)} of the launches recorded since profiling was enabled."""
    buf = C.create_string_buffer(1 << 16)
    load().kda_profile_report(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split(",")
        out[name] = (int(n), float(ms))
    return out
