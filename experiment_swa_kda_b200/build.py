"""In-tree build of libkda_b200.so for sm_100a with nvcc (cross-compiles without a GPU).

    python -m experiment_swa_kda_b200.build          # build if sources are newer than the library
    python -m experiment_swa_kda_b200.build --force

Plays the role of the reference's build loader (nanochat/research/cuda_build.py:116-181,
nanochat/mixers/cuda_kda/__init__.py:33-46): one shared library from the sources under csrc/,
with the exact compiler command recorded next to it (lib/build_receipt.json).
"""

from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libkda_b200.so")
RECEIPT = os.path.join(LIBDIR, "build_receipt.json")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps():
    inc = os.path.join(os.path.dirname(PKG), "include", "kda_b200.h")
    return sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")] + [inc]


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in _deps())


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libkda_b200.so")
    return cand


class _BuildLock:
    """One builder at a time: the ranks of a multi-process launch all find a stale library at once; the first one
    builds, the others wait on the lock and then find it fresh."""

    def __enter__(self):
        import fcntl
        os.makedirs(LIBDIR, exist_ok=True)
        self._f = open(os.path.join(LIBDIR, ".build.lock"), "w")
        fcntl.flock(self._f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl
        fcntl.flock(self._f, fcntl.LOCK_UN)
        self._f.close()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    with _BuildLock():
        if not force and not is_stale():      # another process built it while this one waited
            return LIB
        tmp = LIB + f".{os.getpid()}.tmp"      # never leave a half-written library where a loader can find it
        cmd = [nvcc_path(), *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "--shared", "-Xcompiler", "-fPIC",
               "-lcuda", "-o", tmp, *sources()]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
        os.replace(tmp, LIB)
        if verbose:
            sys.stderr.write(proc.stderr)
        cmd[cmd.index(tmp)] = LIB
        with open(RECEIPT, "w") as f:
            json.dump({"library_path": LIB, "source_paths": sources(), "compiler_command": cmd,
                       "target_arch": "sm_100a"}, f, indent=1)
    return LIB


# ----------------------------------------------------------------------------------------------
# the operator library: TORCH_LIBRARY(nanochat_kda) over the C ABI, compiled by the host compiler against the
# installed PyTorch (the role of torch.utils.cpp_extension.load(is_python_module=False) in the reference loader)
# ----------------------------------------------------------------------------------------------
SHIM_SRC = os.path.join(PKG, "torch_shim", "nanochat_kda_ops.cpp")
SHIM_LIB = os.path.join(LIBDIR, "libkda_b200_torch.so")


def torch_ops_stale() -> bool:
    if not os.path.exists(SHIM_LIB):
        return True
    t = os.path.getmtime(SHIM_LIB)
    inc = os.path.join(os.path.dirname(PKG), "include", "kda_b200.h")
    return os.path.getmtime(SHIM_SRC) > t or os.path.getmtime(inc) > t or os.path.getmtime(LIB) > t


def build_torch_ops(force: bool = False) -> str:
    build()
    if not force and not torch_ops_stale():
        return SHIM_LIB
    import torch
    from torch.utils import cpp_extension as ce
    cxx = shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise RuntimeError("no C++ compiler found: cannot build libkda_b200_torch.so")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(nvcc_path())), "include")
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
           "-I" + os.path.join(os.path.dirname(PKG), "include"), "-I" + cuda_inc, *["-I" + i for i in ce.include_paths()],
           SHIM_SRC, "-o", SHIM_LIB, "-L" + tlib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
           "-L" + LIBDIR, "-lkda_b200", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
    with _BuildLock():
        if not force and not torch_ops_stale():
            return SHIM_LIB
        tmp = SHIM_LIB + f".{os.getpid()}.tmp"
        cmd[cmd.index(SHIM_LIB)] = tmp
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("building libkda_b200_torch.so failed:\n" + proc.stdout + proc.stderr)
        os.replace(tmp, SHIM_LIB)
    return SHIM_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_torch_ops(force="--force" in sys.argv))
