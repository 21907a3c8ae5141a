"""Builds the CUDA library in-tree with nvcc for sm_100a (no other architecture).

    python -m <package>.build        or        from <package>.build import build_library

The shared object lands next to the sources (csrc/libsyfi_moe.so) so it is found
without installation.  Rebuilds only when a source is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
LIB = os.path.join(CSRC, "libsyfi_moe.so")
SOURCES = ["api.cu", "router.cu", "permute.cu", "grouped_gemm.cu", "grouped_gemm_pair.cu", "combine.cu", "ep_exchange.cu", "prepack.cu", "dsa_indexer.cu"]
HEADERS = ["moe_internal.h", "ptx.cuh", os.path.join("..", "..", "include", "syfi_moe.h"),
           os.path.join("..", "..", "include", "syfi_dsa.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the library cannot be built")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, *[os.path.join(CSRC, s) for s in SOURCES], "-o", LIB, "-lcudart"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building " + LIB)
    with open(os.path.join(CSRC, "build.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return LIB


TVMFFI_LIB = os.path.join(CSRC, "libsyfi_moe_tvmffi.so")


def build_tvm_ffi_binding(force: bool = False) -> str | None:
    """Builds csrc/libsyfi_moe_tvmffi.so, which exports the layer as ``__tvm_ffi_run_moe`` (the symbol
    the reference's harness loads).  Needs the tvm-ffi package for its headers and runtime; returns
    None when it is not installed.  The main library must have been built first."""
    try:
        import tvm_ffi
    except Exception:
        return None
    src = os.path.join(CSRC, "tvm_ffi_binding.cc")
    if (not force and os.path.exists(TVMFFI_LIB) and os.path.getmtime(TVMFFI_LIB) >= os.path.getmtime(src)
            and os.path.getmtime(TVMFFI_LIB) >= os.path.getmtime(LIB)):
        return TVMFFI_LIB
    root = os.path.dirname(tvm_ffi.__file__)
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I" + os.path.join(root, "include"),
           "-I" + os.path.join(root, "3rdparty", "dlpack", "include"), src, "-o", TVMFFI_LIB,
           "-L" + CSRC, "-lsyfi_moe", "-L" + os.path.join(root, "lib"), "-ltvm_ffi",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(root, "lib")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("g++ failed building " + TVMFFI_LIB)
    return TVMFFI_LIB


REPO_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_GPU_LIB = os.path.join(REPO_ROOT, "baseline", "_ref", "libref_moe.so")


def build_reference_gpu(force: bool = False) -> str | None:
    """Compiles the reference's own ``moe/solution/cuda/moe.cu`` — unmodified, straight from where it lies —
    for sm_100a into ``baseline/_ref/libref_moe.so`` (git-ignored; a measured baseline, never part of the
    product, see ``baseline/gpu_reference.py``).  The reference has no build file (its harness compiles
    the source with the tvm-ffi binding), so this is that one nvcc command.  The source is looked up in
    ``$SYFI_MOE_REFERENCE_SOURCE`` or in a ``reference`` checkout next to this repository; returns None
    when there is none (then an already built library is used as it is) or tvm-ffi is not installed."""
    src = os.environ.get("SYFI_MOE_REFERENCE_SOURCE") or os.path.join(
        os.path.dirname(REPO_ROOT), "reference", "moe", "solution", "cuda", "moe.cu")
    if not os.path.exists(src):
        return REF_GPU_LIB if os.path.exists(REF_GPU_LIB) else None
    try:
        import tvm_ffi
    except Exception:
        return None
    if not force and os.path.exists(REF_GPU_LIB) and os.path.getmtime(REF_GPU_LIB) >= os.path.getmtime(src):
        return REF_GPU_LIB
    root = os.path.dirname(tvm_ffi.__file__)
    os.makedirs(os.path.dirname(REF_GPU_LIB), exist_ok=True)
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w", "-Xcompiler", "-fPIC",
           "-shared", "-I" + os.path.join(root, "include"), "-I" + os.path.join(root, "3rdparty", "dlpack", "include"),
           src, "-o", REF_GPU_LIB, "-L" + os.path.join(root, "lib"), "-ltvm_ffi", "-lcuda",
           "-Xlinker", "-rpath", "-Xlinker", os.path.join(root, "lib")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("nvcc failed building " + REF_GPU_LIB)
    return REF_GPU_LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
    print(build_tvm_ffi_binding(force="--force" in sys.argv))
    print(build_reference_gpu(force="--force" in sys.argv))
