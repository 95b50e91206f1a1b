"""Builds the shared libraries of ``csrc/`` in-tree with nvcc for sm_100a (no JIT cache, no torch
cpp_extension: each library is a plain C ABI loaded through ctypes).  One library per model family, so that
serving one family compiles only its own kernels: ``libdia_b200.so`` (Dia) and ``liblm_b200.so`` (the
decoder-only language models)."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = CSRC / "libdia_b200.so"
SOURCES = ["step_kernel.cu", "aux_kernels.cu", "gemm_tcgen05.cu", "prefill_kernels.cu", "batch_kernel.cu", "engine.cu"]
HEADERS = ["common.cuh", "engine_internal.h", "sampler.cuh", "gemm_tcgen05.h"]
LM_LIB = CSRC / "liblm_b200.so"
LM_SOURCES = ["lm_kernels.cu", "lm_mixers.cu", "lm_streams.cu", "lm_engine.cu", "gemm_tcgen05.cu"]          # the tensor-core GEMM is shared with Dia
LM_HEADERS = ["lm_internal.h", "lm_device.cuh", "gemm_tcgen05.h", "common.cuh", "engine_internal.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put /usr/local/cuda/bin on PATH)")


TARGETS = {
    "dia": (LIB, SOURCES, HEADERS, "dia_b200.h"),
    "lm": (LM_LIB, LM_SOURCES, LM_HEADERS, "lm_b200.h"),
}


def is_stale(target: str = "dia") -> bool:
    lib, sources, headers, public = TARGETS[target]
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = [CSRC / s for s in sources + headers] + [INCLUDE / public]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, target: str = "dia") -> Path:
    lib, sources, _, _ = TARGETS[target]
    if not force and not is_stale(target):
        return lib
    extra = os.environ.get("DIA_NVCC_EXTRA", "").split()          # e.g. -DDIA_BATCH_TRACE for a bring-up build
    # link to a name of our own first: another process that finds the library missing builds it too, and neither may
    # load a half-written file
    tmp = lib.with_name(f".{lib.name}.{os.getpid()}")
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, f"-I{INCLUDE}", "-o", str(tmp), *[str(CSRC / s) for s in sources]]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    if verbose:
        print(r.stderr)
    return lib


def build_all(force: bool = False, verbose: bool = False) -> list[Path]:
    return [build(force=force, verbose=verbose, target=t) for t in TARGETS]


if __name__ == "__main__":
    import sys
    for t in (sys.argv[1:] or list(TARGETS)):
        print(build(force=True, verbose=True, target=t))
