"""Builds the CUDA library in-tree: ``grad.cpp_b200/libgradb.so``.

nvcc cross-compiles for sm_100a without a GPU. The result is git-ignored and
travels to the GPU machine with the working tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libgradb.so"
LIB_DIAG = HERE / "libgradb_diag.so"  # the diagnostics build (csrc/gradb_diag.h): index checks, traces, test hooks
SOURCES = ["checkpoint.cpp", "model.cu", "step_kernels.cu", "attn_prefill.cu", "attn_prefill_tc.cu", "select_kernels.cu", "gemm_tc.cu", "decode_b1.cu", "session.cu", "capi.cu"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "--expt-extended-lambda"]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False, diagnostics: bool = False) -> Path:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "gradb.h"]
    objdir = HERE / "build" / ("diag" if diagnostics else "product")
    objdir.mkdir(parents=True, exist_ok=True)
    lib = LIB_DIAG if diagnostics else LIB
    flags = NVCC_FLAGS + (["-DGRADB_DIAGNOSTICS"] if diagnostics else [])
    objs, procs = [], []
    for src in SOURCES:
        obj = objdir / (src + ".o")
        objs.append(str(obj))
        if force or _stale(obj, [CSRC / src] + headers):
            cmd = [nvcc, *flags, "-c", str(CSRC / src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed = failed or p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not lib.exists():
        subprocess.run([nvcc, "-shared", "-o", str(lib), *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                       check=True)
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, diagnostics=True))
