"""Builds the attention-stage shared library in-tree with nvcc for sm_100a.

    python -m glinthawk_b200.build [--force] [--verbose]

The result, ``glinthawk_b200/libglinthawk_attn.so``, exports the C ABI declared in ``include/glinthawk_attn.h``.
It links the CUDA runtime statically and resolves the few driver entry points it needs at run time, so it
loads on a machine without a GPU (where every compute entry point then reports an error status).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libglinthawk_attn.so"
SOURCES = ["attn_api.cu", "kv_pool.cu", "gh_driver.cu", "append_kernel.cu", "decode_generic.cu", "decode_mma.cu", "prefill_umma.cu",
           "qkv_umma.cu", "legacy_ops.cu", "decode_noalloc.cu", "router_api.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(obj: Path, src: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *headers])


def build(force: bool = False, verbose: bool = False) -> Path:
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.hh")) + sorted((PKG.parent / "include").glob("*.h"))
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs, procs = [], []
    for name in SOURCES:
        src, obj = CSRC / name, objdir / (name + ".o")
        objs.append(obj)
        if force or _stale(obj, src, headers):
            cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)]
            procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for name, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {name} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not LIB.exists():
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(LIB), *map(str, objs),
               "-cudart", "static"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
