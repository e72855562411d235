"""Builds libcubek_quant_b200.so (sm_100a) in-tree with nvcc.

Run as ``python -m cubek_b200.build``.  Objects are compiled in parallel, one nvcc
process per translation unit, and linked into ``cubek_b200/libcubek_quant_b200.so``.
A source is recompiled only when it or a header is newer than its object.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "csrc" / "build"
LIB = PKG / "libcubek_quant_b200.so"
# The same library with `round` = halves away from zero (-DQK_ROUND_HALF_AWAY): the reference leaves the rounding
# of exact .5 ties to its JIT back end, so both lowerings are built and tested.
LIB_HALF_AWAY = PKG / "libcubek_quant_b200_half_away.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-ccbin", "g++",
]


def _sources():
    return sorted(CSRC.glob("*.cu"))


def _headers():
    inc = PKG.parent / "include"
    return sorted(CSRC.glob("*.cuh")) + sorted(inc.glob("*.h")) + sorted(inc.glob("*.cuh"))


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, verbose: bool, half_away: bool = False) -> Path:
    obj = BUILD / (src.stem + (".half_away.o" if half_away else ".o"))
    if _stale(obj, [src, *_headers()]):
        cmd = [NVCC, *NVCC_FLAGS, *(["-DQK_ROUND_HALF_AWAY"] if half_away else []), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose and not half_away:
            (BUILD / (src.stem + ".ptxas.txt")).write_text(res.stderr)
    return obj


def build(verbose: bool = False, force: bool = False, half_away: bool = False) -> Path:
    """Builds the library (or, with ``half_away``, its round-half-away-from-zero variant) and returns its path."""
    BUILD.mkdir(parents=True, exist_ok=True)
    lib = LIB_HALF_AWAY if half_away else LIB
    if force:
        for o in BUILD.glob("*.half_away.o" if half_away else "*.o"):
            if half_away or not o.name.endswith(".half_away.o"):
                o.unlink()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, half_away), _sources()))
    if _stale(lib, objs):
        cmd = [NVCC, "-shared", "-o", str(lib), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "g++",
               "-Xcompiler", "-fPIC", "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, half_away="--round-half-away" in sys.argv)
    print(path)
