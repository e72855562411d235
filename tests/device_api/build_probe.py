"""Builds the test kernel that exercises the public device header (include/cubek_quant_b200_device.cuh) into a
shared object of its own, loaded only by the GPU test of that header."""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
PROBE_SRC = HERE / "probe.cu"
PROBE_LIB = HERE / "libdevice_api_probe.so"


def build_probe() -> Path:
    from cubek_b200.build import NVCC, NVCC_FLAGS

    deps = [PROBE_SRC, *sorted((ROOT / "include").glob("*"))]
    if not PROBE_LIB.exists() or any(d.stat().st_mtime > PROBE_LIB.stat().st_mtime for d in deps):
        cmd = [NVCC, *NVCC_FLAGS, "-shared", str(PROBE_SRC), "-o", str(PROBE_LIB), "-lcudart_static", "-ldl",
               "-lpthread", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {PROBE_SRC.name}:\n{res.stdout}\n{res.stderr}")
    return PROBE_LIB
