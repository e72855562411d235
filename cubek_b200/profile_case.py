"""Runs a few fused-quantize + dequantize launches of one benchmark workload, optionally on a
reduced number of rows, so that a profiler can capture single launches on a small case.

    python -m cubek_b200.profile_case WORKLOAD [ROWS [ITERATIONS [LAYOUT]]]

LAYOUT is ``contiguous`` (default), ``transposed`` (the float tensors are `.t()` views of [cols, rows] matrices),
``slice`` (column slices of matrices 256 columns wider) or ``twocall`` (contiguous tensors through the reference-shaped
flow: compute_scales, quantize with given scales, dequantize).

e.g.  ncu --set full --clock-control none -k regex:^quantize_kernel -s 1 -c 1 -o report \
          python -m cubek_b200.profile_case q4_block32_bf16_14336x4096 32768 3
"""
from __future__ import annotations

import sys

import torch

from . import ComputeClient, TensorHandleRef, dequantize, quantize
from .synthetic import WORKLOADS, generate


def main(argv) -> None:
    w = WORKLOADS[argv[1]]
    rows = int(argv[2]) if len(argv) > 2 else w.shape[0]
    iters = int(argv[3]) if len(argv) > 3 else 3
    layout = argv[4] if len(argv) > 4 else "contiguous"
    s, cols = w.scheme, w.shape[1]
    x = generate(w, "cuda", rows=rows)

    def like(t):
        if layout == "transposed":
            return torch.empty((cols, rows), dtype=t.dtype, device="cuda").t()
        if layout == "slice":
            return torch.empty((rows, cols + 256), dtype=t.dtype, device="cuda")[:, 128:128 + cols]
        return torch.empty_like(t)

    if layout in ("transposed", "slice"):
        view = like(x)
        view.copy_(x)
        x = view
    code_dtype = torch.int32 if s.store.name == "U32" else torch.uint8
    codes = torch.empty(s.packed_shape((rows, cols)), dtype=code_dtype, device="cuda")
    scales = torch.empty(s.scales_shape((rows, cols)), dtype=torch.float32, device="cuda")
    out = like(x)
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    H, client = TensorHandleRef.from_torch, ComputeClient.current()
    given = torch.empty(s.scales_shape((rows, cols)), dtype=x.dtype, device="cuda")
    for _ in range(iters):
        if layout == "twocall":
            quantize.compute_scales(client, H(x), H(given), s, w.elem, H(ws))
            quantize.launch_ref(client, H(x), H(codes), H(given), H(scales), s, w.elem)
        else:
            quantize.launch_dynamic(client, H(x), H(codes), H(scales), s, w.elem, H(ws))
        dequantize.launch_ref(client, H(codes), H(out), H(scales), s, w.elem)
    torch.cuda.synchronize()
    print("ok", w.name, rows, float(out.float().abs().max()))


if __name__ == "__main__":
    main(sys.argv)
