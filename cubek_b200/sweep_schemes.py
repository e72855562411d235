"""Throughput of every stored-code kind x float type x level through the batch entry points, as a table.

    python -m cubek_b200.sweep_schemes [TENSORS [ITERATIONS]]

Each case quantizes (fused) and dequantizes a batch of TENSORS (default 8) tensors of 117 MB (14336 x 4096 for the
16-bit types, 7168 x 4096 for f32) ITERATIONS (default 30) times between two CUDA events; the figures are
algorithmic GB/s (input + codes + scales, and back)."""
from __future__ import annotations

import itertools
import sys

import torch

from . import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef, dequantize,
               quantize)

TORCH = {ElemType.F32: torch.float32, ElemType.F16: torch.float16, ElemType.BF16: torch.bfloat16}
KINDS = [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4S, QuantStore.U32), (QuantValue.Q2S, QuantStore.U32),
         (QuantValue.Q8S, QuantStore.Native), (QuantValue.E2M1, QuantStore.Native), (QuantValue.E4M3, QuantStore.Native),
         (QuantValue.E5M2, QuantStore.Native)]
LEVELS = [("block 32", QuantLevel.block([32])), ("block 128", QuantLevel.block([128])), ("tensor", QuantLevel.Tensor)]


def timed(fn, iterations: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iterations):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iterations


def main(argv) -> None:
    tensors = int(argv[1]) if len(argv) > 1 else 8
    iterations = int(argv[2]) if len(argv) > 2 else 30
    H, client = TensorHandleRef.from_torch, ComputeClient.current()
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    print("| float | value | store | level | fused quantize GB/s | dequantize GB/s |")
    print("|---|---|---|---|---|---|")
    for elem in (ElemType.F32, ElemType.F16, ElemType.BF16):
        rows = 7168 if elem == ElemType.F32 else 14336
        xs = [torch.randn((rows, 4096), device="cuda", dtype=torch.float32).to(TORCH[elem]) for _ in range(tensors)]
        for (value, store), (level_name, level) in itertools.product(KINDS, LEVELS):
            s = QuantScheme(value=value, store=store, level=level)
            code_t = torch.int32 if store == QuantStore.U32 else torch.uint8
            codes = [torch.empty(s.packed_shape(x.shape), dtype=code_t, device="cuda") for x in xs]
            scales = [torch.empty(s.scales_shape(x.shape), dtype=torch.float32, device="cuda") for x in xs]
            outs = [torch.empty_like(x) for x in xs]
            q = quantize.PreparedDynamicBatch(client, [H(x) for x in xs], [H(c) for c in codes], [H(t) for t in scales],
                                              s, elem, H(ws))
            d = dequantize.PreparedBatch(client, [H(c) for c in codes], [H(o) for o in outs], [H(t) for t in scales], s, elem)
            n, esz = xs[0].numel(), xs[0].element_size()
            code_bytes = codes[0].numel() * codes[0].element_size()
            scale_bytes = scales[0].numel() * 4
            q_bytes = tensors * (n * esz * (2 if level.is_tensor else 1) + code_bytes + scale_bytes)
            d_bytes = tensors * (code_bytes + scale_bytes + n * esz)
            print(f"| {elem.name.lower()} | {value.name} | {store.name} | {level_name} | "
                  f"{q_bytes / timed(q, iterations) / 1e6:.0f} | {d_bytes / timed(d, iterations) / 1e6:.0f} |")


if __name__ == "__main__":
    main(sys.argv)
