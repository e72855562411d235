"""Seeded synthetic inputs with the shapes and value distributions of the benchmark workloads.

No dataset is involved anywhere on this path: the workloads are defined by a shape, a float
type and a distribution, which are reproduced here from a counter-based generator.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Tuple

import torch

from .scheme import ElemType, QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue

TORCH_DTYPE = {ElemType.F32: torch.float32, ElemType.F16: torch.float16, ElemType.BF16: torch.bfloat16}
SEED_BASE = 0x5EED0000


@dataclass(frozen=True)
class Workload:
    name: str
    shape: Tuple[int, int]
    elem: ElemType
    scheme: QuantScheme
    distribution: str
    index: int


def _block(value, block, store=QuantStore.U32):
    return QuantScheme(value=value, store=store, param=QuantParam.F32, level=QuantLevel.block([block]))


WORKLOADS = {
    "q8_tensor_f32_4096x4096": Workload(
        "q8_tensor_f32_4096x4096", (4096, 4096), ElemType.F32,
        QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32, param=QuantParam.F32), "normal(0,1)", 0),
    "q4_block32_bf16_14336x4096": Workload(
        "q4_block32_bf16_14336x4096", (14336, 4096), ElemType.BF16, _block(QuantValue.Q4S, 32),
        "normal(0,0.02) with 0.1% outliers x20", 1),
    "e2m1_block16_f16_8192x4096": Workload(
        "e2m1_block16_f16_8192x4096", (8192, 4096), ElemType.F16,
        _block(QuantValue.E2M1, 16, QuantStore.Native), "row_scale*normal(0,1), row_scale~LogUniform(0.1,10)", 2),
    "e2m1_block32_f16_8192x4096": Workload(
        "e2m1_block32_f16_8192x4096", (8192, 4096), ElemType.F16,
        _block(QuantValue.E2M1, 32, QuantStore.Native), "row_scale*normal(0,1), row_scale~LogUniform(0.1,10)", 2),
    "q2_block64_f32_65536x4096": Workload(
        "q2_block64_f32_65536x4096", (65536, 4096), ElemType.F32, _block(QuantValue.Q2S, 64), "uniform(-1,1)", 3),
    "q8_block128_bf16_14336x4096": Workload(
        "q8_block128_bf16_14336x4096", (14336, 4096), ElemType.BF16, _block(QuantValue.Q8S, 128),
        "normal(0,0.02)", 4),
    "q8_tensor_bf16_14336x4096": Workload(
        "q8_tensor_bf16_14336x4096", (14336, 4096), ElemType.BF16,
        QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32, param=QuantParam.F32), "normal(0,0.02)", 4),
}

# The tensors of one Llama-3-8B-shaped layer and the embedding (rows, cols).
LLAMA3_8B_LAYER = (("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
                   ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336))
LLAMA3_8B_EMBEDDING = ("embedding", 128256, 4096)
LLAMA3_8B_LAYERS = 32


def generate(workload: Workload, device, rows: int | None = None, seed_offset: int = 0) -> torch.Tensor:
    """One tensor of the workload (optionally only ``rows`` rows of it), on ``device``."""
    r, c = workload.shape
    if rows is not None:
        r = rows
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(SEED_BASE + workload.index + 1000003 * seed_offset)
    dt = TORCH_DTYPE[workload.elem]
    d = workload.distribution
    if d == "normal(0,1)":
        x = torch.randn((r, c), generator=g, device=dev, dtype=torch.float32)
    elif d == "normal(0,0.02)":
        x = torch.randn((r, c), generator=g, device=dev, dtype=torch.float32) * 0.02
    elif d.startswith("normal(0,0.02) with"):
        x = torch.randn((r, c), generator=g, device=dev, dtype=torch.float32) * 0.02
        mask = torch.rand((r, c), generator=g, device=dev) < 0.001
        x = torch.where(mask, x * 20.0, x)
    elif d.startswith("row_scale"):
        z = torch.randn((r, c), generator=g, device=dev, dtype=torch.float32)
        u = torch.rand((r, 1), generator=g, device=dev, dtype=torch.float32)
        x = z * torch.exp(math.log(0.1) + u * (math.log(10.0) - math.log(0.1)))
    elif d == "uniform(-1,1)":
        x = torch.rand((r, c), generator=g, device=dev, dtype=torch.float32) * 2.0 - 1.0
    else:
        raise ValueError(d)
    return x.to(dt)
