"""Seeded small inputs used by the parity tests (CPU cross-checks and GPU parity alike)."""
from __future__ import annotations

import itertools

import ml_dtypes
import numpy as np

from cubek_b200 import QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue

bfloat16 = ml_dtypes.bfloat16
FLOATS = {"f32": np.dtype(np.float32), "f16": np.dtype(np.float16), "bf16": np.dtype(bfloat16)}

PACKED_VALUES = [QuantValue.Q8F, QuantValue.Q8S, QuantValue.Q4F, QuantValue.Q4S, QuantValue.Q2F, QuantValue.Q2S,
                 QuantValue.E2M1]
NATIVE_VALUES = [QuantValue.Q8F, QuantValue.Q8S, QuantValue.E2M1, QuantValue.E4M3, QuantValue.E5M2]


def all_value_stores():
    for v in PACKED_VALUES:
        yield v, QuantStore.U32
    for v in NATIVE_VALUES:
        yield v, QuantStore.Native


def random_tensor(shape, dtype, seed, kind="normal"):
    rng = np.random.default_rng(seed)
    if kind == "normal":
        x = rng.standard_normal(shape).astype(np.float32)
    elif kind == "outliers":
        x = (rng.standard_normal(shape) * 0.02).astype(np.float32)
        x = np.where(rng.random(shape) < 0.001, x * 20, x).astype(np.float32)
    elif kind == "uniform":
        x = rng.uniform(-1, 1, shape).astype(np.float32)
    elif kind == "rowscaled":
        x = rng.standard_normal(shape).astype(np.float32)
        x = x * np.exp(rng.uniform(np.log(0.1), np.log(10), (shape[0], 1))).astype(np.float32)
    else:
        raise ValueError(kind)
    return x.astype(dtype)


def adversarial_tensor(shape, dtype, scheme: QuantScheme, seed):
    """Quotients on and next to every half-integer tie, +-absmax, zeros, tiny values, and whole
    blocks of zeros, laid over a random background."""
    rng = np.random.default_rng(seed)
    lo, hi = scheme.value.range()
    n = int(np.prod(shape))
    step = rng.uniform(0.01, 3.0)
    fmax = float(ml_dtypes.finfo(dtype).max) if np.dtype(dtype) == np.dtype(bfloat16) else float(np.finfo(dtype).max)
    step = min(step, fmax / (float(hi) + 2.0) / 4.0)        # keep every value finite in `dtype`
    k = rng.integers(int(lo) - 1, int(hi) + 2, n).astype(np.float32)
    frac = rng.choice(np.array([0.0, 0.5, -0.5, 0.49999997, 0.50000006, 0.25, -0.25], dtype=np.float32), n)
    x = ((k + frac) * np.float32(step)).astype(np.float32)
    x[rng.random(n) < 0.05] = 0.0
    x[rng.random(n) < 0.02] = np.float32(1e-30)
    x = x.reshape(shape)
    if x.ndim == 2 and shape[0] >= 4:
        x[1, :] = 0.0                      # all-zero blocks: scale 0, codes 0
        x[2, : shape[1] // 2] = 0.0
    return x.astype(dtype)


def levels_for(shape, nq):
    """Per tensor plus a few last-dim block sizes that are multiples of num_quants."""
    out = [QuantLevel.Tensor]
    for b in (16, 32, 64, 128):
        if b % nq == 0 and shape[-1] % b == 0:
            out.append(QuantLevel.block([b]))
    return out


def scheme_grid(shape):
    for (value, store), param in itertools.product(all_value_stores(), [QuantParam.F32]):
        nq = QuantScheme(value=value, store=store).num_quants()
        for level in levels_for(shape, nq):
            yield QuantScheme(value=value, store=store, param=param, level=level)


def scheme_id(s: QuantScheme) -> str:
    lvl = "tensor" if s.level.is_tensor else "block" + "x".join(map(str, s.level.block_size.as_slice()))
    return f"{s.value.name}-{s.store.name}-{s.param.name}-{lvl}"
