"""An independent, slow restatement of the same semantics in NumPy + ml_dtypes, used only to
cross-check the C oracle on small cases.  Test infrastructure.

It shares no code with the C file: narrowing to f16 / bf16 goes through ``astype`` of NumPy /
ml_dtypes, rounding through ``np.rint`` (half to even), the fp4 cast through
``ml_dtypes.float4_e2m1fn`` and the fp8 casts through ``ml_dtypes.float8_e4m3fn`` /
``float8_e5m2``.

Semantics restated: crates/cubek-quant/src/quantize.rs:19-98 and :128-171,
crates/cubek-quant/src/dequantize.rs:22-25 and :86-118, layout/scales.rs:144-160,
scale formula crates/cubek-quant/tests/suite/symmetric.rs:35-38 and :175-178.
"""
from __future__ import annotations

import itertools

import ml_dtypes
import numpy as np

from cubek_b200.scheme import QuantParam, QuantScheme, QuantStore, QuantValue

_PARAM_NP = {QuantParam.F32: np.float32, QuantParam.F16: np.float16, QuantParam.BF16: ml_dtypes.bfloat16}


def _block_vec(scheme: QuantScheme, rank: int):
    return None if scheme.level.is_tensor else scheme.level.block_size.to_dim_vec(rank)


def _scale_index(idx, blk):
    return tuple(i // b for i, b in zip(idx, blk))


def compute_scales(x: np.ndarray, scheme: QuantScheme) -> np.ndarray:
    lo, hi = scheme.value.range()
    blk = _block_vec(scheme, x.ndim)
    out = np.zeros(scheme.scales_shape(x.shape), dtype=x.dtype)
    xf = np.abs(x.astype(np.float32))
    if blk is None:
        amax = np.float32(xf.max()) if xf.size else np.float32(0)
        out[0] = (np.float32(2) * amax / np.float32(hi - lo)).astype(x.dtype)
        return out
    for sidx in itertools.product(*[range(s) for s in out.shape]):
        sl = tuple(slice(i * b, (i + 1) * b) for i, b in zip(sidx, blk))
        amax = np.float32(xf[sl].max())
        out[sidx] = (np.float32(2) * amax / np.float32(hi - lo)).astype(x.dtype)
    return out


def _round(t, rounding):
    if rounding == "even":
        return np.rint(t)
    # halves away from zero; the sum is formed in f64, where it is exact for every f32 `t`
    return np.float32(np.copysign(np.floor(np.abs(np.float64(t)) + 0.5), t)) if np.isfinite(t) else t


def _quantize_values(x: np.ndarray, scale: np.ndarray, scheme: QuantScheme, rounding: str = "even"):
    """Integral clamped values (float32) and out_scale."""
    F = x.dtype
    lo, hi = scheme.value.range()
    blk = _block_vec(scheme, x.ndim)
    s_fs = scale.astype(_PARAM_NP[scheme.param])
    s_f = s_fs.astype(F).astype(np.float32)
    c = np.zeros(x.shape, dtype=np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        for idx in itertools.product(*[range(s) for s in x.shape]):
            s = s_f[0] if blk is None else s_f[_scale_index(idx, blk)]
            t = (np.float32(x[idx]) / np.float32(s)).astype(F).astype(np.float32)
            r = _round(t, rounding)
            c[idx] = 0.0 if np.isnan(r) else min(max(r, np.float32(lo)), np.float32(hi))
    return c, s_fs


def quantize(x: np.ndarray, scale: np.ndarray, scheme: QuantScheme, rounding: str = "even"):
    c, s_fs = _quantize_values(x, scale, scheme, rounding)
    nq = scheme.num_quants()
    flat = c.reshape(-1, nq)
    if scheme.store == QuantStore.U32:
        bits = scheme.value.size_bits()
        mask = (1 << bits) - 1
        words = np.zeros(flat.shape[0], dtype=np.uint64)
        for i in range(nq):
            words |= (flat[:, i].astype(np.int64) & mask).astype(np.uint64) << np.uint64(i * bits)
        out = words.astype(np.uint32).reshape(scheme.packed_shape(x.shape))
    elif scheme.value == QuantValue.E2M1:
        codes = flat.astype(ml_dtypes.float4_e2m1fn).view(np.uint8) & 0xF
        out = (codes[:, 0] | (codes[:, 1] << 4)).astype(np.uint8).reshape(scheme.packed_shape(x.shape))
    elif scheme.value == QuantValue.E4M3:
        out = flat.astype(ml_dtypes.float8_e4m3fn).view(np.uint8).reshape(x.shape)
    elif scheme.value == QuantValue.E5M2:
        out = flat.astype(ml_dtypes.float8_e5m2).view(np.uint8).reshape(x.shape)
    else:
        out = flat.astype(np.int8).reshape(x.shape)
    return out, s_fs


def dequantize(values: np.ndarray, params: np.ndarray, scheme: QuantScheme, out_dtype) -> np.ndarray:
    F = np.dtype(out_dtype)
    nq = scheme.num_quants()
    shape = tuple(values.shape[:-1]) + (values.shape[-1] * nq,)
    flat = values.reshape(-1)
    if scheme.store == QuantStore.U32:
        bits = scheme.value.size_bits()
        mask = (1 << bits) - 1
        q = np.zeros((flat.size, nq), dtype=np.int64)
        for i in range(nq):
            raw = (flat.astype(np.int64) >> (i * bits)) & mask
            q[:, i] = raw - np.where(raw >= (1 << (bits - 1)), 1 << bits, 0)
        qf = q.astype(np.float32)
    elif scheme.value == QuantValue.E2M1:
        lo4 = (flat & 0xF).astype(np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float32)
        hi4 = (flat >> 4).astype(np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float32)
        qf = np.stack([lo4, hi4], axis=1)
    elif scheme.value == QuantValue.E4M3:
        qf = flat.view(ml_dtypes.float8_e4m3fn).astype(np.float32).reshape(-1, 1)
    elif scheme.value == QuantValue.E5M2:
        qf = flat.view(ml_dtypes.float8_e5m2).astype(np.float32).reshape(-1, 1)
    else:
        qf = flat.astype(np.float32).reshape(-1, 1)
    qf = qf.reshape(shape)
    blk = _block_vec(scheme, len(shape))
    s_f = params.astype(F).astype(np.float32)
    out = np.zeros(shape, dtype=F)
    for idx in itertools.product(*[range(s) for s in shape]):
        s = s_f[0] if blk is None else s_f[_scale_index(idx, blk)]
        out[idx] = (np.float32(s) * qf[idx].astype(F).astype(np.float32)).astype(F)
    return out
