"""NumPy front end of the C oracle (``cubek_quant_oracle.c``).

Test infrastructure only.  Arrays are NumPy arrays of dtype float32, float16 or
``ml_dtypes.bfloat16``; shapes follow the reference: the quantized tensor has the last dim
divided by ``num_quants`` and the scales tensor has one entry per block (or one in total).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path
from typing import Tuple

import ml_dtypes
import numpy as np

from cubek_b200.scheme import ElemType, QuantParam, QuantScheme, QuantStore, QuantValue

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"
LIB_PATH_HALF_AWAY = HERE / "liboracle_half_away.so"

bfloat16 = ml_dtypes.bfloat16

_NP_OF = {ElemType.F32: np.dtype(np.float32), ElemType.F16: np.dtype(np.float16),
          ElemType.BF16: np.dtype(bfloat16)}


def np_dtype(dt) -> np.dtype:
    return _NP_OF[ElemType(int(dt))]


def elem_type(dtype) -> ElemType:
    dtype = np.dtype(dtype)
    for k, v in _NP_OF.items():
        if v == dtype:
            return k
    raise TypeError(f"unsupported float dtype {dtype}")


def build(force: bool = False) -> Path:
    src = HERE / "cubek_quant_oracle.c"
    for path in (LIB_PATH, LIB_PATH_HALF_AWAY):
        if force or not path.exists() or path.stat().st_mtime < src.stat().st_mtime:
            subprocess.run(["make", "-C", str(HERE), "-B", path.name], check=True, capture_output=True)
    return LIB_PATH


_libs = {}


def lib(rounding: str = "even") -> C.CDLL:
    """The oracle library: ``rounding="even"`` (the default restatement) or ``"away"`` (halves away from zero)."""
    if rounding not in ("even", "away"):
        raise ValueError(rounding)
    if rounding not in _libs:
        path = LIB_PATH if rounding == "even" else LIB_PATH_HALF_AWAY
        if not path.exists():
            build()
        h = C.CDLL(str(path))
        i64p, u8p = C.POINTER(C.c_int64), C.POINTER(C.c_uint8)
        h.oq_compute_scales.restype = C.c_int
        h.oq_compute_scales.argtypes = [C.c_void_p, C.c_int, i64p, C.c_int, C.c_int, C.c_int, u8p, C.c_int,
                                        C.c_void_p, i64p]
        h.oq_quantize.restype = C.c_int
        h.oq_quantize.argtypes = [C.c_void_p, C.c_int, i64p, C.c_int, C.c_void_p, i64p, C.c_int, C.c_int, C.c_int,
                                  C.c_int, u8p, C.c_int, C.c_void_p, C.c_void_p]
        h.oq_dequantize.restype = C.c_int
        h.oq_dequantize.argtypes = [C.c_void_p, i64p, C.c_int, C.c_void_p, i64p, C.c_int, C.c_int, C.c_int, C.c_int,
                                    u8p, C.c_int, C.c_int, C.c_void_p]
        h.oq_max_threads.restype = C.c_int
        h.oq_set_threads.argtypes = [C.c_int]
        for name in ("oq_f32_to_e2m1", "oq_f32_to_e4m3", "oq_f32_to_e5m2"):
            getattr(h, name).restype = C.c_uint8
            getattr(h, name).argtypes = [C.c_float]
        for name in ("oq_e2m1_to_f32", "oq_e4m3_to_f32", "oq_e5m2_to_f32"):
            getattr(h, name).restype = C.c_float
            getattr(h, name).argtypes = [C.c_uint8]
        _libs[rounding] = h
    return _libs[rounding]


class OracleError(AssertionError):
    def __init__(self, status: int):
        super().__init__(f"oracle status {status}")
        self.status = status


def _check(rc: int) -> None:
    if rc != 0:
        raise OracleError(rc)


def _i64(seq):
    return (C.c_int64 * max(len(seq), 1))(*[int(v) for v in seq])


def _block(scheme: QuantScheme):
    if scheme.level.is_tensor:
        return (C.c_uint8 * 8)(), 0, 0
    dims = scheme.level.block_size.as_slice()
    return (C.c_uint8 * 8)(*dims), len(dims), 1


def _elem_strides(a: np.ndarray):
    return [s // a.itemsize for s in a.strides]


def code_dtype(scheme: QuantScheme) -> np.dtype:
    if scheme.store == QuantStore.U32:
        return np.dtype(np.uint32)
    return np.dtype(np.int8) if scheme.value in (QuantValue.Q8F, QuantValue.Q8S) else np.dtype(np.uint8)


def _buffer(out, shape, dtype) -> np.ndarray:
    """A caller-provided output buffer (checked) or a fresh zeroed one."""
    if out is None:
        return np.zeros(shape, dtype=dtype)
    assert out.shape == tuple(shape) and out.dtype == np.dtype(dtype) and out.flags.c_contiguous, "bad output buffer"
    return out


def compute_scales(x: np.ndarray, scheme: QuantScheme, out: np.ndarray | None = None) -> np.ndarray:
    """absmax per tensor / block and ``scale = 2*absmax/(hi-lo)``, typed like ``x``."""
    x = np.ascontiguousarray(x)
    fdt = elem_type(x.dtype)
    out = _buffer(out, tuple(scheme.scales_shape(x.shape)), x.dtype)
    blk, brank, level = _block(scheme)
    strides = _elem_strides(out) if level else [0] * x.ndim
    _check(lib().oq_compute_scales(x.ctypes.data, int(fdt), _i64(x.shape), x.ndim, int(scheme.value), level,
                                   blk, brank, out.ctypes.data, _i64(strides)))
    return out


def quantize(x: np.ndarray, scale: np.ndarray, scheme: QuantScheme, out: np.ndarray | None = None,
             out_scale: np.ndarray | None = None, rounding: str = "even") -> Tuple[np.ndarray, np.ndarray]:
    """``quantize::launch_ref``: returns (quantized tensor, out_scale typed as the param)."""
    x = np.ascontiguousarray(x)
    fdt = elem_type(x.dtype)
    assert scale.dtype == x.dtype, "scale is typed like the input"
    blk, brank, level = _block(scheme)
    nq = scheme.num_quants()
    if x.shape[-1] % nq:
        raise OracleError(3)
    out = _buffer(out, tuple(scheme.packed_shape(x.shape)), code_dtype(scheme))
    out_scale = _buffer(out_scale, tuple(scale.shape), np_dtype(int(scheme.param)))
    strides = _elem_strides(scale) if level else [0] * x.ndim
    _check(lib(rounding).oq_quantize(x.ctypes.data, int(fdt), _i64(x.shape), x.ndim, scale.ctypes.data, _i64(strides),
                             int(scheme.value), int(scheme.store), int(scheme.param), level, blk, brank,
                             out.ctypes.data, out_scale.ctypes.data))
    return out, out_scale


def dequantize(values: np.ndarray, params: np.ndarray, scheme: QuantScheme, out_dtype,
               out: np.ndarray | None = None) -> np.ndarray:
    """``dequantize::launch_ref``: returns the float tensor of the unpacked shape."""
    values = np.ascontiguousarray(values)
    odt = elem_type(out_dtype)
    nq = scheme.num_quants()
    shape = tuple(values.shape[:-1]) + (values.shape[-1] * nq,)
    out = _buffer(out, shape, np_dtype(odt))
    blk, brank, level = _block(scheme)
    strides = _elem_strides(params) if level else [0] * len(shape)
    _check(lib().oq_dequantize(values.ctypes.data, _i64(shape), len(shape), params.ctypes.data, _i64(strides),
                               int(scheme.value), int(scheme.store), int(scheme.param), level, blk, brank,
                               int(odt), out.ctypes.data))
    return out


def quantize_dynamic(x: np.ndarray, scheme: QuantScheme, rounding: str = "even"):
    """compute_scales followed by quantize."""
    return quantize(x, compute_scales(x, scheme), scheme, rounding=rounding)


def max_threads() -> int:
    return lib().oq_max_threads()


def set_threads(n: int) -> None:
    lib().oq_set_threads(int(n))
