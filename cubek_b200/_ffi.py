"""ctypes binding of libcubek_quant_b200.so (the C ABI declared in include/cubek_quant_b200.h).

There is no CPU fallback: if the library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Sequence

from .scheme import QuantScheme
from .tensor import TensorHandleRef

LIB_PATH = Path(__file__).resolve().parent / "libcubek_quant_b200.so"
# the build that rounds halves away from zero (`python -m cubek_b200.build --round-half-away`)
LIB_PATH_HALF_AWAY = Path(__file__).resolve().parent / "libcubek_quant_b200_half_away.so"

QK_OK = 0
QK_ERR_UNSUPPORTED_SCHEME = 1
QK_ERR_BLOCK_SIZE = 2
QK_ERR_SHAPE = 3
QK_ERR_DTYPE = 4
QK_ERR_LAYOUT = 5
QK_ERR_ALIGN = 6
QK_ERR_NULL = 7
QK_ERR_WORKSPACE = 8
QK_ERR_TOO_LARGE = 9
QK_ERR_NCCL = 10
QK_ERR_TIMEOUT = 11
QK_ERR_DEVICE = 12
QK_ERR_CUDA = 1000

# Status codes that stand for a `panic!` / `assert!` in the reference.
PANIC_CLASS = (QK_ERR_UNSUPPORTED_SCHEME, QK_ERR_BLOCK_SIZE, QK_ERR_SHAPE, QK_ERR_DTYPE)

(TUNE_THREADS, TUNE_CTAS_PER_SM, TUNE_FORCE_EXACT, TUNE_FORCE_GENERAL, TUNE_PDL, TUNE_QUANT_WAVES, TUNE_DEQUANT_WAVES,
 TUNE_COOP_TENSOR, TUNE_STAGED, TUNE_SLICE_KIB, TUNE_SLOTS, TUNE_STAGES) = range(12)


class QkScheme(C.Structure):
    _fields_ = [("value", C.c_int32), ("param", C.c_int32), ("store", C.c_int32),
                ("level", C.c_int32), ("mode", C.c_int32), ("block_rank", C.c_int32),
                ("block", C.c_uint8 * 8)]


class QkTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("rank", C.c_int32), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("elem_size", C.c_int32)]


class QkReduceStrategy(C.Structure):
    _fields_ = [("use_planes", C.c_int32), ("shared", C.c_int32)]


class LaunchError(RuntimeError):
    """A launch failed (the reference's ``Err(LaunchError)``)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}] {message}")
        self.status = status


class QuantPanic(AssertionError):
    """The reference would ``panic!`` / ``assert!`` on these arguments."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}] {message}")
        self.status = status


_lib = None

_SIGNATURES = {
    "qk_num_quants": (C.c_int, [C.POINTER(QkScheme)]),
    "qk_value_range": (C.c_int, [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "qk_quantize": (C.c_int, [C.POINTER(QkTensor)] * 4 + [C.POINTER(QkScheme), C.c_int, C.c_void_p]),
    "qk_dequantize": (C.c_int, [C.POINTER(QkTensor)] * 3 + [C.POINTER(QkScheme), C.c_int, C.c_void_p]),
    "qk_compute_scales": (C.c_int, [C.POINTER(QkTensor)] * 2 + [C.POINTER(QkScheme), C.c_int, C.c_void_p,
                                                               C.c_size_t, C.c_void_p]),
    "qk_quantize_dynamic": (C.c_int, [C.POINTER(QkTensor)] * 3 + [C.POINTER(QkScheme), C.c_int, C.c_void_p,
                                                                 C.c_size_t, C.c_void_p]),
    "qk_reduce_maxabs": (C.c_int, [C.POINTER(QkTensor)] * 2 + [C.c_int, C.c_int, C.c_void_p]),
    "qk_reduce": (C.c_int, [C.POINTER(QkTensor)] * 2 + [C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "qk_quantize_dynamic_batch": (C.c_int, [C.c_int] + [C.POINTER(QkTensor)] * 3 + [C.POINTER(QkScheme), C.c_int, C.c_void_p,
                                                    C.c_size_t, C.c_void_p]),
    "qk_dequantize_batch": (C.c_int, [C.c_int] + [C.POINTER(QkTensor)] * 3 + [C.POINTER(QkScheme), C.c_int, C.c_void_p]),
    "qk_quantize_dynamic_noalloc": (C.c_int, [C.POINTER(QkTensor)] * 3 + [C.POINTER(QkScheme), C.c_int, C.c_void_p]),
    "qk_noalloc_scratch_bytes": (C.c_size_t, []),
    "qk_absmax_f32": (C.c_int, [C.POINTER(QkTensor), C.c_int, C.c_void_p, C.c_void_p]),
    "qk_quantize_from_absmax": (C.c_int, [C.POINTER(QkTensor)] * 3 + [C.c_void_p, C.POINTER(QkScheme), C.c_int,
                                                                     C.c_void_p]),
    "qk_absmax_batch": (C.c_int, [C.c_int, C.POINTER(QkTensor), C.c_int, C.c_void_p, C.c_void_p]),
    "qk_quantize_from_absmax_batch": (C.c_int, [C.c_int] + [C.POINTER(QkTensor)] * 3 + [C.c_void_p, C.POINTER(QkScheme), C.c_int,
                                                        C.c_void_p]),
    "qk_allreduce_max_f32": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "qk_allreduce_max_f32_deadline": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int]),
    "qk_workspace_bytes": (C.c_size_t, []),
    "qk_workspace_bytes_for": (C.c_size_t, [C.POINTER(QkTensor), C.POINTER(QkScheme), C.c_int]),
    "qk_roundtrip_host": (C.c_int, [C.POINTER(QkTensor)] * 4 + [C.POINTER(QkScheme), C.c_int, C.c_void_p,
                                                               C.c_size_t, C.c_int]),
    "qk_host_roundtrip_staging_bytes": (C.c_size_t, [C.POINTER(QkTensor), C.POINTER(QkScheme), C.c_int]),
    "qk_roundtrip_host_batch": (C.c_int, [C.c_int] + [C.POINTER(QkTensor)] * 4 + [C.POINTER(QkScheme), C.c_int, C.c_void_p,
                                                      C.c_size_t, C.c_int]),
    "qk_host_roundtrip_staging_bytes_batch": (C.c_size_t, [C.c_int, C.POINTER(QkTensor), C.POINTER(QkScheme), C.c_int]),
    "qk_into_contiguous_packed": (C.c_int, [C.POINTER(QkTensor)] * 2 + [C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_void_p]),
    "qk_strerror": (C.c_char_p, [C.c_int]),
    "qk_version": (C.c_char_p, []),
    "qk_launch_count": (C.c_uint64, []),
    "qk_device_error": (C.c_int, [C.POINTER(C.c_int)]),
}

# include/cubek_quant_b200_testing.h: hooks for tests and measurements, not part of the drop-in interface
ALLREDUCE_HOOK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p, C.c_void_p)
ASYNC_ERROR_HOOK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_int))
STREAM_QUERY_HOOK = C.CFUNCTYPE(C.c_int, C.c_void_p)
_TESTING_SIGNATURES = {
    "qk_set_tuning": (None, [C.c_int, C.c_int]),
    "qk_get_tuning": (C.c_int, [C.c_int]),
    "qk_testing_set_collective_hooks": (None, [C.c_void_p, C.c_void_p, C.c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)
TESTING_SYMBOLS = tuple(_TESTING_SIGNATURES)


def load(path: Path) -> C.CDLL:
    """Load one build of the library and bind every entry point.  Raises ``OSError`` with a build hint when the
    file is missing (there is no CPU fallback)."""
    if not Path(path).exists():
        raise OSError(f"{path} not found: build it with `python -m cubek_b200.build` (there is no CPU fallback)")
    handle = C.CDLL(str(path))
    for name, (res, args) in {**_SIGNATURES, **_TESTING_SIGNATURES}.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    return handle


def lib() -> C.CDLL:
    """The library (round-half-to-even build), loaded once."""
    global _lib
    if _lib is None:
        _lib = load(LIB_PATH)
    return _lib


def strerror(status: int) -> str:
    return lib().qk_strerror(status).decode()


def check(status: int) -> None:
    if status == QK_OK:
        return
    msg = strerror(status)
    if status in PANIC_CLASS:
        raise QuantPanic(status, msg)
    raise LaunchError(status, msg)


def c_scheme(scheme: QuantScheme) -> QkScheme:
    s = QkScheme()
    s.value, s.param, s.store, s.mode = int(scheme.value), int(scheme.param), int(scheme.store), int(scheme.mode)
    if scheme.level.is_tensor:
        s.level, s.block_rank = 0, 0
    else:
        dims = scheme.level.block_size.as_slice()
        s.level, s.block_rank = 1, len(dims)
        for i, d in enumerate(dims):
            s.block[i] = d
    return s


class CTensor:
    """Keeps the shape/stride arrays alive next to the QkTensor that points at them."""

    def __init__(self, t: TensorHandleRef):
        rank = len(t.shape)
        self._shape = (C.c_int64 * max(rank, 1))(*t.shape)
        self._strides = (C.c_int64 * max(rank, 1))(*t.strides)
        self.c = QkTensor(C.c_void_p(t.handle), rank, self._shape, self._strides, t.elem_size)

    def ref(self):
        return C.byref(self.c)


def c_tensors(*tensors: TensorHandleRef) -> Sequence[CTensor]:
    return [CTensor(t) for t in tensors]


class CTensorArray:
    """A contiguous C array of QkTensor (for the batch entry points), keeping its parts alive."""

    def __init__(self, tensors: Sequence[TensorHandleRef]):
        self._items = [CTensor(t) for t in tensors]
        self.array = (QkTensor * max(len(self._items), 1))(*[t.c for t in self._items])
        self.count = len(self._items)
