"""cubek-quant for B200: the quantize / dequantize path of ``cubek::quantization``
(crates/cubek/src/lib.rs:1-2) as hand-written sm_100a kernels behind a C ABI.

Modules mirror the reference crate: ``scheme``, ``quantize``, ``dequantize``, ``layout``.
"""
from . import dequantize, quantize, scheme  # noqa: F401
from ._ffi import LaunchError, QuantPanic  # noqa: F401
from .scheme import (BlockSize, ElemType, Flex32, QuantLevel, QuantMode, QuantParam, QuantScheme,  # noqa: F401
                     QuantStore, QuantValue)
from .tensor import ComputeClient, TensorHandleRef  # noqa: F401

__version__ = "0.2.0"
