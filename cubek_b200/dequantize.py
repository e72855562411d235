"""``cubek_quant::dequantize`` for B200: mirrors ``launch_ref``
(crates/cubek-quant/src/dequantize.rs:171-229)."""
from __future__ import annotations

from . import _ffi
from .scheme import ElemType, QuantScheme
from .tensor import ComputeClient, TensorHandleRef


def launch_ref(client: ComputeClient, values: TensorHandleRef, output: TensorHandleRef,
               params: TensorHandleRef, scheme: QuantScheme, input_dtype: ElemType) -> None:
    """Convert the quantized ``values`` back to the float type ``input_dtype`` (the reference's
    name for the type of ``output``): ``output = cast(params) * q``."""
    tv, to, tp = _ffi.c_tensors(values, output, params)
    _ffi.check(_ffi.lib().qk_dequantize(tv.ref(), to.ref(), tp.ref(), _ffi.c_scheme(scheme),
                                        int(input_dtype), client.stream))


class Prepared:
    """``launch_ref`` with the argument marshalling done once (see ``quantize.PreparedDynamic``)."""

    def __init__(self, client: ComputeClient, values: TensorHandleRef, output: TensorHandleRef,
                 params: TensorHandleRef, scheme: QuantScheme, input_dtype: ElemType):
        self._keep = _ffi.c_tensors(values, output, params)
        self._scheme = _ffi.c_scheme(scheme)
        self._args = (self._keep[0].ref(), self._keep[1].ref(), self._keep[2].ref(), self._scheme, int(input_dtype),
                      client.stream)
        self._fn = _ffi.lib().qk_dequantize

    def __call__(self) -> None:
        status = self._fn(*self._args)
        if status:
            _ffi.check(status)


class PreparedBatch:
    """Dequantize of a set of tensors, one launch per group of up to 64 compatible tensors
    (``qk_dequantize_batch``); same results as ``launch_ref`` per tensor."""

    def __init__(self, client: ComputeClient, values, outputs, params, scheme: QuantScheme, input_dtype: ElemType):
        self._v, self._o, self._p = _ffi.CTensorArray(values), _ffi.CTensorArray(outputs), _ffi.CTensorArray(params)
        if not (self._v.count == self._o.count == self._p.count):
            raise ValueError("values, outputs and params must have the same length")
        self._scheme = _ffi.c_scheme(scheme)
        self._args = (self._v.count, self._v.array, self._o.array, self._p.array, self._scheme, int(input_dtype),
                      client.stream)
        self._fn = _ffi.lib().qk_dequantize_batch

    def __call__(self) -> None:
        status = self._fn(*self._args)
        if status:
            _ffi.check(status)


def launch_batch(client: ComputeClient, values, outputs, params, scheme: QuantScheme, input_dtype: ElemType) -> None:
    PreparedBatch(client, values, outputs, params, scheme, input_dtype)()
