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
