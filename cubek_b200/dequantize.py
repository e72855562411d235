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
