"""``cubek_reduce::reduce`` restricted to the ``MaxAbs`` instruction, the reduction callers of the
quantize path use for absmax (crates/cubek-reduce/src/lib.rs:93-131,
crates/cubek-reduce/src/instructions/maxabs.rs:31-87)."""
from __future__ import annotations

from . import _ffi
from .scheme import ElemType
from .tensor import ComputeClient, TensorHandleRef


def reduce_maxabs(client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef, axis: int,
                  dtype: ElemType) -> None:
    """``output[.., 0, ..] = max |input[.., :, ..]|`` along ``axis``.  ``output`` has the input's shape
    with extent 1 at ``axis`` (``valid_output_shape``, lib.rs:142-150) and the input's element type."""
    ti, to = _ffi.c_tensors(input, output)
    _ffi.check(_ffi.lib().qk_reduce_maxabs(ti.ref(), to.ref(), int(axis), int(dtype), client.stream))
