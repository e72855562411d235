"""``cubek_reduce::reduce`` for the instructions the quantize path's callers use - ``MaxAbs`` (absmax before the
scale formula), ``Max`` and ``Min`` (ranges) - with the reference's strategy surface
(crates/cubek-reduce/src/lib.rs:93-131, strategy.rs:7-16, instructions/maxabs.rs, max.rs, min.rs)."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional

from . import _ffi
from .scheme import ElemType
from .tensor import ComputeClient, TensorHandleRef


class ReduceInst(enum.IntEnum):
    MaxAbs = 0
    Max = 1
    Min = 2


@dataclass(frozen=True)
class ReduceStrategy:
    """``ReduceStrategy { use_planes, shared }``: ``shared`` - all units of a cube (CTA) reduce one output item
    together; otherwise each plane (warp, if ``use_planes``) or each unit (thread) reduces an item by itself.  On
    this hardware planes always exist with one fixed size, so ``validate`` never fails."""

    use_planes: bool = True
    shared: bool = True

    @staticmethod
    def new(client: ComputeClient, shared: bool) -> "ReduceStrategy":
        return ReduceStrategy(use_planes=True, shared=shared)


def reduce(client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef, axis: int,
           strategy: Optional[ReduceStrategy], inst: ReduceInst, dtype: ElemType) -> None:
    """``output[.., 0, ..] = inst(input[.., :, ..])`` along ``axis``.  ``output`` has the input's shape with extent 1
    at ``axis`` (``valid_output_shape``, lib.rs:142-160) and the input's element type.  ``strategy=None`` is the
    reference's default (the library then picks the thread group by shape)."""
    ti, to = _ffi.c_tensors(input, output)
    st = None
    if strategy is not None:
        st = C.byref(_ffi.QkReduceStrategy(int(strategy.use_planes), int(strategy.shared)))
    _ffi.check(_ffi.lib().qk_reduce(ti.ref(), to.ref(), int(axis), int(inst), st, int(dtype), client.stream))


def reduce_maxabs(client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef, axis: int,
                  dtype: ElemType) -> None:
    """``reduce`` with ``MaxAbs`` and the default strategy."""
    reduce(client, input, output, axis, None, ReduceInst.MaxAbs, dtype)
