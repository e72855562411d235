"""The quantized-input contract of the reference's matmul, so that tensors quantized here can be
handed to it unchanged: ``MatmulInputHandleRef::quantized(data, scale, shape, scheme, data_dtype,
scale_dtype)`` (crates/cubek-matmul/src/base.rs:436-452) and the layout it derives from the handle
(``from_quantized_handle``, crates/cubek-matmul/src/components/global/memory/layout.rs:213-262):

* ``shape`` is the logical (unpacked) shape; ``data`` holds ``num_quants`` values per stored item along
  the contiguous matrix dim: ``(row, col / packing)`` for a row-major operand, ``(row / packing, col)`` for a
  column-major one (layout.rs:131-134) - the transposed view of a tensor quantized along its rows;
* ``into_contiguous`` rewrites a column-major operand as a row-major one packed along the columns
  (``into_contiguous_packed``, base.rs:489-541);
* per-block scales use ``block_size.as_dim::<2>()`` = ``[block_row, block_col]`` over the last two dims,
  and the scales tensor is addressed as ``[row / block_row, col / block_col]`` through its own strides;
* the consumer reads with line size 1 on quantized operands, and a block must cover at least one
  stored item: ``block_col % num_quants == 0``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

from . import _ffi
from .scheme import ElemType, QuantScheme, QuantStore, QuantValue
from .tensor import ComputeClient, TensorHandleRef


@dataclass(frozen=True)
class MatmulInputHandleRef:
    """``MatmulInputHandleRef::Quantized`` (base.rs:309-317)."""

    data: TensorHandleRef
    scale: TensorHandleRef
    shape: Tuple[int, ...]
    scheme: QuantScheme
    data_dtype: str
    scale_dtype: ElemType

    @staticmethod
    def quantized(data: TensorHandleRef, scale: TensorHandleRef, shape, scheme: QuantScheme,
                  scale_dtype: ElemType | None = None) -> "MatmulInputHandleRef":
        shape = tuple(int(s) for s in shape)
        h = MatmulInputHandleRef(data, scale, shape, scheme, _data_dtype(scheme),
                                 scale_dtype if scale_dtype is not None else ElemType(int(scheme.param)))
        h.validate()
        return h

    def block_dims(self) -> Tuple[int, int]:
        """``block_size.as_dim::<2>()``: [block_row, block_col], left-padded with 1."""
        if self.scheme.level.is_tensor:
            return (self.shape[-2], self.shape[-1])
        dims = self.scheme.level.block_size.as_dim(2) if len(self.scheme.level.block_size.as_slice()) <= 2 else None
        if dims is None:
            raise ValueError("matmul inputs take at most 2 block dims")
        return dims

    @property
    def col_major(self) -> bool:
        """The packing runs along the rows: ``data`` is [.., rows / num_quants, cols] with stride 1 on the row dim."""
        return len(self.data.shape) >= 2 and self.data.strides[-1] != 1 and self.data.strides[-2] == 1

    def validate(self) -> None:
        if len(self.shape) < 2:
            raise ValueError("a matmul operand has at least 2 dims")
        nq = self.scheme.num_quants()
        rows, cols = self.shape[-2], self.shape[-1]
        if self.col_major:
            if rows % nq:
                raise ValueError("the contiguous dim (rows) must be a multiple of num_quants")
            if tuple(self.data.shape) != tuple(self.shape[:-2]) + (rows // nq, cols):
                raise ValueError(f"data shape {self.data.shape} is not the column-major packed form of {self.shape}")
        else:
            if cols % nq:
                raise ValueError("the contiguous dim must be a multiple of num_quants")
            if tuple(self.data.shape) != tuple(self.shape[:-1]) + (cols // nq,):
                raise ValueError(f"data shape {self.data.shape} is not the packed form of {self.shape}")
            if self.data.strides[-1] != 1:
                raise ValueError("packing runs along the contiguous matrix dim")
        if not self.scheme.level.is_tensor:
            br, bc = self.block_dims()
            if (br if self.col_major else bc) % nq:
                raise ValueError("the block extent along the packed dim must be a multiple of num_quants")   # lib.rs:20-33
            want = tuple(self.shape[:-2]) + (-(-rows // br), -(-cols // bc))
            if tuple(self.scale.shape) != want:
                raise ValueError(f"scales shape {self.scale.shape}, expected {want}")
        elif int(_numel(self.scale.shape)) != 1:
            raise ValueError("per-tensor scales hold one element")

    def into_contiguous(self, client: ComputeClient, out: TensorHandleRef) -> "MatmulInputHandleRef":
        """``MatmulInputHandleRef::into_contiguous`` for quantized operands (base.rs:489-541): the values are
        re-packed into ``out`` (caller-allocated, contiguous, ``shape`` with the last dim divided by the packing)
        so that the packing runs along the columns; scales are kept as they are.  Native one-value-per-byte
        stores have packing 1: a plain gather."""
        packing = self.scheme.num_quants()
        ti, to = _ffi.c_tensors(self.data, out)
        import ctypes as C

        shape = (C.c_int64 * len(self.shape))(*self.shape)
        _ffi.check(_ffi.lib().qk_into_contiguous_packed(ti.ref(), to.ref(), shape, len(self.shape), packing, client.stream))
        return MatmulInputHandleRef(out, self.scale, self.shape, self.scheme, self.data_dtype, self.scale_dtype)


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def _data_dtype(scheme: QuantScheme) -> str:
    if scheme.store == QuantStore.U32:
        return "u32"
    return {QuantValue.Q8F: "i8", QuantValue.Q8S: "i8", QuantValue.E2M1: "e2m1x2", QuantValue.E4M3: "e4m3",
            QuantValue.E5M2: "e5m2"}[scheme.value]
