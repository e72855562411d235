"""Quantization scheme: the host-side mirror of ``cubecl_common::quant::scheme``.

The reference re-exports that module as ``cubek_quant::scheme``
(crates/cubek-quant/src/lib.rs:14) and uses it through the builder
``QuantScheme::default().with_level(..).with_mode(..).with_value(..).with_store(..).with_param(..)``
(crates/cubek-quant/tests/suite/symmetric.rs:60-66).  The numeric constants follow the public
cubecl-common API; the source of that crate is not part of the reference checkout.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, replace
from typing import Sequence, Tuple


class ElemType(enum.IntEnum):
    """Float element types accepted as ``input_elem`` (quantize.rs:181).  ``Flex32`` is the
    reference tests' name for f32 data (symmetric.rs:106) and is the same type here."""

    F32 = 0
    F16 = 1
    BF16 = 2

    @property
    def size(self) -> int:
        return 4 if self == ElemType.F32 else 2


Flex32 = ElemType.F32


class QuantValue(enum.IntEnum):
    Q8F = 0
    Q8S = 1
    Q4F = 2
    Q4S = 3
    Q2F = 4
    Q2S = 5
    E4M3 = 6
    E5M2 = 7
    E2M1 = 8

    def range(self) -> Tuple[float, float]:
        """``QuantValue::range`` (quantize.rs:243, :296): "F" is the full two's-complement
        range, "S" the symmetric one."""
        return {
            QuantValue.Q8F: (-128.0, 127.0), QuantValue.Q8S: (-127.0, 127.0),
            QuantValue.Q4F: (-8.0, 7.0), QuantValue.Q4S: (-7.0, 7.0),
            QuantValue.Q2F: (-2.0, 1.0), QuantValue.Q2S: (-1.0, 1.0),
            QuantValue.E4M3: (-448.0, 448.0), QuantValue.E5M2: (-57344.0, 57344.0),
            QuantValue.E2M1: (-6.0, 6.0),
        }[self]

    def size_bits(self) -> int:
        if self in (QuantValue.Q8F, QuantValue.Q8S, QuantValue.E4M3, QuantValue.E5M2):
            return 8
        if self in (QuantValue.Q4F, QuantValue.Q4S, QuantValue.E2M1):
            return 4
        return 2


class QuantStore(enum.IntEnum):
    Native = 0
    U32 = 1


class QuantParam(enum.IntEnum):
    F32 = 0
    F16 = 1
    BF16 = 2

    @property
    def size(self) -> int:
        return 4 if self == QuantParam.F32 else 2


class QuantMode(enum.IntEnum):
    Symmetric = 0


@dataclass(frozen=True)
class BlockSize:
    """Block extents, each a ``u8`` as in the reference (``QuantLevel::block([b as u8])``,
    symmetric.rs:202)."""

    dims: Tuple[int, ...]

    def __post_init__(self):
        if not 1 <= len(self.dims) <= 8:
            raise ValueError("a block size has 1 to 8 dims")
        for d in self.dims:
            if not 0 <= int(d) <= 255:
                raise ValueError("block extents are u8")

    def as_slice(self) -> Tuple[int, ...]:
        return self.dims

    def to_dim_vec(self, rank: int) -> Tuple[int, ...]:
        """Right-align to ``rank`` dims, padding with 1 on the left (layout/scales.rs:239)."""
        if len(self.dims) > rank:
            raise ValueError("block has more dims than the tensor")
        return (1,) * (rank - len(self.dims)) + tuple(self.dims)

    def as_dim(self, n: int) -> Tuple[int, ...]:
        return self.to_dim_vec(n)


@dataclass(frozen=True)
class QuantLevel:
    block_size: BlockSize | None = None  # None = per tensor

    Tensor = None  # set below

    @staticmethod
    def block(dims: Sequence[int]) -> "QuantLevel":
        return QuantLevel(BlockSize(tuple(int(d) for d in dims)))

    @property
    def is_tensor(self) -> bool:
        return self.block_size is None


QuantLevel.Tensor = QuantLevel(None)


@dataclass(frozen=True)
class QuantScheme:
    """``QuantScheme { value, param, store, level, mode }``; the default matches the
    reference's ``QuantScheme::default()``."""

    value: QuantValue = QuantValue.Q8F
    param: QuantParam = QuantParam.F32
    store: QuantStore = QuantStore.U32
    level: QuantLevel = QuantLevel.Tensor
    mode: QuantMode = QuantMode.Symmetric

    def with_level(self, level: QuantLevel) -> "QuantScheme":
        return replace(self, level=level)

    def with_mode(self, mode: QuantMode) -> "QuantScheme":
        return replace(self, mode=mode)

    def with_value(self, value: QuantValue) -> "QuantScheme":
        return replace(self, value=value)

    def with_store(self, store: QuantStore) -> "QuantScheme":
        return replace(self, store=store)

    def with_param(self, param: QuantParam) -> "QuantScheme":
        return replace(self, param=param)

    def size_bits_stored(self) -> int:
        if self.store == QuantStore.U32:
            return 32
        return 8 if self.value == QuantValue.E2M1 else self.value.size_bits()

    def num_quants(self) -> int:
        """Quantized values per stored item: 32/bits for the u32 store; native fp4 keeps two
        codes per byte (crates/cubek-matmul/src/base.rs:506-512), other native stores one."""
        return self.size_bits_stored() // self.value.size_bits()

    def packed_shape(self, shape: Sequence[int]) -> Tuple[int, ...]:
        """Shape of the quantized tensor "from the POV of packed" items (symmetric.rs:68-69)."""
        nq = self.num_quants()
        if shape[-1] % nq:
            raise ValueError(f"last dim {shape[-1]} is not a multiple of num_quants {nq}")
        return tuple(shape[:-1]) + (shape[-1] // nq,)

    def scales_shape(self, shape: Sequence[int]) -> Tuple[int, ...]:
        """[1] per tensor; ceil(shape/block) per block (symmetric.rs:158-159)."""
        if self.level.is_tensor:
            return (1,)
        blk = self.level.block_size.to_dim_vec(len(shape))
        return tuple(-(-s // b) for s, b in zip(shape, blk))
