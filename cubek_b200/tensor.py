"""Borrowed tensor handles and the compute client: the fields of the reference's
``TensorHandleRef`` that the path reads (``handle``, ``shape``, ``strides``, ``elem_size``:
crates/cubek-quant/src/layout/scales.rs:213-215, quantize.rs:234-239) and a ``ComputeClient``
reduced to what a launch needs here: a CUDA device and a stream."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, Tuple


def contiguous_strides(shape: Sequence[int]) -> Tuple[int, ...]:
    strides, acc = [], 1
    for s in reversed(shape):
        strides.append(acc)
        acc *= s
    return tuple(reversed(strides))


@dataclass(frozen=True)
class TensorHandleRef:
    """A borrowed device buffer.  ``handle`` is the device address; strides are in elements."""

    handle: int
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    elem_size: int

    @staticmethod
    def from_torch(t) -> "TensorHandleRef":
        return TensorHandleRef(t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.element_size())

    @staticmethod
    def from_raw_parts(handle: int, shape: Sequence[int], elem_size: int,
                       strides: Sequence[int] | None = None) -> "TensorHandleRef":
        shape = tuple(int(s) for s in shape)
        return TensorHandleRef(int(handle), shape,
                               tuple(strides) if strides is not None else contiguous_strides(shape),
                               int(elem_size))


@dataclass(frozen=True)
class ComputeClient:
    """Launch context: kernels are enqueued on ``stream`` (a raw ``cudaStream_t`` value; 0 is
    the default stream) of ``device`` and the call returns without synchronising, like
    ``launch_unchecked`` in the reference (quantize.rs:256-271)."""

    device: int = 0
    stream: int = 0

    @staticmethod
    def current() -> "ComputeClient":
        import torch

        return ComputeClient(torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)
