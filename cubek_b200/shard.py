"""Sharding of one tensor (or a set of tensors) over the GPUs of a node.

The reference is single-device; this is the one data-parallel scheme the path needs.  A 2-D
tensor is split into contiguous row ranges, one per rank.  Blocks lie along the last dim, so a
block never straddles two shards and per-block quantization needs no communication at all.
Per-tensor quantization needs one exchange: the shard-local absmax scalars are max-reduced
(``all_reduce(MAX)`` over NCCL; exact and order independent because absmax >= 0), after which
every rank derives the same scale bits and quantizes its own rows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence, Tuple

from . import quantize as _quantize
from .scheme import ElemType, QuantScheme
from .tensor import ComputeClient, TensorHandleRef


@dataclass(frozen=True)
class RowShard:
    rank: int
    row_start: int
    rows: int


def row_granularity(cols: int, elem: ElemType, scheme: QuantScheme) -> int:
    """Smallest number of rows whose bytes are a multiple of 256 (keeps every shard base aligned
    for 256-bit accesses on input, codes and scales) and whose elements fill whole stored items."""
    nq = scheme.num_quants()
    code_bytes_per_row_x8 = cols * scheme.size_bits_stored() // nq  # bits per row of codes
    g = 1
    for bytes_per_row in (cols * elem.size, max(code_bytes_per_row_x8 // 8, 1)):
        need = 256 // math.gcd(256, bytes_per_row)
        g = g * need // math.gcd(g, need)
    return g


def plan_rows(rows: int, cols: int, world: int, elem: ElemType, scheme: QuantScheme) -> List[RowShard]:
    """Contiguous, non-overlapping row ranges covering ``rows``; every range but the last is a
    multiple of ``row_granularity`` and ranges differ by at most one granule."""
    if world < 1:
        raise ValueError("world must be >= 1")
    if cols % scheme.num_quants():
        raise ValueError("last dim must be a multiple of num_quants")
    if not scheme.level.is_tensor:
        blk = scheme.level.block_size.to_dim_vec(2)
        if blk[0] != 1 or cols % blk[1]:
            raise ValueError("row sharding needs blocks along the last dim that divide it")
    g = row_granularity(cols, elem, scheme)
    granules = -(-rows // g)
    base, extra = divmod(granules, world)
    shards, start = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * g
        n = max(0, min(n, rows - start))
        shards.append(RowShard(r, start, n))
        start += n
    assert start == rows
    return shards


def assign_round_robin(sizes: Sequence[int], world: int) -> List[List[int]]:
    """Whole-tensor placement for weight sets: greedy longest-first onto the least loaded rank.
    Returns, per rank, the indices of the tensors it owns."""
    load = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(sizes)), key=lambda i: -sizes[i]):
        r = min(range(world), key=lambda r: (load[r], r))
        owned[r].append(i)
        load[r] += sizes[i]
    for o in owned:
        o.sort()
    return owned


def allreduce_absmax(absmax, group=None, async_op: bool = False):
    """In-place MAX all-reduce of a tensor of absmax scalars (one per row-sharded tensor).  With ``async_op`` the
    collective is only started: the returned handle's ``wait()`` makes the current stream wait for it (the host
    does not block), so kernels enqueued in between run while the exchange is in flight.  ``None`` is returned
    when there is nothing to wait for."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        return dist.all_reduce(absmax, op=dist.ReduceOp.MAX, group=group, async_op=async_op)
    return None


def quantize_per_tensor_sharded(client: ComputeClient, shard: TensorHandleRef, output: TensorHandleRef,
                                out_scale: TensorHandleRef, absmax, scheme: QuantScheme, elem: ElemType,
                                group=None) -> None:
    """Per-tensor quantization of this rank's rows of a row-sharded tensor.

    ``absmax`` is a 1-element float32 torch tensor on the shard's device.  The three steps run on
    the current stream with no host synchronisation: local absmax, all-reduce(MAX), quantize with
    the scale derived on the device from the reduced value.
    """
    _quantize.absmax(client, shard, elem, absmax.data_ptr())
    allreduce_absmax(absmax, group)
    _quantize.launch_from_absmax(client, shard, output, out_scale, absmax.data_ptr(), scheme, elem)


class ShardedPerTensorSet:
    """Per-tensor quantization of a set of row-sharded tensors: this rank's shards are reduced to one
    absmax each (``qk_absmax_batch``), ONE all-reduce(MAX) of ``len(shards)`` floats makes them global, and
    the shards are quantized in batched launches with scales derived on the device.  Everything is
    enqueued on the current stream; nothing synchronises with the host."""

    def __init__(self, client: ComputeClient, shards, outputs, out_scales, absmax, scheme: QuantScheme,
                 elem: ElemType, group=None):
        from . import _ffi

        if not scheme.level.is_tensor:
            raise ValueError("per-tensor schemes only; per-block shards need no exchange")
        self._in, self._out, self._sc = _ffi.CTensorArray(shards), _ffi.CTensorArray(outputs), _ffi.CTensorArray(out_scales)
        if not (self._in.count == self._out.count == self._sc.count == absmax.numel()):
            raise ValueError("one output, one scale and one absmax cell per shard")
        self._absmax, self._group, self._scheme = absmax, group, _ffi.c_scheme(scheme)
        self._elem, self._stream, self._lib, self._ffi = int(elem), client.stream, _ffi.lib(), _ffi

    def absmax(self) -> None:
        """Phase 1: one absmax per shard into the cells (``qk_absmax_batch``: a memset and one launch per 128 tensors)."""
        self._ffi.check(self._lib.qk_absmax_batch(self._in.count, self._in.array, self._elem, self._absmax.data_ptr(),
                                                  self._stream))

    def exchange(self) -> None:
        """Phase 2: the only collective of the path, MAX over the ranks of one f32 per tensor."""
        allreduce_absmax(self._absmax, self._group)

    def exchange_begin(self) -> None:
        """Phase 2 started, not awaited: independent work enqueued before ``exchange_end`` overlaps it.  Not a gain
        for this library's own kernels: the collective's resident CTAs take SM slots from their one-wave persistent
        grids, and the displaced CTAs run as a second wave (measured on two GPUs: a step 23 % slower)."""
        self._pending = allreduce_absmax(self._absmax, self._group, async_op=True)

    def exchange_end(self) -> None:
        """The current stream waits for the exchange started by ``exchange_begin``."""
        pending, self._pending = getattr(self, "_pending", None), None
        if pending is not None:
            pending.wait()

    def quantize(self) -> None:
        """Phase 3: quantize every shard with the scale derived on the device from its (global) absmax cell."""
        self._ffi.check(self._lib.qk_quantize_from_absmax_batch(self._in.count, self._in.array, self._out.array,
                                                                self._sc.array, self._absmax.data_ptr(), self._scheme,
                                                                self._elem, self._stream))

    def __call__(self) -> None:
        self.absmax()
        self.exchange()
        self.quantize()
