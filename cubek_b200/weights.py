"""Quantized weight sets: a named collection of quantized tensors (codes + scales + scheme) and a
plain on-disk container for it.

The reference has no serialisation for quantized tensors; this is the format the whole-model
quantize flow of this package reads and writes.  A file is

    8 bytes   magic  b"CUBEKQ1\\n"
    8 bytes   little-endian length L of the header
    L bytes   UTF-8 JSON header: {"version": 1, "tensors": [{name, shape, elem, scheme, codes: {dtype,
              shape, offset, nbytes}, scales: {dtype, shape, offset, nbytes}, rows: [start, count] | null}]}
    padding   to a multiple of 256 bytes, then the raw little-endian buffers at their offsets
              (relative to the end of the padded header), each aligned to 256 bytes.

A row-sharded save writes one file per rank; every entry records the row range it holds so that
shards can be concatenated on load.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

from .scheme import (ElemType, QuantLevel, QuantMode, QuantParam, QuantScheme, QuantStore, QuantValue)

MAGIC = b"CUBEKQ1\n"
ALIGN = 256


def scheme_to_dict(s: QuantScheme) -> dict:
    return {"value": s.value.name, "param": s.param.name, "store": s.store.name, "mode": s.mode.name,
            "level": "tensor" if s.level.is_tensor else list(s.level.block_size.as_slice())}


def scheme_from_dict(d: dict) -> QuantScheme:
    level = QuantLevel.Tensor if d["level"] == "tensor" else QuantLevel.block(d["level"])
    return QuantScheme(value=QuantValue[d["value"]], param=QuantParam[d["param"]], store=QuantStore[d["store"]],
                       level=level, mode=QuantMode[d["mode"]])


@dataclass
class QuantizedTensor:
    """Host copy of one quantized tensor.  ``codes`` is uint32 (u32 store) or int8 / uint8 (native);
    ``scales`` is stored as raw bits (uint32 for f32 params, uint16 for f16 / bf16)."""

    name: str
    shape: Tuple[int, ...]          # unpacked shape of this piece
    elem: ElemType                  # float type the tensor dequantizes to
    scheme: QuantScheme
    codes: np.ndarray
    scales: np.ndarray
    rows: Optional[Tuple[int, int]] = None   # (row_start, row_count) when this is a row shard


def _pad(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def save(path, tensors: Iterable[QuantizedTensor]) -> None:
    tensors = list(tensors)
    entries, offset = [], 0
    for t in tensors:
        e = {"name": t.name, "shape": list(t.shape), "elem": t.elem.name, "scheme": scheme_to_dict(t.scheme),
             "rows": list(t.rows) if t.rows else None}
        for key, arr in (("codes", t.codes), ("scales", t.scales)):
            arr = np.ascontiguousarray(arr)
            e[key] = {"dtype": arr.dtype.str, "shape": list(arr.shape), "offset": offset, "nbytes": arr.nbytes}
            offset += _pad(arr.nbytes)
        entries.append(e)
    header = json.dumps({"version": 1, "tensors": entries}).encode()
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        f.write(b"\0" * (_pad(16 + len(header)) - 16 - len(header)))
        for t in tensors:
            for arr in (t.codes, t.scales):
                raw = np.ascontiguousarray(arr).tobytes()
                f.write(raw)
                f.write(b"\0" * (_pad(len(raw)) - len(raw)))


def load(path) -> List[QuantizedTensor]:
    data = Path(path).read_bytes()
    if data[:8] != MAGIC:
        raise ValueError(f"{path}: not a quantized weight file")
    (hlen,) = struct.unpack("<Q", data[8:16])
    header = json.loads(data[16:16 + hlen].decode())
    if header.get("version") != 1:
        raise ValueError(f"{path}: unsupported version {header.get('version')}")
    base = _pad(16 + hlen)
    out = []
    for e in header["tensors"]:
        arrs = {}
        for key in ("codes", "scales"):
            m = e[key]
            start = base + m["offset"]
            arrs[key] = np.frombuffer(data, dtype=np.dtype(m["dtype"]), count=int(np.prod(m["shape"], dtype=np.int64)),
                                      offset=start).reshape(m["shape"]).copy()
        out.append(QuantizedTensor(e["name"], tuple(e["shape"]), ElemType[e["elem"]], scheme_from_dict(e["scheme"]),
                                   arrs["codes"], arrs["scales"], tuple(e["rows"]) if e["rows"] else None))
    return out


def merge_row_shards(pieces: Iterable[QuantizedTensor]) -> QuantizedTensor:
    """Concatenate the row shards of one tensor (per-block schemes, or per-tensor ones quantized with the
    all-reduced absmax, whose single scale is identical on every shard)."""
    pieces = sorted(pieces, key=lambda p: p.rows[0])
    first = pieces[0]
    expect = 0
    for p in pieces:
        if p.rows is None or p.rows[0] != expect or p.name != first.name or p.scheme != first.scheme:
            raise ValueError("shards do not tile the tensor")
        expect += p.rows[1]
    codes = np.concatenate([p.codes for p in pieces], axis=0)
    if first.scheme.level.is_tensor:
        if any(p.scales.tobytes() != first.scales.tobytes() for p in pieces):
            raise ValueError("per-tensor shards disagree on the scale")
        scales = first.scales
    else:
        scales = np.concatenate([p.scales for p in pieces], axis=0)
    return QuantizedTensor(first.name, (expect,) + tuple(first.shape[1:]), first.elem, first.scheme, codes, scales, None)


def llama3_8b_shapes() -> List[Tuple[str, int, int]]:
    """(name, rows, cols) of the 225 matrices of a Llama-3-8B-shaped model (32 layers + embedding)."""
    from .synthetic import LLAMA3_8B_EMBEDDING, LLAMA3_8B_LAYER, LLAMA3_8B_LAYERS

    out = []
    for layer in range(LLAMA3_8B_LAYERS):
        out += [(f"layers.{layer}.{n}", r, c) for n, r, c in LLAMA3_8B_LAYER]
    out.append(LLAMA3_8B_EMBEDDING)
    return out
