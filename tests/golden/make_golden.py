"""Generates tests/golden/quant_golden.npz.

Run from the repository root:  python tests/golden/make_golden.py

The reference cannot be executed where this repository is built (Rust + an un-vendored JIT
dependency), so these vectors are NOT outputs of the reference.  They are outputs of the C
oracle, written only after the independent NumPy / ml_dtypes restatement reproduced every one of
them bit for bit; they freeze today's agreed semantics so that a later change to either the
oracle or the kernels is caught.  Arrays of bfloat16 are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from cubek_b200 import QuantLevel, QuantParam, QuantScheme, QuantStore  # noqa: E402
from oracle import numpy_restatement as R  # noqa: E402
from oracle import oracle as O  # noqa: E402
from tests._cases import FLOATS, adversarial_tensor, all_value_stores, random_tensor, scheme_id  # noqa: E402

OUT = Path(__file__).resolve().parent / "quant_golden.npz"
SHAPE = (8, 128)


def raw(a: np.ndarray) -> np.ndarray:
    return a.view(np.uint16) if a.dtype == FLOATS["bf16"] else a


def cases():
    for fname in FLOATS:
        for value, store in all_value_stores():
            for level in (QuantLevel.Tensor, QuantLevel.block([32])):
                param = QuantParam.F32 if level.is_tensor else (QuantParam.F32, QuantParam.BF16)[value % 2]
                yield fname, QuantScheme(value=value, store=store, level=level, param=param)


def main():
    arrays = {}
    names = []
    for i, (fname, scheme) in enumerate(cases()):
        F = FLOATS[fname]
        x = random_tensor(SHAPE, F, 1000 + i) if i % 2 else adversarial_tensor(SHAPE, F, scheme, 1000 + i)
        scale = O.compute_scales(x, scheme)
        codes, out_scale = O.quantize(x, scale, scheme)
        restored = O.dequantize(codes, out_scale, scheme, F)
        # independent restatement must agree before a vector is written
        assert scale.tobytes() == R.compute_scales(x, scheme).tobytes()
        c2, os2 = R.quantize(x, scale, scheme)
        assert codes.tobytes() == c2.tobytes() and out_scale.tobytes() == os2.tobytes()
        assert restored.tobytes() == R.dequantize(c2, os2, scheme, F).tobytes()
        key = f"{fname}-{scheme_id(scheme)}"
        names.append(key)
        for part, arr in (("x", x), ("scale", scale), ("codes", codes), ("out_scale", out_scale),
                          ("restored", restored)):
            arrays[f"{key}/{part}"] = raw(arr)
    arrays["names"] = np.array(names)
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(names)} cases)")


if __name__ == "__main__":
    main()
