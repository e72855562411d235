"""Committed golden vectors (tests/golden/quant_golden.npz, made by tests/golden/make_golden.py):
the oracle must still reproduce them on CPU, and the CUDA kernels must reproduce them on a GPU
without consulting the oracle at all."""
from pathlib import Path

import numpy as np
import pytest

from cubek_b200 import QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue
from tests._cases import FLOATS

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "quant_golden.npz")
NAMES = [str(n) for n in GOLDEN["names"]]


def parse(name):
    fname, value, store, param, level = name.split("-")
    lvl = QuantLevel.Tensor if level == "tensor" else QuantLevel.block([int(v) for v in level[5:].split("x")])
    return FLOATS[fname], QuantScheme(value=QuantValue[value], store=QuantStore[store], param=QuantParam[param],
                                      level=lvl)


def load(name, part, dtype=None):
    a = GOLDEN[f"{name}/{part}"]
    if dtype is not None and a.dtype == np.uint16 and np.dtype(dtype) == FLOATS["bf16"]:
        a = a.view(FLOATS["bf16"])
    return a


def param_dtype(scheme):
    return {QuantParam.F32: FLOATS["f32"], QuantParam.F16: FLOATS["f16"], QuantParam.BF16: FLOATS["bf16"]}[scheme.param]


def test_fixture_is_complete():
    assert len(NAMES) == 72


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_golden(name):
    from oracle import oracle as O

    F, scheme = parse(name)
    x = load(name, "x", F)
    scale = O.compute_scales(x, scheme)
    assert scale.tobytes() == load(name, "scale", F).tobytes()
    codes, out_scale = O.quantize(x, scale, scheme)
    assert codes.tobytes() == load(name, "codes").tobytes()
    assert out_scale.tobytes() == load(name, "out_scale", param_dtype(scheme)).tobytes()
    assert O.dequantize(codes, out_scale, scheme, F).tobytes() == load(name, "restored", F).tobytes()


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_gpu_reproduces_golden(name):
    from tests._util import assert_bits_equal, gpu_compute_scales, gpu_dequantize, gpu_quantize, gpu_quantize_dynamic

    F, scheme = parse(name)
    x = np.ascontiguousarray(load(name, "x", F))
    want_scale = load(name, "scale", F)
    want_codes = load(name, "codes")
    want_out_scale = load(name, "out_scale", param_dtype(scheme))
    want_restored = load(name, "restored", F)

    assert_bits_equal(gpu_compute_scales(x, scheme), want_scale, "scale")
    codes, out_scale = gpu_quantize(x, want_scale, scheme)
    assert_bits_equal(codes, want_codes, "codes")
    assert_bits_equal(out_scale, want_out_scale, "out_scale")
    codes2, out_scale2 = gpu_quantize_dynamic(x, scheme)
    assert_bits_equal(codes2, want_codes, "codes (fused)")
    assert_bits_equal(out_scale2, want_out_scale, "out_scale (fused)")
    assert_bits_equal(gpu_dequantize(want_codes, want_out_scale, scheme, F), want_restored, "restored")
