"""The reference's own quantization tests, restated: 6 values x 2 shapes x {tensor, block}
(crates/cubek-quant/tests/suite/mod.rs:15-57), with its inputs, its scale formula and its
tolerance (crates/cubek-quant/tests/suite/symmetric.rs:24-141 and :143-284).

On CPU they pin the oracle; on a GPU the same bodies run through the C ABI.
"""
import numpy as np
import pytest

from cubek_b200 import QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue
from oracle import oracle as O

VALUES = [QuantValue.Q8F, QuantValue.Q8S, QuantValue.Q4F, QuantValue.Q4S, QuantValue.Q2F, QuantValue.Q2S]
SHAPES = [(32, 32), (16, 64)]


def tensor_case(m, n, value):
    num = m * n
    half = np.float32(num) / np.float32(2)
    data = (np.arange(num, dtype=np.float32) - half).reshape(m, n)          # symmetric.rs:29-31
    q_min, q_max = value.range()
    scale = np.array([(np.float32(2) * half) / np.float32(q_max - q_min)], dtype=np.float32)  # :35-38
    scheme = QuantScheme(value=value, store=QuantStore.U32, param=QuantParam.F32, level=QuantLevel.Tensor)
    return data, scale, scheme


def block_case(m, n, value):
    block = m                                                                # "Shape x as block_size", :19-21
    num = m * n
    half = np.float32(num) / np.float32(2)
    data = ((np.arange(num, dtype=np.float32) - half) / np.float32(num)).reshape(m, n)   # :150-152
    q_min, q_max = value.range()
    blocks = data.reshape(-1, block)
    rng = np.float32(2) * np.maximum(np.abs(blocks.min(axis=1)), np.abs(blocks.max(axis=1)))
    scale = (rng / np.float32(q_max - q_min)).astype(np.float32).reshape(m, n // block)     # :161-179
    scheme = QuantScheme(value=value, store=QuantStore.U32, param=QuantParam.F32, level=QuantLevel.block([block]))
    return data, scale, scheme


def check_tolerance(data, restored, scale, block):
    rel_tol = np.float32(1e-4)
    per_elem = np.repeat(scale.reshape(-1), block) if block else np.full(data.size, scale[0], dtype=np.float32)
    max_err = (per_elem / np.float32(2)) * (np.float32(1) + rel_tol)         # :130-131, :275
    diff = np.abs(restored.reshape(-1) - data.reshape(-1))
    assert np.all(diff <= max_err), f"max diff/tol = {np.max(diff / max_err)}"


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("value", VALUES)
def test_quantization_symmetric_tensor_oracle(shape, value):
    data, scale, scheme = tensor_case(*shape, value)
    q, out_scale = O.quantize(data, scale, scheme)
    assert q.shape == (shape[0], shape[1] // scheme.num_quants()) and q.dtype == np.uint32
    assert out_scale.tobytes() == scale.tobytes()
    restored = O.dequantize(q, out_scale, scheme, np.float32)
    check_tolerance(data, restored, scale, 0)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("value", VALUES)
def test_quantization_symmetric_block_oracle(shape, value):
    data, scale, scheme = block_case(*shape, value)
    # the formula of the reference test is what compute_scales implements
    assert O.compute_scales(data, scheme).tobytes() == scale.tobytes()
    q, out_scale = O.quantize(data, scale, scheme)
    restored = O.dequantize(q, out_scale, scheme, np.float32)
    check_tolerance(data, restored, scale, shape[0])


@pytest.mark.gpu
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("value", VALUES)
def test_quantization_symmetric_tensor_gpu(shape, value):
    from tests._util import assert_bits_equal, gpu_dequantize, gpu_quantize

    data, scale, scheme = tensor_case(*shape, value)
    q, out_scale = gpu_quantize(data, scale, scheme)
    restored = gpu_dequantize(q, out_scale, scheme, np.float32)
    check_tolerance(data, restored, scale, 0)
    oq, oscale = O.quantize(data, scale, scheme)
    assert_bits_equal(q, oq, "codes")
    assert_bits_equal(out_scale, oscale, "out_scale")
    assert_bits_equal(restored, O.dequantize(oq, oscale, scheme, np.float32), "restored")


@pytest.mark.gpu
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("value", VALUES)
def test_quantization_symmetric_block_gpu(shape, value):
    from tests._util import assert_bits_equal, gpu_compute_scales, gpu_dequantize, gpu_quantize

    data, scale, scheme = block_case(*shape, value)
    assert_bits_equal(gpu_compute_scales(data, scheme), scale, "scales")
    q, out_scale = gpu_quantize(data, scale, scheme)
    restored = gpu_dequantize(q, out_scale, scheme, np.float32)
    check_tolerance(data, restored, scale, shape[0])
    oq, oscale = O.quantize(data, scale, scheme)
    assert_bits_equal(q, oq, "codes")
    assert_bits_equal(restored, O.dequantize(oq, oscale, scheme, np.float32), "restored")
