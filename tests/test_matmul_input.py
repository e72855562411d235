"""Tensors quantized with [block_row, block_col] tiles satisfy the reference matmul's quantized-input
contract, and the tile kernels (one warp per tile for the scales, streaming kernels with tile scale
indexing) agree with the oracle bit for bit."""
import numpy as np
import pytest

from cubek_b200 import ElemType, QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue, TensorHandleRef
from cubek_b200.matmul_input import MatmulInputHandleRef
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor


def consumer_view(codes, scales, shape, scheme):
    """Dequantize the way the matmul's global reader addresses a quantized operand: value (row, col) is
    field col % packing of item (row, col / packing); its scale is scales[row / block_row, col / block_col]."""
    nq, bits = scheme.num_quants(), scheme.value.size_bits()
    rows, cols = shape
    br, bc = scheme.level.block_size.as_dim(2)
    out = np.zeros(shape, dtype=np.float32)
    for r in range(rows):
        for c in range(cols):
            raw = (int(codes[r, c // nq]) >> ((c % nq) * bits)) & ((1 << bits) - 1)
            q = raw - (1 << bits) if raw >= (1 << (bits - 1)) else raw
            out[r, c] = np.float32(scales[r // br, c // bc]) * np.float32(q)
    return out


def test_contract_checks():
    scheme = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32, 32]))
    data = TensorHandleRef.from_raw_parts(0x1000, (64, 16), 4)
    scale = TensorHandleRef.from_raw_parts(0x2000, (2, 4), 4)
    h = MatmulInputHandleRef.quantized(data, scale, (64, 128), scheme)
    assert h.block_dims() == (32, 32) and h.data_dtype == "u32" and h.scale_dtype == ElemType.F32
    with pytest.raises(ValueError):
        MatmulInputHandleRef.quantized(data, TensorHandleRef.from_raw_parts(0x2000, (64, 4), 4), (64, 128), scheme)
    with pytest.raises(ValueError):
        MatmulInputHandleRef.quantized(TensorHandleRef.from_raw_parts(0x1000, (64, 16), 4, strides=(1, 64)), scale,
                                       (64, 128), scheme)
    one_d = QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([32]))
    h = MatmulInputHandleRef.quantized(TensorHandleRef.from_raw_parts(0x1000, (8, 16), 4),
                                       TensorHandleRef.from_raw_parts(0x2000, (8, 2), 4), (8, 64), one_d)
    assert h.block_dims() == (1, 32)


def test_oracle_output_reads_back_through_the_consumer_addressing():
    scheme = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([8, 16]))
    x = random_tensor((24, 64), np.float32, 5)
    codes, scales = O.quantize_dynamic(x, scheme)
    assert scales.shape == (3, 4)
    want = O.dequantize(codes, scales, scheme, np.float32)
    assert np.array_equal(consumer_view(codes, scales, x.shape, scheme), want)


@pytest.mark.gpu
@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("shape,block", [((128, 256), [32, 32]), ((256, 512), [128, 128]), ((70, 128), [32, 64]),
                                         ((4, 64, 128), [1, 32, 32]), ((3, 64, 64), [16, 32]), ((48, 96), [16, 32])])
def test_tile_schemes_on_gpu(fname, shape, block):
    from tests._util import (assert_bits_equal, gpu_compute_scales, gpu_dequantize, gpu_quantize, gpu_quantize_dynamic)

    F = FLOATS[fname]
    for value, store in ((QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4F, QuantStore.U32),
                         (QuantValue.E2M1, QuantStore.Native), (QuantValue.Q8S, QuantStore.Native)):
        scheme = QuantScheme(value=value, store=store, level=QuantLevel.block(block), param=QuantParam.F32)
        x = random_tensor(shape, F, 6, "outliers")
        scale = O.compute_scales(x, scheme)
        codes, out_scale = O.quantize(x, scale, scheme)
        assert_bits_equal(gpu_compute_scales(x, scheme), scale, "scales")
        g_codes, g_out_scale = gpu_quantize(x, scale, scheme)
        assert_bits_equal(g_codes, codes, "codes")
        assert_bits_equal(g_out_scale, out_scale, "out_scale")
        d_codes, d_out_scale = gpu_quantize_dynamic(x, scheme)
        assert_bits_equal(d_codes, codes, "codes (fused)")
        assert_bits_equal(d_out_scale, out_scale, "out_scale (fused)")
        assert_bits_equal(gpu_dequantize(codes, out_scale, scheme, F), O.dequantize(codes, out_scale, scheme, F), "restored")
