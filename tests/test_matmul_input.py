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


def unpack_fields(items, bits):
    """[.., n] items -> [.., n * per] raw fields (element 0 in the least significant bits)."""
    per = items.dtype.itemsize * 8 // bits
    shifts = (np.arange(per) * bits).astype(np.uint32)
    f = (items.astype(np.uint32)[..., None] >> shifts) & np.uint32((1 << bits) - 1)
    return f.reshape(items.shape[:-1] + (items.shape[-1] * per,))


def pack_fields(fields, bits, dtype):
    per = np.dtype(dtype).itemsize * 8 // bits
    f = fields.reshape(fields.shape[:-1] + (fields.shape[-1] // per, per)).astype(np.uint32)
    shifts = (np.arange(per) * bits).astype(np.uint32)
    return (f << shifts).sum(axis=-1).astype(np.uint32).astype(dtype)


def test_column_major_contract_checks():
    scheme = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32, 32]))
    # logical (64, 128), packed along the rows: data [64 / 8, 128] with stride 1 on the row dim
    data = TensorHandleRef.from_raw_parts(0x1000, (8, 128), 4, strides=(1, 8))
    scale = TensorHandleRef.from_raw_parts(0x2000, (2, 4), 4)
    h = MatmulInputHandleRef.quantized(data, scale, (64, 128), scheme)
    assert h.col_major
    with pytest.raises(ValueError):     # the row block must hold whole stored items
        MatmulInputHandleRef.quantized(data, TensorHandleRef.from_raw_parts(0x2000, (16, 4), 4), (64, 128),
                                       QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([4, 32])))


@pytest.mark.gpu
@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("value,store", [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4S, QuantStore.U32),
                                         (QuantValue.Q2F, QuantStore.U32), (QuantValue.E2M1, QuantStore.Native),
                                         (QuantValue.Q8S, QuantStore.Native)])
def test_strided_quantized_tensors(fname, value, store):
    """The quantized tensor as a transposed view (memory laid out [n / num_quants, rows]): quantize writes it and
    dequantize reads it through the strides, like the reference's `linear_view(output, 1)`."""
    import torch

    from cubek_b200 import ComputeClient, dequantize, quantize
    from tests._util import assert_bits_equal, code_dtype, elem_of, empty_device, to_device, to_numpy

    F = FLOATS[fname]
    H = TensorHandleRef.from_torch
    for level in (QuantLevel.Tensor, QuantLevel.block([32])):
        scheme = QuantScheme(value=value, store=store, level=level)
        x = random_tensor((48, 256), F, 8, "normal")
        scale = O.compute_scales(x, scheme)
        want_codes, want_scale = O.quantize(x, scale, scheme)
        packed = scheme.packed_shape(x.shape)
        memory = empty_device((packed[1], packed[0]), code_dtype(scheme))
        view = memory.t()                                   # shape `packed`, strides (1, rows)
        assert tuple(view.shape) == tuple(packed) and not view.is_contiguous()
        dos = empty_device(scale.shape, np.float32)
        client = ComputeClient.current()
        dx, dscale = to_device(x), to_device(scale)        # kept alive: handles only borrow
        quantize.launch_ref(client, H(dx), H(view), H(dscale), H(dos), scheme, elem_of(F))
        torch.cuda.synchronize()
        assert_bits_equal(np.ascontiguousarray(to_numpy(memory, code_dtype(scheme)).T), want_codes, "codes through strides")
        assert_bits_equal(to_numpy(dos, np.float32), want_scale, "out_scale")
        out = empty_device(x.shape, F)
        dequantize.launch_ref(client, H(view), H(out), H(dos), scheme, elem_of(F))
        torch.cuda.synchronize()
        assert_bits_equal(to_numpy(out, F), O.dequantize(want_codes, want_scale, scheme, F), "restored through strides")


@pytest.mark.gpu
@pytest.mark.parametrize("value,store", [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4S, QuantStore.U32),
                                         (QuantValue.Q2S, QuantStore.U32), (QuantValue.E2M1, QuantStore.Native),
                                         (QuantValue.E4M3, QuantStore.Native)])
@pytest.mark.parametrize("batch", [(), (3,)])
def test_column_major_operand_into_contiguous(value, store, batch):
    """W is quantized as its transpose (rows of W^T are columns of W), handed over as a column-major operand and
    re-packed along the columns; field for field it must be the oracle's codes, transposed."""
    import torch

    from cubek_b200 import ComputeClient
    from tests._util import assert_bits_equal, code_dtype, empty_device, gpu_quantize_dynamic, to_device, to_numpy

    rows, cols = 96, 160
    scheme = QuantScheme(value=value, store=store, level=QuantLevel.block([32]))
    nq, bits = scheme.num_quants(), scheme.value.size_bits()
    cdt = code_dtype(scheme)
    wt = random_tensor(batch + (cols, rows), np.float32, 9, "normal")               # W^T, contiguous
    codes_t, scales_t = gpu_quantize_dynamic(wt, scheme)                            # [.., cols, rows / nq]
    o_codes_t, _ = O.quantize_dynamic(wt, scheme)
    assert_bits_equal(codes_t, o_codes_t, "codes of the transpose")
    d_codes_t = to_device(codes_t)
    d_scales_t = to_device(scales_t)
    data = TensorHandleRef.from_torch(d_codes_t.transpose(-1, -2))                  # [.., rows / nq, cols], stride 1 on rows
    scale = TensorHandleRef.from_torch(d_scales_t.transpose(-1, -2))                # [.., rows / 32, cols]
    operand_scheme = QuantScheme(value=value, store=store, level=QuantLevel.block([32, 1]))
    h = MatmulInputHandleRef.quantized(data, scale, batch + (rows, cols), operand_scheme)
    assert h.col_major
    out = empty_device(batch + (rows, cols // nq), cdt)
    h2 = h.into_contiguous(ComputeClient.current(), TensorHandleRef.from_torch(out))
    torch.cuda.synchronize()
    assert not h2.col_major
    fields_t = unpack_fields(codes_t.view(np.uint8) if cdt.itemsize == 1 else codes_t, bits)      # [.., cols, rows]
    want = pack_fields(np.swapaxes(fields_t, -1, -2), bits, np.uint8 if cdt.itemsize == 1 else np.uint32)
    got = to_numpy(out, cdt)
    assert_bits_equal(got.view(np.uint8) if cdt.itemsize == 1 else got, want, "re-packed codes")
