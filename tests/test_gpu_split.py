"""How the streaming kernels hand units to CTAs and threads: contiguous runs of 32-unit rows per CTA, a partial
last pass, half-unit blocks (two 16-element blocks of a 16-bit type in one 64-byte unit).  Sizes are chosen so
that rows do not divide by the grid, units do not fill the last row and tensors of a batch end inside a row;
every result is compared with the oracle bit for bit."""
import numpy as np
import pytest
import torch

from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef,
                        dequantize, quantize)
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import (NP_FLOAT, assert_bits_equal, code_dtype, elem_of, empty_device, gpu_compute_scales,
                         gpu_dequantize, gpu_quantize, gpu_quantize_dynamic, to_device, to_numpy)

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch


def round_trip_matches_oracle(x, scheme):
    F = x.dtype
    codes, out_scale = O.quantize_dynamic(x, scheme)
    g_codes, g_scale = gpu_quantize_dynamic(x, scheme)
    assert_bits_equal(g_scale, out_scale, "out_scale (fused)")
    assert_bits_equal(g_codes, codes, "codes (fused)")
    scale = O.compute_scales(x, scheme)
    assert_bits_equal(gpu_compute_scales(x, scheme), scale, "scale")
    g_codes, g_scale = gpu_quantize(x, scale, scheme)
    assert_bits_equal(g_codes, codes, "codes (given scales)")
    assert_bits_equal(gpu_dequantize(codes, out_scale, scheme, F), O.dequantize(codes, out_scale, scheme, F), "restored")


@pytest.mark.parametrize("fname", ["f16", "bf16"])
@pytest.mark.parametrize("value,store", [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q8F, QuantStore.Native),
                                         (QuantValue.Q4S, QuantStore.U32), (QuantValue.Q4F, QuantStore.U32),
                                         (QuantValue.Q2S, QuantStore.U32), (QuantValue.E2M1, QuantStore.Native),
                                         (QuantValue.E4M3, QuantStore.Native), (QuantValue.E5M2, QuantStore.Native)])
def test_two_blocks_per_unit(fname, value, store):
    """Blocks of 16 elements of a 16-bit type: the fused kernel runs them as halves of 64-byte units."""
    scheme = QuantScheme(value=value, store=store, level=QuantLevel.block([16]))
    F = FLOATS[fname]
    round_trip_matches_oracle(random_tensor((1031, 4096), F, 41, "rowscaled"), scheme)
    round_trip_matches_oracle(random_tensor((3, 32), F, 42, "normal"), scheme)
    x = random_tensor((257, 160), F, 43, "outliers")
    x[5, :] = 0                     # zero blocks: scale 0, reference-arithmetic route inside one half
    x[7, 16:32] = 0
    round_trip_matches_oracle(x, scheme)


def test_two_blocks_per_unit_with_scales_off_the_8_byte_boundary():
    """The two scales of a unit leave as one 8-byte store; a scales buffer that starts 4 bytes off takes the
    one-block-per-unit kernel instead.  Same bits either way."""
    scheme = QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16]))
    x = random_tensor((512, 1024), np.float16, 44, "rowscaled")
    want_codes, want_scale = O.quantize_dynamic(x, scheme)
    dx = to_device(x)
    dq = empty_device(scheme.packed_shape(x.shape), code_dtype(scheme))
    pool = torch.zeros(want_scale.size + 1, dtype=torch.float32, device="cuda")
    ds = pool[1:].view(want_scale.shape)
    assert ds.data_ptr() % 8 == 4
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic(ComputeClient.current(), H(dx), H(dq), H(ds), scheme, ElemType.F16, H(ws))
    torch.cuda.synchronize()
    assert_bits_equal(to_numpy(dq, code_dtype(scheme)), want_codes, "codes")
    assert_bits_equal(to_numpy(ds, np.float32), want_scale, "scales")
    assert float(pool[0]) == 0.0


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("rows,cols", [(1, 64), (37, 64), (4099, 192), (2 * 148 * 3 * 8 + 5, 2048), (9001, 4096)])
@pytest.mark.parametrize("level", ["tensor", "block32", "block64"])
def test_uneven_work_split(fname, rows, cols, level):
    F = FLOATS[fname]
    lvl = QuantLevel.Tensor if level == "tensor" else QuantLevel.block([int(level[5:])])
    for value in (QuantValue.Q8S, QuantValue.Q4S):
        round_trip_matches_oracle(random_tensor((rows, cols), F, rows + cols, "normal"),
                                  QuantScheme(value=value, store=QuantStore.U32, level=lvl))


def test_batch_members_that_end_inside_a_row_of_units():
    """Tensors of 3, 1, 50 and 7 units (64 bytes each) in one launch: warps hold units of several tensors."""
    scheme = QuantScheme(value=QuantValue.Q4S, store=QuantStore.U32, level=QuantLevel.block([32]))
    elem, F = ElemType.BF16, NP_FLOAT[ElemType.BF16]
    shapes = [(3, 32), (1, 32), (50, 32), (7, 32), (1000, 4096), (1, 64)]
    xs = [random_tensor(sh, F, 50 + i, "normal") for i, sh in enumerate(shapes)]
    dxs = [to_device(x) for x in xs]
    codes = [empty_device(scheme.packed_shape(x.shape), np.uint32) for x in xs]
    scales = [empty_device(scheme.scales_shape(x.shape), np.float32) for x in xs]
    outs = [empty_device(x.shape, F) for x in xs]
    client = ComputeClient.current()
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic_batch(client, [H(t) for t in dxs], [H(t) for t in codes], [H(t) for t in scales], scheme, elem, H(ws))
    dequantize.launch_batch(client, [H(t) for t in codes], [H(t) for t in outs], [H(t) for t in scales], scheme, elem)
    torch.cuda.synchronize()
    for i, x in enumerate(xs):
        o_codes, o_scale = O.quantize_dynamic(x, scheme)
        assert_bits_equal(to_numpy(codes[i], np.uint32), o_codes, f"codes {i}")
        assert_bits_equal(to_numpy(scales[i], np.float32), o_scale, f"scales {i}")
        assert_bits_equal(to_numpy(outs[i], F), O.dequantize(o_codes, o_scale, scheme, F), f"restored {i}")


def test_two_blocks_per_unit_dequantize_with_params_off_the_8_byte_boundary():
    """The dequantize kernel fetches the two scales of a unit with one 8-byte load; params that start 4 bytes off
    take the one-block-per-unit kernel.  Same bits either way."""
    scheme = QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16]))
    x = random_tensor((512, 1024), np.float16, 45, "rowscaled")
    codes, scales = O.quantize_dynamic(x, scheme)
    want = O.dequantize(codes, scales, scheme, np.float16)
    dcodes = to_device(codes)
    pool = torch.zeros(scales.size + 1, dtype=torch.float32, device="cuda")
    dparams = pool[1:].view(scales.shape)
    dparams.copy_(to_device(scales))
    assert dparams.data_ptr() % 8 == 4
    for params in (dparams, to_device(scales)):
        out = empty_device(x.shape, np.float16)
        dequantize.launch_ref(ComputeClient.current(), H(dcodes), H(out), H(params), scheme, ElemType.F16)
        torch.cuda.synchronize()
        assert_bits_equal(to_numpy(out, np.float16), want, "restored")
