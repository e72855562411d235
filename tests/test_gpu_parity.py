"""CUDA kernels against the oracle, bit for bit, through the C ABI: every value x store x float
type x level, on random and adversarial inputs; the streaming kernels, their reference-arithmetic
route and the layout-general kernels must all give the same bits."""
import itertools

import numpy as np
import pytest

from cubek_b200 import ElemType, QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue
from cubek_b200 import _ffi
from oracle import oracle as O
from tests._cases import FLOATS, adversarial_tensor, all_value_stores, random_tensor, scheme_grid, scheme_id
from tests._util import (assert_bits_equal, gpu_compute_scales, gpu_dequantize, gpu_quantize, gpu_quantize_dynamic)

pytestmark = pytest.mark.gpu

SHAPE = (64, 256)


def full_check(x, scheme, F):
    scale = O.compute_scales(x, scheme)
    codes, out_scale = O.quantize(x, scale, scheme)
    restored = O.dequantize(codes, out_scale, scheme, F)
    assert_bits_equal(gpu_compute_scales(x, scheme), scale, "scale")
    g_codes, g_out_scale = gpu_quantize(x, scale, scheme)
    assert_bits_equal(g_codes, codes, "codes")
    assert_bits_equal(g_out_scale, out_scale, "out_scale")
    d_codes, d_out_scale = gpu_quantize_dynamic(x, scheme)
    assert_bits_equal(d_codes, codes, "codes (fused)")
    assert_bits_equal(d_out_scale, out_scale, "out_scale (fused)")
    assert_bits_equal(gpu_dequantize(codes, out_scale, scheme, F), restored, "restored")


@pytest.fixture
def tuning():
    yield lambda key, value: _ffi.lib().qk_set_tuning(key, value)
    for key in (_ffi.TUNE_FORCE_EXACT, _ffi.TUNE_FORCE_GENERAL, _ffi.TUNE_STAGED):
        _ffi.lib().qk_set_tuning(key, 0)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", list(scheme_grid(SHAPE)), ids=scheme_id)
def test_streaming_kernels(fname, scheme):
    F = FLOATS[fname]
    full_check(random_tensor(SHAPE, F, 1), scheme, F)
    full_check(adversarial_tensor(SHAPE, F, scheme, 2), scheme, F)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", list(scheme_grid(SHAPE)), ids=scheme_id)
def test_reference_arithmetic_route(fname, scheme, tuning):
    tuning(_ffi.TUNE_FORCE_EXACT, 1)
    F = FLOATS[fname]
    full_check(adversarial_tensor(SHAPE, F, scheme, 3), scheme, F)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", list(scheme_grid(SHAPE)), ids=scheme_id)
def test_layout_general_kernels(fname, scheme, tuning):
    tuning(_ffi.TUNE_FORCE_GENERAL, 1)
    F = FLOATS[fname]
    full_check(adversarial_tensor(SHAPE, F, scheme, 4), scheme, F)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("param", [QuantParam.F16, QuantParam.BF16])
@pytest.mark.parametrize("value,store", [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4F, QuantStore.U32),
                                         (QuantValue.E2M1, QuantStore.Native), (QuantValue.Q8F, QuantStore.Native)])
def test_half_precision_params(fname, param, value, store):
    F = FLOATS[fname]
    for level in (QuantLevel.Tensor, QuantLevel.block([32])):
        scheme = QuantScheme(value=value, store=store, param=param, level=level)
        full_check(random_tensor(SHAPE, F, 5), scheme, F)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("shape,block", [((6, 10, 48), [2, 16]), ((5, 96), [24]), ((7, 3, 40), [3, 1, 8]),
                                         ((33, 24), [8]), ((4, 4, 4, 16), [2, 2, 16])])
def test_nd_blocks_and_ragged_shapes(fname, shape, block):
    """Blocks over several dims (clipped at the edges), block sizes that are not powers of two
    and sizes that do not fill whole units all go through the layout-general kernels."""
    F = FLOATS[fname]
    for value, store in ((QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4S, QuantStore.U32),
                         (QuantValue.Q8S, QuantStore.Native), (QuantValue.E2M1, QuantStore.Native)):
        scheme = QuantScheme(value=value, store=store, level=QuantLevel.block(block))
        if block[-1] % scheme.num_quants() or shape[-1] % scheme.num_quants():
            continue
        full_check(random_tensor(shape, F, 6), scheme, F)


def test_strided_scales_are_honoured():
    """scale / out_scale / params may be views with their own strides (the reference builds its
    scales layout from the handle's strides, layout/scales.rs:233-234)."""
    import torch
    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from tests._util import to_device, to_numpy

    F = np.float32
    scheme = QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([32]))
    x = random_tensor(SHAPE, F, 7)
    scale = O.compute_scales(x, scheme)
    codes, out_scale = O.quantize(x, scale, scheme)
    dx = to_device(x)
    wide = torch.zeros((SHAPE[0], 2 * scale.shape[1]), device="cuda")
    dscale = wide[:, ::2]
    dscale.copy_(torch.from_numpy(scale))
    wide_out = torch.full((SHAPE[0], 3 * scale.shape[1]), -1.0, device="cuda")
    dos = wide_out[:, 1::3]
    dq = torch.zeros(codes.shape, dtype=torch.int32, device="cuda")
    client = ComputeClient.current()
    quantize.launch_ref(client, TensorHandleRef.from_torch(dx), TensorHandleRef.from_torch(dq),
                        TensorHandleRef.from_torch(dscale), TensorHandleRef.from_torch(dos), scheme, ElemType.F32)
    do = torch.zeros(SHAPE, device="cuda")
    dequantize.launch_ref(client, TensorHandleRef.from_torch(dq), TensorHandleRef.from_torch(do),
                          TensorHandleRef.from_torch(dos), scheme, ElemType.F32)
    torch.cuda.synchronize()
    assert_bits_equal(to_numpy(dq, np.uint32), codes, "codes")
    assert_bits_equal(dos.contiguous().cpu().numpy(), out_scale, "out_scale")
    assert float(wide_out[:, 0::3].max()) == -1.0 and float(wide_out[:, 2::3].max()) == -1.0
    assert_bits_equal(do.cpu().numpy(), O.dequantize(codes, out_scale, scheme, F), "restored")


def test_e2m1_nibble_order_and_code_table():
    """All 16 fp4 codes through the native dequantize, and the integers -6..6 through the native
    quantize: even element in the low nibble, 5 -> 4."""
    scheme = QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native)
    one = np.array([1.0], dtype=np.float32)
    codes = np.array([[lo | (hi << 4) for lo, hi in zip(range(0, 16, 2), range(1, 16, 2))]], dtype=np.uint8)
    got = gpu_dequantize(codes, one, scheme, np.float32)
    want = np.array([[0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]], dtype=np.float32)
    assert np.array_equal(got, want)
    assert_bits_equal(got, O.dequantize(codes, one, scheme, np.float32), "e2m1 table")
    x = np.array([[-6, -5, -4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 6, 7, 0.4, 2.5]], dtype=np.float32)
    q, _ = gpu_quantize(x, one, scheme)
    oq, _ = O.quantize(x, one, scheme)
    assert_bits_equal(q, oq, "e2m1 codes")
    back = gpu_dequantize(q, one, scheme, np.float32)
    assert back.reshape(-1).tolist() == [-6, -4, -4, -3, -2, -1, 0, 1, 2, 3, 4, 4, 6, 6, 0, 2]


@pytest.mark.parametrize("fname", ["f16", "bf16"])
@pytest.mark.parametrize("value,store", [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4S, QuantStore.U32),
                                         (QuantValue.Q2F, QuantStore.U32), (QuantValue.E2M1, QuantStore.Native),
                                         (QuantValue.E4M3, QuantStore.Native)])
def test_every_finite_half_value_as_input(fname, value, store):
    """All 2^16 bit patterns of the input type (non-finite and huge ones replaced by 0) against several
    scales: exercises every rounding boundary of the narrowed quotient."""
    F = FLOATS[fname]
    bits = np.arange(65536, dtype=np.uint16)
    x = bits.view(F).copy()
    xf = x.astype(np.float32)
    x[~np.isfinite(xf) | (np.abs(xf) > 1e18)] = 0     # 2*absmax must stay finite in f32
    x = x.reshape(256, 256)
    scheme = QuantScheme(value=value, store=store)
    for s in (1.0, 0.37109375, 3.0, 0.0078125, 119.5):
        scale = np.array([s], dtype=F)
        codes, out_scale = O.quantize(x, scale, scheme)
        g_codes, g_out_scale = gpu_quantize(x, scale, scheme)
        assert_bits_equal(g_codes, codes, f"codes at scale {s}")
        assert_bits_equal(g_out_scale, out_scale, "out_scale")
    codes, out_scale = O.quantize_dynamic(x, scheme)
    assert_bits_equal(gpu_dequantize(codes, out_scale, scheme, F), O.dequantize(codes, out_scale, scheme, F), "restored")


@pytest.mark.parametrize("fname,kind,value,store,level", [
    ("f32", "normal", QuantValue.Q8S, QuantStore.U32, QuantLevel.Tensor),
    ("bf16", "outliers", QuantValue.Q4S, QuantStore.U32, QuantLevel.block([32])),
    ("f16", "rowscaled", QuantValue.E2M1, QuantStore.Native, QuantLevel.block([16])),
    ("f16", "rowscaled", QuantValue.E2M1, QuantStore.Native, QuantLevel.block([32])),
    ("f32", "uniform", QuantValue.Q2S, QuantStore.U32, QuantLevel.block([64])),
    ("bf16", "normal", QuantValue.Q8S, QuantStore.U32, QuantLevel.block([128])),
    ("bf16", "normal", QuantValue.Q8S, QuantStore.U32, QuantLevel.Tensor),
])
def test_benchmark_configurations_medium(fname, kind, value, store, level):
    """The benchmark schemes and distributions on 1024 x 4096 tensors: large enough that every
    CTA loops and the grid cap is reached, small enough for the oracle."""
    F = FLOATS[fname]
    scheme = QuantScheme(value=value, store=store, level=level)
    full_check(random_tensor((1024, 4096), F, 8, kind), scheme, F)


def test_scale_extremes_take_the_reference_route():
    """Scales outside the shortcut window (zero, subnormal, huge, negative) and quotients that
    overflow must match the oracle too."""
    scheme = QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([32]))
    x = random_tensor((8, 256), np.float32, 9)
    x[0] *= 1e30
    x[1] *= 1e-30
    x[2] *= 1e-42
    scale = O.compute_scales(x, scheme)
    scale[3] = 1e-38
    scale[4] = -0.01
    scale[5] = 3e38
    scale[6] = 1e-45
    codes, out_scale = O.quantize(x, scale, scheme)
    g_codes, g_out_scale = gpu_quantize(x, scale, scheme)
    assert_bits_equal(g_codes, codes, "codes")
    d_codes, _ = gpu_quantize_dynamic(x, scheme)
    assert_bits_equal(d_codes, O.quantize_dynamic(x, scheme)[0], "codes (fused)")


@pytest.mark.parametrize("fname", ["f16", "bf16"])
@pytest.mark.parametrize("value", [QuantValue.E5M2, QuantValue.E4M3])
def test_fp8_codes_of_half_inputs_up_to_and_past_the_clamp(fname, value):
    """fp8 codes of 16-bit inputs take the shortcut arithmetic up to the clamp bound (57344 for e5m2);
    quotients that overflow f16 to infinity, or land between the bound and the largest finite value,
    must clamp like the reference arithmetic.  Both routes are compared with the oracle."""
    F = FLOATS[fname]
    scheme = QuantScheme(value=value, store=QuantStore.Native, level=QuantLevel.block([32]))
    lo, hi = scheme.value.range()
    rng = np.random.default_rng(1234)
    shape = (64, 256)
    n = shape[0] * shape[1]
    # quotients spread log-uniformly from 1/4 to 4 x the bound, both signs, plus exact bounds and ties
    q = np.exp(rng.uniform(np.log(0.25), np.log(4.0 * hi), n)).astype(np.float32) * rng.choice([-1.0, 1.0], n).astype(np.float32)
    q[::97] = hi
    q[1::97] = -hi
    q[2::97] = np.float32(hi) * np.float32(1.0009765625)
    q[3::97] = 2.5
    x = (q * np.float32(0.25)).reshape(shape).astype(F)            # given scale 0.25: exact in every F
    scale = np.full(scheme.scales_shape(shape), 0.25, dtype=F)
    codes, out_scale = O.quantize(x, scale, scheme)
    g_codes, g_out_scale = gpu_quantize(x, scale, scheme)
    assert_bits_equal(g_codes, codes, "codes (given scale)")
    assert_bits_equal(g_out_scale, out_scale, "out_scale")
    d_codes, d_scale = gpu_quantize_dynamic(x, scheme)
    o_codes, o_scale = O.quantize_dynamic(x, scheme)
    assert_bits_equal(d_codes, o_codes, "codes (fused)")
    assert_bits_equal(d_scale, o_scale, "scales (fused)")


@pytest.mark.parametrize("fname", list(FLOATS))
def test_per_tensor_routes_agree(fname, tuning):
    """Per tensor, the fused call has two routes: one cooperative launch (absmax, grid barrier,
    quantize) when the workspace holds a partial per CTA, else absmax kernel + quantize kernel.
    Both must give the oracle's bits, on tensors of many CTAs and of a single one."""
    import torch
    from cubek_b200 import ComputeClient, TensorHandleRef, quantize
    from tests._util import code_dtype, elem_of, empty_device, to_device, to_numpy

    F = FLOATS[fname]
    H = TensorHandleRef.from_torch
    for value, store in ((QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4F, QuantStore.U32),
                         (QuantValue.E2M1, QuantStore.Native)):
        scheme = QuantScheme(value=value, store=store)
        for shape in ((1024, 4096), (8, 256), (3, 32)):
            x = random_tensor(shape, F, 77)
            want_codes, want_scale = O.quantize_dynamic(x, scheme)
            for ws_bytes in (8192, 256):
                dx = to_device(x)
                dq = empty_device(scheme.packed_shape(shape), code_dtype(scheme))
                ds = empty_device((1,), np.float32)
                ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
                quantize.launch_dynamic(ComputeClient.current(), H(dx), H(dq), H(ds), scheme, elem_of(F), H(ws))
                torch.cuda.synchronize()
                assert_bits_equal(to_numpy(dq, code_dtype(scheme)), want_codes, f"codes ws={ws_bytes}")
                assert_bits_equal(to_numpy(ds, np.float32), want_scale, f"scale ws={ws_bytes}")


@pytest.mark.parametrize("fname", list(FLOATS))
def test_strided_float_tensors(fname):
    """Inputs of quantize / compute_scales and outputs of dequantize may be strided views
    (transposed, sliced): the reference reads them through `linear_view`."""
    import torch
    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from tests._util import code_dtype, elem_of, empty_device, to_device, to_numpy

    F = FLOATS[fname]
    H = TensorHandleRef.from_torch
    client = ComputeClient.current()
    for scheme in (QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([32])),
                   QuantScheme(value=QuantValue.Q4S), QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native,
                                                                  level=QuantLevel.block([2, 16]))):
        base = random_tensor((96, 80), F, 88)
        views = {"transposed": (to_device(base).t(), np.ascontiguousarray(base.T)),
                 "sliced": (to_device(base)[8:72, 16:80], np.ascontiguousarray(base[8:72, 16:80]))}
        for name, (dv, x) in views.items():
            assert not dv.is_contiguous()
            want_scale = O.compute_scales(x, scheme)
            want_codes, want_out_scale = O.quantize(x, want_scale, scheme)
            ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
            dscale = empty_device(want_scale.shape, F)
            quantize.compute_scales(client, H(dv), H(dscale), scheme, elem_of(F), H(ws))
            dq = empty_device(want_codes.shape, code_dtype(scheme))
            dos = empty_device(want_out_scale.shape, np.float32)
            quantize.launch_ref(client, H(dv), H(dq), H(dscale), H(dos), scheme, elem_of(F))
            dq2 = empty_device(want_codes.shape, code_dtype(scheme))
            dos2 = empty_device(want_out_scale.shape, np.float32)
            quantize.launch_dynamic(client, H(dv), H(dq2), H(dos2), scheme, elem_of(F), H(ws))
            # dequantize into a strided view of a larger buffer
            big = torch.zeros((x.shape[0], 2 * x.shape[1]), dtype=dv.dtype, device="cuda")
            dout = big[:, ::2]
            dequantize.launch_ref(client, H(dq), H(dout), H(dos), scheme, elem_of(F))
            torch.cuda.synchronize()
            assert_bits_equal(to_numpy(dscale, F), want_scale, f"{name} scale")
            assert_bits_equal(to_numpy(dq, code_dtype(scheme)), want_codes, f"{name} codes")
            assert_bits_equal(to_numpy(dq2, code_dtype(scheme)), want_codes, f"{name} codes (fused)")
            assert_bits_equal(to_numpy(dos2, np.float32), want_out_scale, f"{name} out_scale (fused)")
            assert_bits_equal(to_numpy(dout.contiguous(), F), O.dequantize(want_codes, want_out_scale, scheme, F),
                              f"{name} restored")
            assert float(big[:, 1::2].float().abs().max()) == 0.0


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("offset_bytes", [16, 8, 4, 48])
def test_odd_base_alignments(fname, offset_bytes):
    """Tensors that start 4, 8, 16 or 48 bytes into an allocation: 256-bit accesses are not allowed
    (128-bit route), or not even those (general kernels).  Same bits either way."""
    import torch
    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from tests._util import code_dtype, elem_of, to_numpy

    F = FLOATS[fname]
    H = TensorHandleRef.from_torch
    client = ComputeClient.current()
    shape = (64, 512)
    n = shape[0] * shape[1]
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[fname]
    esz = np.dtype(F).itemsize
    for scheme in (QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32])),
                   QuantScheme(value=QuantValue.Q8S), QuantScheme(value=QuantValue.Q2S, level=QuantLevel.block([64]))):
        x = random_tensor(shape, F, 91)
        want_codes, want_scale = O.quantize_dynamic(x, scheme)
        want_restored = O.dequantize(want_codes, want_scale, scheme, F)
        raw_in = torch.zeros(n * esz + 256, dtype=torch.uint8, device="cuda")
        dx = raw_in[offset_bytes: offset_bytes + n * esz].view(tdt).view(shape)
        dx.copy_(torch.from_numpy(x.view(np.int16) if fname == "bf16" else x).cuda().view(tdt))
        ncode = want_codes.size * 4
        raw_codes = torch.zeros(ncode + 256, dtype=torch.uint8, device="cuda")
        dq = raw_codes[offset_bytes: offset_bytes + ncode].view(torch.int32).view(want_codes.shape)
        ds = torch.zeros(want_scale.shape, dtype=torch.float32, device="cuda")
        raw_out = torch.zeros(n * esz + 256, dtype=torch.uint8, device="cuda")
        do = raw_out[offset_bytes: offset_bytes + n * esz].view(tdt).view(shape)
        ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
        quantize.launch_dynamic(client, H(dx), H(dq), H(ds), scheme, elem_of(F), H(ws))
        dequantize.launch_ref(client, H(dq), H(do), H(ds), scheme, elem_of(F))
        torch.cuda.synchronize()
        assert_bits_equal(to_numpy(dq.contiguous(), np.uint32), want_codes, "codes")
        assert_bits_equal(to_numpy(ds, np.float32), want_scale, "scales")
        assert_bits_equal(to_numpy(do.contiguous(), F), want_restored, "restored")
        # nothing outside the views was touched
        assert int(raw_codes[:offset_bytes].sum()) == 0 and int(raw_codes[offset_bytes + ncode:].sum()) == 0
        assert int(raw_out[:offset_bytes].sum()) == 0 and int(raw_out[offset_bytes + n * esz:].sum()) == 0


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", list(scheme_grid(SHAPE)), ids=scheme_id)
def test_bulk_copy_staged_variant(fname, scheme, tuning):
    """The quantize kernels with their input staged through shared memory by `cp.async.bulk` + mbarriers
    give the same bits, and no bounded wait gave up."""
    import ctypes

    F = FLOATS[fname]
    for mode in (1, 2):                                            # always staged, never staged
        tuning(_ffi.TUNE_STAGED, mode)
        full_check(adversarial_tensor(SHAPE, F, scheme, 5), scheme, F)
        full_check(random_tensor((1024, 1024), F, 6), scheme, F)  # several tiles per CTA, ragged last tile
    flag = ctypes.c_int(-1)
    assert _ffi.lib().qk_device_error(ctypes.byref(flag)) == 0 and flag.value == 0


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", [
    QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32])),
    QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([128])),
    QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16])),
    QuantScheme(value=QuantValue.Q8S),
    QuantScheme(value=QuantValue.Q2S, level=QuantLevel.block([64])),
])
def test_column_slices_of_wider_tensors(fname, scheme):
    """Rows contiguous, rows a constant stride apart (a column slice of a wider matrix, also with leading
    dims): the streaming kernels address such tensors row by row.  Results equal the oracle's on the dense
    copy, and the dequantize writes nothing outside the slice."""
    import torch
    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from tests._util import code_dtype, elem_of, empty_device, to_device, to_numpy

    F = FLOATS[fname]
    elem = elem_of(F)
    H = TensorHandleRef.from_torch
    client = ComputeClient.current()
    for shape, pad_left, pad_right in (((300, 1024), 64, 192), ((3, 40, 512), 16, 48), ((700, 256), 0, 32)):
        x = random_tensor(shape, F, 4321)
        wide_shape = shape[:-1] + (pad_left + shape[-1] + pad_right,)
        wide = to_device(random_tensor(wide_shape, F, 99))
        view = wide[..., pad_left:pad_left + shape[-1]]
        view.copy_(to_device(x))
        assert not view.is_contiguous()
        want_codes, want_scale = O.quantize_dynamic(x, scheme)
        dq = empty_device(scheme.packed_shape(shape), code_dtype(scheme))
        ds = empty_device(scheme.scales_shape(shape), np.float32)
        ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
        quantize.launch_dynamic(client, H(view), H(dq), H(ds), scheme, elem, H(ws))
        dscale = empty_device(scheme.scales_shape(shape), F)
        quantize.compute_scales(client, H(view), H(dscale), scheme, elem, H(ws))
        dq2 = empty_device(scheme.packed_shape(shape), code_dtype(scheme))
        ds2 = empty_device(scheme.scales_shape(shape), np.float32)
        quantize.launch_ref(client, H(view), H(dq2), H(dscale), H(ds2), scheme, elem)
        out_wide = to_device(random_tensor(wide_shape, F, 100))
        before = out_wide.clone()
        out_view = out_wide[..., pad_left:pad_left + shape[-1]]
        dequantize.launch_ref(client, H(dq), H(out_view), H(ds), scheme, elem)
        torch.cuda.synchronize()
        assert_bits_equal(to_numpy(dq, code_dtype(scheme)), want_codes, "codes")
        assert_bits_equal(to_numpy(ds, np.float32), want_scale, "scales")
        assert_bits_equal(to_numpy(dq2, code_dtype(scheme)), want_codes, "codes (two calls)")
        assert_bits_equal(to_numpy(out_view.contiguous(), F), O.dequantize(want_codes, want_scale, scheme, F), "restored")
        out_wide[..., pad_left:pad_left + shape[-1]] = before[..., pad_left:pad_left + shape[-1]]
        assert torch.equal(out_wide.view(torch.uint8), before.view(torch.uint8)), "bytes outside the slice changed"


@pytest.mark.parametrize("fname,scheme", [
    ("bf16", QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32]))),
    ("bf16", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([32]))),
    ("f16", QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16]))),
    ("f16", QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([32]))),
    ("f32", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([16]))),
    ("f32", QuantScheme(value=QuantValue.Q2S, level=QuantLevel.block([16]))),
    ("f32", QuantScheme(value=QuantValue.Q8S)),
    ("bf16", QuantScheme(value=QuantValue.Q8S)),
    ("f16", QuantScheme(value=QuantValue.E4M3, store=QuantStore.Native)),
    ("bf16", QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([64]))),     # blocks of two units
    ("bf16", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([128]))),    # four units
    ("f32", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([128]))),     # eight units
    ("f16", QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([64]), param=QuantParam.F16)),
    ("f32", QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([24]))),      # not a power of two: general kernels
])
def test_transposed_matrix_views(fname, scheme):
    """`w.t()` of a row-major matrix (also of a column slice of it, ld > rows): blocks and packed words run
    across memory rows.  Fused, two-call and dequantize results equal the oracle's on a contiguous copy, and
    the dequantize writes nothing outside the view."""
    import torch
    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from tests._util import NP_FLOAT, code_dtype, elem_of, empty_device, to_device, to_numpy

    F = FLOATS[fname]
    elem = elem_of(F)
    H = TensorHandleRef.from_torch
    client = ComputeClient.current()
    pdt = NP_FLOAT[ElemType(int(scheme.param))]
    for (rows, cols), pad in (((300, 1536), 0), ((1000, 384), 24), ((33, 384), 7)):
        x = random_tensor((rows, cols), F, 2468)
        store = to_device(random_tensor((cols, rows + pad), F, 1))       # memory: [cols, ld]
        view = store[:, :rows].t()                                      # logical [rows, cols], strides (1, ld)
        view.copy_(to_device(x))
        assert tuple(view.shape) == (rows, cols) and view.stride(0) == 1
        want_codes, want_scale = O.quantize_dynamic(x, scheme)
        dq = empty_device(scheme.packed_shape((rows, cols)), code_dtype(scheme))
        ds = empty_device(scheme.scales_shape((rows, cols)), pdt)
        ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
        quantize.launch_dynamic(client, H(view), H(dq), H(ds), scheme, elem, H(ws))
        dscale = empty_device(scheme.scales_shape((rows, cols)), F)
        quantize.compute_scales(client, H(view), H(dscale), scheme, elem, H(ws))
        dq2 = empty_device(scheme.packed_shape((rows, cols)), code_dtype(scheme))
        ds2 = empty_device(scheme.scales_shape((rows, cols)), pdt)
        quantize.launch_ref(client, H(view), H(dq2), H(dscale), H(ds2), scheme, elem)
        out_store = to_device(random_tensor((cols, rows + pad), F, 2))
        before = out_store.clone()
        out_view = out_store[:, :rows].t()
        dequantize.launch_ref(client, H(dq), H(out_view), H(ds), scheme, elem)
        torch.cuda.synchronize()
        assert_bits_equal(to_numpy(dq, code_dtype(scheme)), want_codes, "codes")
        assert_bits_equal(to_numpy(ds, pdt), want_scale, "scales")
        assert_bits_equal(to_numpy(dscale, F), O.compute_scales(x, scheme), "compute_scales")
        assert_bits_equal(to_numpy(dq2, code_dtype(scheme)), want_codes, "codes (two calls)")
        assert_bits_equal(to_numpy(ds2, pdt), want_scale, "scales (two calls)")
        assert_bits_equal(to_numpy(out_view.contiguous(), F), O.dequantize(want_codes, want_scale, scheme, F), "restored")
        out_store[:, :rows] = before[:, :rows]
        assert torch.equal(out_store.view(torch.uint8), before.view(torch.uint8)), "bytes outside the view changed"
