"""The batch entry points give, tensor for tensor, the bits of the single-tensor entry points:
mixed shapes in one call, more tensors than one launch holds, per-block and per-tensor schemes,
and members that fall back to the layout-general kernels in the middle of a batch."""
import numpy as np
import pytest
import torch

from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef,
                        dequantize, quantize)
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import NP_FLOAT, assert_bits_equal, code_dtype, empty_device, to_device, to_numpy

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch


def run_batch(xs, scheme, F, ws_bytes=1 << 20):
    elem = {np.dtype(np.float32): ElemType.F32, np.dtype(np.float16): ElemType.F16}.get(np.dtype(F), ElemType.BF16)
    client = ComputeClient.current()
    dx = [to_device(x) for x in xs]
    dq = [empty_device(scheme.packed_shape(x.shape), code_dtype(scheme)) for x in xs]
    ds = [empty_device(scheme.scales_shape(x.shape), np.float32) for x in xs]
    do = [empty_device(x.shape, F) for x in xs]
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic_batch(client, [H(t) for t in dx], [H(t) for t in dq], [H(t) for t in ds], scheme, elem, H(ws))
    dequantize.launch_batch(client, [H(t) for t in dq], [H(t) for t in do], [H(t) for t in ds], scheme, elem)
    torch.cuda.synchronize()
    return ([to_numpy(t, code_dtype(scheme)) for t in dq], [to_numpy(t, np.float32) for t in ds],
            [to_numpy(t, F) for t in do])


@pytest.mark.parametrize("fname,scheme", [
    ("bf16", QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32]))),
    ("bf16", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([128]))),
    ("f32", QuantScheme(value=QuantValue.Q2S, level=QuantLevel.block([64]))),
    ("f16", QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16]))),
    ("bf16", QuantScheme(value=QuantValue.Q8S)),                      # per tensor: one absmax cell each
    ("f32", QuantScheme(value=QuantValue.Q8F)),
])
def test_batch_equals_single_tensor_calls(fname, scheme):
    F = FLOATS[fname]
    shapes = [(64, 256), (8, 128), (300, 512), (1, 128), (128, 1024), (16, 256)]
    xs = [random_tensor(s, F, 50 + i) * np.float32(1 + i).astype(F) for i, s in enumerate(shapes)]
    codes, scales, restored = run_batch(xs, scheme, F)
    for x, c, s, r in zip(xs, codes, scales, restored):
        oc, os_ = O.quantize_dynamic(x, scheme)
        assert_bits_equal(c, oc, "codes")
        assert_bits_equal(s, os_, "scales")
        assert_bits_equal(r, O.dequantize(oc, os_, scheme, F), "restored")


@pytest.mark.parametrize("fname", ["f32", "bf16"])
def test_per_tensor_batch_with_minimal_workspace(fname):
    """With only the absmax cells as workspace the per-tensor batch takes one batched absmax launch and
    batched quantize launches (no cooperative kernels); ragged members get their own absmax launch."""
    F = FLOATS[fname]
    scheme = QuantScheme(value=QuantValue.Q8S)
    shapes = [(64, 256), (3, 36), (300, 512), (1, 128), (128, 1024), (5, 4), (16, 256)] + [(8, 64)] * 140
    xs = [random_tensor(s, F, 500 + i) * np.float32(1 + i % 7).astype(F) for i, s in enumerate(shapes)]
    codes, scales, restored = run_batch(xs, scheme, F, ws_bytes=1024)
    for x, c, s, r in zip(xs, codes, scales, restored):
        oc, os_ = O.quantize_dynamic(x, scheme)
        assert_bits_equal(c, oc, "codes")
        assert_bits_equal(s, os_, "scales")
        assert_bits_equal(r, O.dequantize(oc, os_, scheme, F), "restored")


def test_more_tensors_than_one_launch_and_general_members():
    F = FLOATS["bf16"]
    scheme = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32]))
    shapes = [(4, 64)] * 70 + [(3, 96)] + [(4, 64)] * 5        # 96 = 3 blocks of 32: still streaming; 76 tensors > 64
    xs = [random_tensor(s, F, 200 + i) for i, s in enumerate(shapes)]
    codes, scales, restored = run_batch(xs, scheme, F)
    for x, c, s, r in zip(xs, codes, scales, restored):
        oc, os_ = O.quantize_dynamic(x, scheme)
        assert_bits_equal(c, oc, "codes")
        assert_bits_equal(s, os_, "scales")
        assert_bits_equal(r, O.dequantize(oc, os_, scheme, F), "restored")
    # a block size that is not a power of two sends one member through the general kernels
    scheme = QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([24]))
    xs = [random_tensor((8, 96), np.float32, 300 + i) for i in range(3)]
    codes, scales, restored = run_batch(xs, scheme, np.float32)
    for x, c, s in zip(xs, codes, scales):
        oc, os_ = O.quantize_dynamic(x, scheme)
        assert_bits_equal(c, oc, "codes")
        assert_bits_equal(s, os_, "scales")


def test_per_tensor_batch_with_strided_members():
    """Float tensors of a per-tensor batch may be strided views (a transposed matrix, every other column):
    their absmax comes from the strided kernel, their codes from the layout-general one."""
    scheme = QuantScheme(value=QuantValue.Q8S)
    client = ComputeClient.current()
    base = [torch.from_numpy(random_tensor((64, 128), np.float32, 900 + i)).cuda() for i in range(4)]
    views = [base[0], base[1].t(), base[2][:, ::2], base[3]]
    dq = [empty_device(scheme.packed_shape(tuple(v.shape)), code_dtype(scheme)) for v in views]
    ds = [empty_device((1,), np.float32) for _ in views]
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic_batch(client, [H(v) for v in views], [H(t) for t in dq], [H(t) for t in ds], scheme,
                                  ElemType.F32, H(ws))
    torch.cuda.synchronize()
    for v, c, s in zip(views, dq, ds):
        oc, os_ = O.quantize_dynamic(np.ascontiguousarray(v.cpu().numpy()), scheme)
        assert_bits_equal(to_numpy(c, code_dtype(scheme)), oc, "codes")
        assert_bits_equal(to_numpy(s, np.float32), os_, "scales")


@pytest.mark.parametrize("mode,stages", [(1, 2), (1, 3), (1, 4), (2, 2)])
def test_batches_through_staged_and_direct_kernels(mode, stages):
    """Tiles of the staged kernels never span two tensors of a batch; ragged tensors end in partial tiles."""
    import ctypes
    from cubek_b200 import _ffi

    _ffi.lib().qk_set_tuning(_ffi.TUNE_STAGED, mode)
    _ffi.lib().qk_set_tuning(_ffi.TUNE_STAGES, stages)
    try:
        F = FLOATS["f16"]
        scheme = QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16]))
        shapes = [(33, 272), (700, 512), (1, 16), (129, 1040), (64, 4096)]
        xs = [random_tensor(s, F, 400 + i) for i, s in enumerate(shapes)]
        codes, scales, restored = run_batch(xs, scheme, F)
        for x, c, s in zip(xs, codes, scales):
            oc, os_ = O.quantize_dynamic(x, scheme)
            assert_bits_equal(c, oc, "codes")
            assert_bits_equal(s, os_, "scales")
        flag = ctypes.c_int(-1)
        assert _ffi.lib().qk_device_error(ctypes.byref(flag)) == 0 and flag.value == 0
    finally:
        _ffi.lib().qk_set_tuning(_ffi.TUNE_STAGED, 0)
        _ffi.lib().qk_set_tuning(_ffi.TUNE_STAGES, 2)


def test_empty_batch_and_length_mismatch():
    client = ComputeClient.current()
    scheme = QuantScheme(value=QuantValue.Q8S)
    quantize.launch_dynamic_batch(client, [], [], [], scheme, ElemType.F32, None)
    with pytest.raises(ValueError):
        quantize.PreparedDynamicBatch(client, [], [H(torch.zeros(4, device="cuda"))], [], scheme, ElemType.F32)
