"""The public device header (include/cubek_quant_b200_device.cuh) gives, from inside a caller's kernel,
the bits `qk_dequantize` writes: a probe kernel built on the header alone dequantizes lines of stored
items with `dequantize_symmetric_packed_values` and is compared with the library and the oracle."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest
import torch

from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue,
                        TensorHandleRef, _ffi, dequantize, quantize)
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import NP_FLOAT, assert_bits_equal, code_dtype, elem_of, empty_device, to_device, to_numpy

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch
PROBE = Path(__file__).resolve().parent / "device_api" / "libdevice_api_probe.so"


@pytest.fixture(scope="module")
def probe():
    if not PROBE.exists():
        pytest.fail(f"{PROBE} is missing: tests/device_api/build_probe.py builds it")
    lib = C.CDLL(str(PROBE))
    lib.probe_dequantize.restype = C.c_int
    lib.probe_dequantize.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.POINTER(_ffi.QkScheme),
                                     C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_void_p]
    return lib


U32, NAT = QuantStore.U32, QuantStore.Native
CASES = [
    # float, param, value, store, level, shape, line
    ("f32", QuantParam.F32, QuantValue.Q8S, U32, QuantLevel.Tensor, (32, 64), 4),
    ("f32", QuantParam.F32, QuantValue.Q8F, U32, QuantLevel.block([32]), (16, 128), 1),
    ("bf16", QuantParam.F32, QuantValue.Q4S, U32, QuantLevel.block([32]), (64, 256), 4),
    ("bf16", QuantParam.F32, QuantValue.Q4F, U32, QuantLevel.block([16]), (8, 64), 1),
    ("f16", QuantParam.F32, QuantValue.Q2S, U32, QuantLevel.block([64]), (8, 256), 4),
    ("f32", QuantParam.F32, QuantValue.Q2F, U32, QuantLevel.block([16]), (4, 64), 1),
    ("f16", QuantParam.F16, QuantValue.Q8S, U32, QuantLevel.block([32]), (16, 128), 4),
    ("bf16", QuantParam.BF16, QuantValue.Q4S, U32, QuantLevel.block([32]), (16, 128), 1),
    ("f32", QuantParam.BF16, QuantValue.Q8S, U32, QuantLevel.Tensor, (8, 64), 1),
    ("f32", QuantParam.F32, QuantValue.Q8S, U32, QuantLevel.block([2, 8]), (6, 32), 1),       # N-d blocks
    ("f32", QuantParam.F32, QuantValue.Q4S, U32, QuantLevel.block([2, 2, 16]), (4, 6, 32), 4),
    ("f16", QuantParam.F32, QuantValue.E2M1, NAT, QuantLevel.block([16]), (32, 128), 4),
    ("bf16", QuantParam.F32, QuantValue.E2M1, NAT, QuantLevel.block([32]), (8, 64), 1),
    ("f32", QuantParam.F32, QuantValue.E4M3, NAT, QuantLevel.block([32]), (8, 64), 4),
    ("f16", QuantParam.F32, QuantValue.E5M2, NAT, QuantLevel.Tensor, (8, 64), 1),
    ("bf16", QuantParam.F32, QuantValue.Q8S, NAT, QuantLevel.block([32]), (8, 64), 4),
]


@pytest.mark.parametrize("fname,param,value,store,level,shape,line", CASES)
def test_device_header_matches_library_and_oracle(probe, fname, param, value, store, level, shape, line):
    F = FLOATS[fname]
    elem = elem_of(F)
    scheme = QuantScheme(value=value, param=param, store=store, level=level)
    x = random_tensor(shape, F, 4242)
    client = ComputeClient.current()
    dx = to_device(x)
    codes = empty_device(scheme.packed_shape(shape), code_dtype(scheme))
    pdt = NP_FLOAT[ElemType(int(param))]
    scales = empty_device(scheme.scales_shape(shape), pdt)
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic(client, H(dx), H(codes), H(scales), scheme, elem, H(ws))
    want = empty_device(shape, F)
    dequantize.launch_ref(client, H(codes), H(want), H(scales), scheme, elem)

    got = empty_device(shape, F)
    nitems = codes.numel()
    assert nitems % line == 0
    sch = _ffi.c_scheme(scheme)
    rank = len(shape)
    vshape = (C.c_int64 * rank)(*codes.shape)
    sstrides = (C.c_int64 * rank)(*(scales.stride() if not level.is_tensor else [0] * rank))
    rc = probe.probe_dequantize(codes.data_ptr(), scales.data_ptr(), got.data_ptr(), nitems // line, line, C.byref(sch),
                                int(elem), rank, vshape, sstrides, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert_bits_equal(to_numpy(got, F), to_numpy(want, F), "device header vs qk_dequantize")
    oc, os_ = O.quantize_dynamic(x, scheme)
    assert_bits_equal(to_numpy(got, F), O.dequantize(oc, os_, scheme, F), "device header vs oracle")
