"""`qk_roundtrip_host`: host buffers in, host buffers out, against the oracle."""
import numpy as np
import pytest
import torch

from cubek_b200 import ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef
from cubek_b200 import _ffi
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import assert_bits_equal, code_dtype, elem_of

pytestmark = pytest.mark.gpu


def roundtrip(x: np.ndarray, scheme: QuantScheme):
    lib = _ffi.lib()
    elem = elem_of(x.dtype)
    codes = np.zeros(scheme.packed_shape(x.shape), dtype=code_dtype(scheme))
    scales = np.zeros(scheme.scales_shape(x.shape), dtype=np.float32)
    restored = np.zeros_like(x)

    def handle(a):
        return _ffi.CTensor(TensorHandleRef.from_raw_parts(a.ctypes.data, a.shape, a.itemsize))

    ci, cc, cs, co = handle(x), handle(codes), handle(scales), handle(restored)
    sch = _ffi.c_scheme(scheme)
    need = lib.qk_host_roundtrip_staging_bytes(ci.ref(), sch, int(elem))
    staging = torch.empty(int(need), dtype=torch.uint8, device="cuda")
    _ffi.check(lib.qk_roundtrip_host(ci.ref(), cc.ref(), cs.ref(), co.ref(), sch, int(elem), staging.data_ptr(),
                                     int(need), torch.cuda.current_device()))
    return codes, scales, restored


@pytest.mark.parametrize("fname,scheme,shape", [
    ("bf16", QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32])), (20000, 4096)),   # several slices
    ("f32", QuantScheme(value=QuantValue.Q8S), (1000, 512)),                                     # per tensor, one slice
    ("f16", QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16])), (513, 1024)),
    ("f32", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([2, 16])), (64, 96)),       # N-d blocks, one slice
])
def test_host_roundtrip_matches_oracle(fname, scheme, shape):
    F = FLOATS[fname]
    x = random_tensor(shape, F, 21)
    codes, scales, restored = roundtrip(x, scheme)
    o_codes, o_scales = O.quantize_dynamic(x, scheme)
    assert_bits_equal(codes, o_codes, "codes")
    assert_bits_equal(scales, o_scales, "scales")
    assert_bits_equal(restored, O.dequantize(o_codes, o_scales, scheme, F), "restored")


def test_staging_too_small_is_rejected():
    lib = _ffi.lib()
    x = np.zeros((64, 64), dtype=np.float32)
    scheme = QuantScheme(value=QuantValue.Q8S)
    t = _ffi.CTensor(TensorHandleRef.from_raw_parts(x.ctypes.data, x.shape, 4))
    c = _ffi.CTensor(TensorHandleRef.from_raw_parts(x.ctypes.data, (64, 16), 4))
    s = _ffi.CTensor(TensorHandleRef.from_raw_parts(x.ctypes.data, (1,), 4))
    staging = torch.empty(256, dtype=torch.uint8, device="cuda")
    rc = lib.qk_roundtrip_host(t.ref(), c.ref(), s.ref(), t.ref(), _ffi.c_scheme(scheme), 0, staging.data_ptr(), 256, 0)
    assert rc == _ffi.QK_ERR_WORKSPACE


@pytest.mark.parametrize("fname,scheme", [
    ("bf16", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([128]))),
    ("f32", QuantScheme(value=QuantValue.Q8S)),                                      # per tensor: every tensor one slice
])
def test_host_roundtrip_batch_matches_oracle(fname, scheme):
    """Tensors of several sizes (several slices, one slice, a single row) through one ring of staging slots."""
    lib = _ffi.lib()
    F = FLOATS[fname]
    elem = elem_of(F)
    shapes = [(9000, 4096), (64, 4096), (1, 128), (3000, 1024), (5, 256)]
    xs = [random_tensor(sh, F, 30 + i) for i, sh in enumerate(shapes)]
    codes = [np.zeros(scheme.packed_shape(x.shape), dtype=code_dtype(scheme)) for x in xs]
    scales = [np.zeros(scheme.scales_shape(x.shape), dtype=np.float32) for x in xs]
    restored = [np.zeros_like(x) for x in xs]

    def handles(arrays):
        return _ffi.CTensorArray([TensorHandleRef.from_raw_parts(a.ctypes.data, a.shape, a.itemsize) for a in arrays])

    hi, hc, hs, ho = handles(xs), handles(codes), handles(scales), handles(restored)
    sch = _ffi.c_scheme(scheme)
    need = int(lib.qk_host_roundtrip_staging_bytes_batch(hi.count, hi.array, sch, int(elem)))
    assert need > 0
    staging = torch.empty(need, dtype=torch.uint8, device="cuda")
    _ffi.check(lib.qk_roundtrip_host_batch(hi.count, hi.array, hc.array, hs.array, ho.array, sch, int(elem),
                                           staging.data_ptr(), need, torch.cuda.current_device()))
    for i, x in enumerate(xs):
        o_codes, o_scales = O.quantize_dynamic(x, scheme)
        assert_bits_equal(codes[i], o_codes, f"codes {i}")
        assert_bits_equal(scales[i], o_scales, f"scales {i}")
        assert_bits_equal(restored[i], O.dequantize(o_codes, o_scales, scheme, F), f"restored {i}")
    # too little staging for the largest member
    assert lib.qk_roundtrip_host_batch(hi.count, hi.array, hc.array, hs.array, ho.array, sch, int(elem),
                                       staging.data_ptr(), 1024, torch.cuda.current_device()) == _ffi.QK_ERR_WORKSPACE
