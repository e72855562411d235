"""`qk_quantize_dynamic_noalloc`, the entry point for callers that cannot allocate device memory
(its scratch is a fixed array inside the library instead of a caller-provided workspace).

Checked through the C ABI against `qk_quantize_dynamic` and against the CPU oracle on the same inputs: the
bits must be identical, on two calls in a row with different data (the second call finds the first call's
leftovers in the shared array and must not be affected by them).  Collected last on purpose, so a
run that stops at the first failure has already exercised everything else.
"""
import numpy as np
import pytest

from cubek_b200 import ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef
from cubek_b200 import _ffi
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import NP_FLOAT, assert_bits_equal, code_dtype, elem_of, empty_device, to_device, to_numpy, workspace

pytestmark = pytest.mark.gpu


def run(x: np.ndarray, scheme: QuantScheme, noalloc: bool):
    import torch

    lib = _ffi.lib()
    elem = elem_of(x.dtype)
    dx = to_device(x)
    dq = empty_device(scheme.packed_shape(x.shape), code_dtype(scheme))
    pdt = NP_FLOAT[ElemType(int(scheme.param))]
    ds = empty_device(scheme.scales_shape(x.shape), pdt)
    ti, tq, ts = _ffi.c_tensors(*(TensorHandleRef.from_torch(t) for t in (dx, dq, ds)))
    sch = _ffi.c_scheme(scheme)
    stream = torch.cuda.current_stream().cuda_stream
    if noalloc:
        status = lib.qk_quantize_dynamic_noalloc(ti.ref(), tq.ref(), ts.ref(), sch, int(elem), stream)
    else:
        need = int(lib.qk_workspace_bytes_for(ti.ref(), sch, int(elem)))
        ws = workspace(need)
        status = lib.qk_quantize_dynamic(ti.ref(), tq.ref(), ts.ref(), sch, int(elem), ws.data_ptr(), need, stream)
    torch.cuda.synchronize()
    return status, to_numpy(dq, code_dtype(scheme)), to_numpy(ds, pdt)


CASES = [
    # per tensor: every CTA max-reduces into the scratch cell
    ("f32", QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32), (512, 1024)),
    ("bf16", QuantScheme(value=QuantValue.Q4S, store=QuantStore.U32), (256, 2048)),
    # general layout: the scales of the N-d blocks are staged in the scratch array
    ("f16", QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32, level=QuantLevel.block([2, 16])), (64, 96)),
    # streaming per-block layout: no scratch needed, must still work
    ("bf16", QuantScheme(value=QuantValue.Q4S, store=QuantStore.U32, level=QuantLevel.block([32])), (128, 1024)),
]


@pytest.mark.parametrize("fname,scheme,shape", CASES)
def test_noalloc_matches_workspace_entry_point_twice_in_a_row(fname, scheme, shape):
    F = FLOATS[fname]
    first = random_tensor(shape, F, 31, "normal")
    second = (random_tensor(shape, F, 32, "uniform").astype(np.float32) * 0.01).astype(F)   # much smaller absmax
    for x in (first, second):
        want_status, want_codes, want_scale = run(x, scheme, noalloc=False)
        status, codes, scale = run(x, scheme, noalloc=True)
        assert want_status == 0 and status == 0, _ffi.strerror(status)
        assert_bits_equal(codes, want_codes, "codes")
        assert_bits_equal(scale, want_scale, "out_scale")
        # and against the CPU oracle, so that the check does not rest on another CUDA path alone
        o_codes, o_scale = O.quantize_dynamic(x, scheme)
        assert_bits_equal(codes, o_codes, "codes vs oracle")
        assert_bits_equal(scale, o_scale, "out_scale vs oracle")


def test_noalloc_rejects_layouts_whose_staged_scales_do_not_fit():
    lib = _ffi.lib()
    limit = int(lib.qk_noalloc_scratch_bytes())
    assert limit == 64 * 1024
    # 3-wide blocks take the general kernels: 1024 x 96 f32 -> 32768 scales x 4 bytes > 64 KiB
    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.Native, level=QuantLevel.block([3]))
    x = random_tensor((1024, 96), np.float32, 33)
    status, _, _ = run(x, scheme, noalloc=True)
    assert status == _ffi.QK_ERR_TOO_LARGE
    assert "size" in _ffi.strerror(status)
    # the same layout with few enough blocks is accepted and matches
    x = random_tensor((128, 96), np.float32, 34)
    want = run(x, scheme, noalloc=False)
    got = run(x, scheme, noalloc=True)
    assert got[0] == 0 and want[0] == 0
    assert_bits_equal(got[1], want[1], "codes")
    assert_bits_equal(got[2], want[2], "out_scale")
