"""`qk_reduce` (MaxAbs, Max, Min) against NumPy.  Every result is one of the inputs, so the comparison is bit for
bit; all strategies (a thread, a warp or a CTA per output item, or the library's choice) must agree."""
import numpy as np
import pytest
import torch

from cubek_b200 import ComputeClient, QuantPanic, TensorHandleRef
from cubek_b200.reduce import ReduceInst, ReduceStrategy, reduce, reduce_maxabs
from tests._cases import FLOATS, random_tensor
from tests._util import assert_bits_equal, elem_of, empty_device, to_device, to_numpy

H = TensorHandleRef.from_torch
STRATEGIES = [None, ReduceStrategy(False, False), ReduceStrategy(True, False), ReduceStrategy(True, True)]
SHAPES = [((64, 4096), 1), ((64, 4096), 0), ((7, 33), 1), ((7, 33), 0), ((5, 6, 40), 1), ((5, 6, 40), 2), ((3, 1, 8), 1),
          ((1000, 16), 1), ((2, 300, 64), 1), ((513, 8192), 1), ((4, 70, 4096), 1), ((9, 3, 5), 0)]


def numpy_reduce(x, axis, inst):
    f = x.astype(np.float32)
    if inst == ReduceInst.MaxAbs:
        return np.abs(f).max(axis=axis, keepdims=True).astype(x.dtype)
    if inst == ReduceInst.Max:
        return f.max(axis=axis, keepdims=True).astype(x.dtype)
    return f.min(axis=axis, keepdims=True).astype(x.dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("inst", list(ReduceInst))
@pytest.mark.parametrize("shape,axis", SHAPES)
def test_reduce_matches_numpy_under_every_strategy(fname, inst, shape, axis):
    F = FLOATS[fname]
    x = random_tensor(shape, F, 61)
    want = numpy_reduce(x, axis, inst)
    dx = to_device(x)
    for strategy in STRATEGIES:
        do = empty_device(want.shape, F)
        reduce(ComputeClient.current(), H(dx), H(do), axis, strategy, inst, elem_of(F))
        torch.cuda.synchronize()
        assert_bits_equal(to_numpy(do, F), want, f"{inst.name} with {strategy}")


@pytest.mark.gpu
@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("inst", list(ReduceInst))
def test_reduce_strided_views(fname, inst):
    """A transposed matrix, a column slice of a wider one and a strided output take the per-item kernel."""
    F = FLOATS[fname]
    x = random_tensor((48, 200), F, 62)
    base = to_device(x)
    for view, ref in ((base.t(), x.T), (base[:, 8:136], x[:, 8:136]), (base[::3, :], x[::3, :])):
        for axis in (0, 1):
            want = numpy_reduce(np.ascontiguousarray(ref), axis, inst)
            do = empty_device(want.shape, F)
            reduce(ComputeClient.current(), H(view), H(do), axis, None, inst, elem_of(F))
            torch.cuda.synchronize()
            assert_bits_equal(to_numpy(do, F), want, f"{inst.name} axis {axis}")
    # strided output: every second element of a wider buffer
    want = numpy_reduce(x, 1, inst)
    wide = empty_device((48, 2), F)
    reduce(ComputeClient.current(), H(base), H(wide[:, 1:2]), 1, None, inst, elem_of(F))
    torch.cuda.synchronize()
    assert_bits_equal(to_numpy(wide[:, 1:2].contiguous(), F), want, "strided output")


@pytest.mark.gpu
def test_null_accumulators_and_nan_elements():
    """Max / Min start from the lowest / highest FINITE value of the type (the reference's `min_value()` /
    `max_value()`), so a row of -inf gives that value under Max; NaN elements do not take part."""
    x = np.full((4, 64), -np.inf, dtype=np.float32)
    x[1, 5] = 3.0
    x[2, :] = np.nan
    x[3, 7] = np.nan
    x[3, 9] = -2.0
    dx = to_device(x)
    for strategy in STRATEGIES:
        do = empty_device((4, 1), np.float32)
        reduce(ComputeClient.current(), H(dx), H(do), 1, strategy, ReduceInst.Max, elem_of(np.float32))
        torch.cuda.synchronize()
        got = to_numpy(do, np.float32).reshape(-1)
        lowest = np.finfo(np.float32).min
        assert got.tolist() == [lowest, 3.0, lowest, -2.0]
    half = np.full((2, 16), np.inf, dtype=np.float16)
    do = empty_device((2, 1), np.float16)
    dhalf = to_device(half)
    reduce(ComputeClient.current(), H(dhalf), H(do), 1, None, ReduceInst.Min, elem_of(np.float16))
    torch.cuda.synchronize()
    assert to_numpy(do, np.float16).reshape(-1).tolist() == [65504.0, 65504.0]


@pytest.mark.gpu
def test_maxabs_shortcut():
    x = random_tensor((33, 777), np.float32, 63)
    do = empty_device((33, 1), np.float32)
    dx = to_device(x)
    reduce_maxabs(ComputeClient.current(), H(dx), H(do), 1, elem_of(np.float32))
    torch.cuda.synchronize()
    assert_bits_equal(to_numpy(do, np.float32), numpy_reduce(x, 1, ReduceInst.MaxAbs), "maxabs")


def test_reduce_rejects_bad_axis_shape_and_instruction():
    client = ComputeClient(0, 0)
    t = TensorHandleRef.from_raw_parts(0x10000, (4, 8), 4)
    with pytest.raises(QuantPanic):      # InvalidAxis
        reduce_maxabs(client, t, TensorHandleRef.from_raw_parts(0x20000, (4, 1), 4), 2, 0)
    with pytest.raises(QuantPanic):      # MismatchShape
        reduce_maxabs(client, t, TensorHandleRef.from_raw_parts(0x20000, (4, 8), 4), 1, 0)
    with pytest.raises(QuantPanic):      # an instruction outside MaxAbs / Max / Min
        reduce(client, t, TensorHandleRef.from_raw_parts(0x20000, (4, 1), 4), 1, None, 7, 0)
