"""`qk_reduce_maxabs` against NumPy (the result is exact: it is the magnitude of one input)."""
import numpy as np
import pytest
import torch

from cubek_b200 import ComputeClient, LaunchError, QuantPanic, TensorHandleRef
from cubek_b200.reduce import reduce_maxabs
from tests._cases import FLOATS, random_tensor
from tests._util import assert_bits_equal, elem_of, empty_device, to_device, to_numpy

H = TensorHandleRef.from_torch


@pytest.mark.gpu
@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("shape,axis", [((64, 4096), 1), ((64, 4096), 0), ((7, 33), 1), ((7, 33), 0),
                                        ((5, 6, 40), 1), ((5, 6, 40), 2), ((3, 1, 8), 1), ((1000, 16), 1)])
def test_maxabs_matches_numpy(fname, shape, axis):
    F = FLOATS[fname]
    x = random_tensor(shape, F, 61)
    want = np.abs(x.astype(np.float32)).max(axis=axis, keepdims=True).astype(F)
    dx = to_device(x)
    do = empty_device(want.shape, F)
    reduce_maxabs(ComputeClient.current(), H(dx), H(do), axis, elem_of(F))
    torch.cuda.synchronize()
    assert_bits_equal(to_numpy(do, F), want, "maxabs")


def test_maxabs_rejects_bad_axis_and_shape():
    client = ComputeClient(0, 0)
    t = TensorHandleRef.from_raw_parts(0x10000, (4, 8), 4)
    with pytest.raises(QuantPanic):
        reduce_maxabs(client, t, TensorHandleRef.from_raw_parts(0x20000, (4, 1), 4), 2, 0)
    with pytest.raises(QuantPanic):
        reduce_maxabs(client, t, TensorHandleRef.from_raw_parts(0x20000, (4, 8), 4), 1, 0)
