"""The one-launch per-tensor quantize (absmax, grid barrier, quantize in one cooperative kernel): the kernel walks
the tensor in rows of grid x 256 units, four at a time, and keeps the last rows in registers and shared memory
for its second pass.  Sizes are chosen so that the row count takes every remainder of four, the last row is
ragged, and the rows kept in shared memory are none, a few, or as many as fit; every result is compared with the
oracle bit for bit, and with the two-launch route."""
import numpy as np
import pytest

from cubek_b200 import QuantScheme, QuantStore, QuantValue
from cubek_b200 import _ffi
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import assert_bits_equal, gpu_quantize_dynamic

pytestmark = pytest.mark.gpu

TUNE_COOP, TUNE_SMEM_ROWS = 7, 12


@pytest.fixture
def knobs():
    lib = _ffi.lib()
    saved = {k: lib.qk_get_tuning(k) for k in (TUNE_COOP, TUNE_SMEM_ROWS)}
    yield lib
    for k, v in saved.items():
        lib.qk_set_tuning(k, v)


# rows of 4096 f32 (256 units each); with 296 resident CTAs a kernel row is 75776 units
@pytest.mark.parametrize("rows", [1, 100, 296, 1000, 1300, 1700, 2000, 2100, 2700, 3300, 4099])
@pytest.mark.parametrize("kept", [-1, 0, 2])
def test_f32_q8_row_counts(knobs, rows, kept):
    scheme = QuantScheme(value=QuantValue.Q8S)
    x = random_tensor((rows, 4096), np.float32, 100 + rows, "normal")
    x[rows // 2, 17] = 9.5          # the absmax sits in the middle of the walk
    want_codes, want_scale = O.quantize_dynamic(x, scheme)
    knobs.qk_set_tuning(TUNE_SMEM_ROWS, kept)
    codes, scale = gpu_quantize_dynamic(x, scheme)
    assert_bits_equal(scale, want_scale, "scale")
    assert_bits_equal(codes, want_codes, "codes")


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("value,store", [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q8F, QuantStore.Native),
                                         (QuantValue.Q4S, QuantStore.U32), (QuantValue.Q2S, QuantStore.U32),
                                         (QuantValue.E2M1, QuantStore.Native), (QuantValue.E4M3, QuantStore.Native),
                                         (QuantValue.E5M2, QuantStore.Native)])
def test_every_kind_matches_the_oracle_and_the_two_launch_route(knobs, fname, value, store):
    F = FLOATS[fname]
    scheme = QuantScheme(value=value, store=store)
    x = random_tensor((3001, 2048), F, 7, "outliers")
    want_codes, want_scale = O.quantize_dynamic(x, scheme)
    codes, scale = gpu_quantize_dynamic(x, scheme)
    assert_bits_equal(scale, want_scale, "scale (one launch)")
    assert_bits_equal(codes, want_codes, "codes (one launch)")
    knobs.qk_set_tuning(TUNE_COOP, 0)
    codes2, scale2 = gpu_quantize_dynamic(x, scheme)
    assert_bits_equal(scale2, scale, "scale (two launches)")
    assert_bits_equal(codes2, codes, "codes (two launches)")


def test_all_zero_and_single_unit_tensors(knobs):
    scheme = QuantScheme(value=QuantValue.Q8S)
    for shape in [(1, 16), (3, 16), (700, 4096)]:
        x = np.zeros(shape, dtype=np.float32)
        want_codes, want_scale = O.quantize_dynamic(x, scheme)
        codes, scale = gpu_quantize_dynamic(x, scheme)
        assert_bits_equal(scale, want_scale, "scale")
        assert_bits_equal(codes, want_codes, "codes")
