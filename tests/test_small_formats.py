"""The oracle's fp4 / fp8 tables against ml_dtypes (an independent implementation)."""
import ml_dtypes
import numpy as np

from oracle import oracle as O


def test_e2m1_decode_all_codes():
    codes = np.arange(16, dtype=np.uint8)
    want = codes.view(ml_dtypes.float4_e2m1fn).astype(np.float32)
    got = np.array([O.lib().oq_e2m1_to_f32(int(c)) for c in codes], dtype=np.float32)
    assert got.tobytes() == want.tobytes()


def test_e2m1_encode_matches_ml_dtypes_on_a_dense_grid():
    grid = np.concatenate([np.arange(-8, 8, 1 / 64, dtype=np.float32),
                           np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 100.0], dtype=np.float32)])
    want = grid.astype(ml_dtypes.float4_e2m1fn).view(np.uint8) & 0xF
    got = np.array([O.lib().oq_f32_to_e2m1(float(v)) for v in grid], dtype=np.uint8)
    # -0.0 / +0.0: both encode a zero magnitude; compare magnitudes and signs of non-zeros
    nz = (want & 7) != 0
    assert np.array_equal(got[nz], want[nz])
    assert np.all((got[~nz] & 7) == 0)


def test_integers_through_e2m1_show_the_five_to_four_rounding():
    # the reference rounds to an integer before the fp4 cast (quantize.rs:19-43), so 5 -> 4
    vals = {v: O.lib().oq_e2m1_to_f32(O.lib().oq_f32_to_e2m1(float(v))) for v in range(-6, 7)}
    assert vals[5] == 4.0 and vals[-5] == -4.0
    for v in (-6, -4, -3, -2, -1, 0, 1, 2, 3, 4, 6):
        assert vals[v] == float(v)


def test_fp8_tables():
    codes = np.arange(256, dtype=np.uint8)
    for name, dt in (("e4m3", ml_dtypes.float8_e4m3fn), ("e5m2", ml_dtypes.float8_e5m2)):
        want = codes.view(dt).astype(np.float32)
        got = np.array([getattr(O.lib(), f"oq_{name}_to_f32")(int(c)) for c in codes], dtype=np.float32)
        finite = np.isfinite(want)
        assert got[finite].tobytes() == want[finite].tobytes()
        ints = np.arange(-448, 449, dtype=np.float32)
        enc = np.array([getattr(O.lib(), f"oq_f32_to_{name}")(float(v)) for v in ints], dtype=np.uint8)
        assert np.array_equal(enc.view(dt).astype(np.float32), ints.astype(dt).astype(np.float32))
