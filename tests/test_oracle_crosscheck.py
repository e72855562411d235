"""The C oracle against the independent NumPy / ml_dtypes restatement, bit for bit, on small
random and adversarial inputs (exact .5 ties, +-absmax, zeros, all-zero blocks)."""
import numpy as np
import pytest

from cubek_b200 import QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue
from oracle import numpy_restatement as R
from oracle import oracle as O
from tests._cases import FLOATS, adversarial_tensor, all_value_stores, random_tensor, scheme_id

LEVELS = [QuantLevel.Tensor, QuantLevel.block([16]), QuantLevel.block([2, 16]), QuantLevel.block([3, 32])]


def _schemes():
    for value, store in all_value_stores():
        for level in LEVELS:
            for param in (QuantParam.F32, QuantParam.BF16, QuantParam.F16):
                yield QuantScheme(value=value, store=store, level=level, param=param)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", list(_schemes()), ids=scheme_id)
def test_oracle_equals_numpy_restatement(fname, scheme):
    F = FLOATS[fname]
    shape = (6, 32)
    for seed, x in enumerate([random_tensor(shape, F, 11), adversarial_tensor(shape, F, scheme, 12)]):
        s = O.compute_scales(x, scheme)
        assert s.tobytes() == R.compute_scales(x, scheme).tobytes()
        q, os_ = O.quantize(x, s, scheme)
        q2, os2 = R.quantize(x, s, scheme)
        assert q.tobytes() == q2.tobytes() and os_.tobytes() == os2.tobytes()
        d = O.dequantize(q, os_, scheme, F)
        assert d.tobytes() == R.dequantize(q2, os2, scheme, F).tobytes()


def test_pack_order_and_twos_complement():
    # element 0 in the least significant bits; negative codes masked to the field width
    # (crates/cubek-quant/src/quantize.rs:61-81)
    scheme = QuantScheme(value=QuantValue.Q4F, store=QuantStore.U32)
    x = np.array([[-8, -1, 0, 1, 2, 3, 7, -3]], dtype=np.float32)
    q, _ = O.quantize(x, np.array([1.0], dtype=np.float32), scheme)
    assert q.shape == (1, 1)
    assert int(q[0, 0]) == 0xD73210F8
    d = O.dequantize(q, np.array([1.0], dtype=np.float32), scheme, np.float32)
    assert np.array_equal(d, x)


def test_round_half_to_even_and_clamp():
    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32)
    x = np.array([[0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 1000.0, -1000.0]], dtype=np.float32)
    q, _ = O.quantize(x, np.array([1.0], dtype=np.float32), scheme)
    codes = q.view(np.int8).reshape(-1)
    assert codes.tolist() == [0, 2, 2, 0, -2, -2, 127, -127]


def test_zero_scale_block_gives_zero_codes():
    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32, level=QuantLevel.block([4]))
    x = np.array([[0, 0, 0, 0, 1, -2, 3, -4]], dtype=np.float32)
    s = O.compute_scales(x, scheme)
    assert s[0, 0] == 0.0
    q, os_ = O.quantize(x, s, scheme)
    assert int(q[0, 0]) == 0
    d = O.dequantize(q, os_, scheme, np.float32)
    assert np.all(d[0, :4] == 0)


def test_half_type_quotient_is_rounded_before_round():
    # bf16: 2.4921875 rounds to 2.5 in bf16 (8 significant bits), and 2.5 rounds to 2 (half even);
    # in f32 the same quotient rounds to 2 as well, but 3.4921875 -> bf16 3.5 -> 4 whereas f32 -> 3.
    import ml_dtypes

    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32)
    one = np.array([1.0], dtype=ml_dtypes.bfloat16)
    x32 = np.array([[3.4921875, 0, 0, 0]], dtype=np.float32)
    q32, _ = O.quantize(x32, np.array([1.0], dtype=np.float32), scheme)
    assert q32.view(np.int8)[0, 0] == 3
    # the bf16 input itself already rounds to 3.5
    xb = x32.astype(ml_dtypes.bfloat16)
    qb, _ = O.quantize(xb, one, scheme)
    assert qb.view(np.int8)[0, 0] == 4
    # a quotient that only becomes a tie after narrowing: 7 / 2.796875 = 2.5027...; bf16 -> 2.5 -> 2
    xb = np.array([[7.0, 0, 0, 0]], dtype=ml_dtypes.bfloat16)
    sb = np.array([2.796875], dtype=ml_dtypes.bfloat16)
    qb, _ = O.quantize(xb, sb, scheme)
    assert qb.view(np.int8)[0, 0] == 2


def test_error_codes():
    x = np.zeros((4, 30), dtype=np.float32)
    with pytest.raises(O.OracleError):
        O.quantize(x, np.ones(1, dtype=np.float32), QuantScheme(value=QuantValue.Q8S))          # 30 % 4
    x = np.zeros((4, 32), dtype=np.float32)
    sch = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([4]))                         # 4 % 8
    with pytest.raises(O.OracleError) as e:
        O.quantize(x, np.ones((4, 8), dtype=np.float32), sch)
    assert e.value.status == 2
    sch = QuantScheme(value=QuantValue.Q4S, store=QuantStore.Native)                             # quantize.rs:213-219
    with pytest.raises(O.OracleError) as e:
        O.quantize(x, np.ones(1, dtype=np.float32), sch)
    assert e.value.status == 1
