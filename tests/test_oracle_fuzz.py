"""Property-based cross-check of the two CPU restatements (C oracle vs NumPy / ml_dtypes) over random
shapes, block layouts, value types and float types, plus algebraic properties of the oracle itself."""
import numpy as np
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from cubek_b200 import QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue
from oracle import numpy_restatement as R
from oracle import oracle as O
from tests._cases import FLOATS, all_value_stores

VALUE_STORES = list(all_value_stores())


@st.composite
def cases(draw):
    value, store = draw(st.sampled_from(VALUE_STORES))
    fname = draw(st.sampled_from(list(FLOATS)))
    param = draw(st.sampled_from(list(QuantParam)))
    nq = QuantScheme(value=value, store=store).num_quants()
    rank = draw(st.integers(1, 3))
    last = nq * draw(st.integers(1, 6))
    shape = tuple(draw(st.integers(1, 5)) for _ in range(rank - 1)) + (last,)
    if draw(st.booleans()):
        level = QuantLevel.Tensor
    else:
        brank = draw(st.integers(1, rank))
        blk = [draw(st.integers(1, 4)) for _ in range(brank - 1)] + [nq * draw(st.integers(1, 3))]
        level = QuantLevel.block(blk)
    seed = draw(st.integers(0, 2**31 - 1))
    mag = draw(st.sampled_from([1e-3, 1.0, 37.5, 1e4]))
    return fname, QuantScheme(value=value, store=store, param=param, level=level), shape, seed, mag


@settings(max_examples=150, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(cases())
def test_restatements_agree(case):
    fname, scheme, shape, seed, mag = case
    F = FLOATS[fname]
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(shape) * mag).astype(np.float32).astype(F)
    s = O.compute_scales(x, scheme)
    assert s.tobytes() == R.compute_scales(x, scheme).tobytes()
    q, os_ = O.quantize(x, s, scheme)
    q2, os2 = R.quantize(x, s, scheme)
    assert q.tobytes() == q2.tobytes() and os_.tobytes() == os2.tobytes()
    d = O.dequantize(q, os_, scheme, F)
    assert d.tobytes() == R.dequantize(q2, os2, scheme, F).tobytes()


@settings(max_examples=60, deadline=None)
@given(st.sampled_from([QuantValue.Q8S, QuantValue.Q4S, QuantValue.Q2S]), st.integers(0, 2**31 - 1))
def test_symmetric_ranges_negate(value, seed):
    """Symmetric ranges and round-half-to-even make quantization odd: q(-x) = -q(x), so the restored
    tensors are exact negatives (f32, power-of-two free scale)."""
    scheme = QuantScheme(value=value, store=QuantStore.U32, level=QuantLevel.block([16]))
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((4, 64)).astype(np.float32)
    qa, sa = O.quantize_dynamic(x, scheme)
    qb, sb = O.quantize_dynamic(-x, scheme)
    assert sa.tobytes() == sb.tobytes()
    da, db = O.dequantize(qa, sa, scheme, np.float32), O.dequantize(qb, sb, scheme, np.float32)
    assert np.array_equal(da, -db)


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 2**31 - 1), st.integers(-8, 8))
def test_power_of_two_scaling_commutes(seed, k):
    """Multiplying the input by 2^k multiplies scales and restored values by 2^k and leaves the codes."""
    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32, level=QuantLevel.block([32]))
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((4, 64)).astype(np.float32)
    f = np.float32(2.0 ** k)
    qa, sa = O.quantize_dynamic(x, scheme)
    qb, sb = O.quantize_dynamic(x * f, scheme)
    assert qa.tobytes() == qb.tobytes() and np.array_equal(sa * f, sb)
