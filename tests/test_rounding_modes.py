"""The rounding of exact .5 ties is the one point of the path the reference leaves to its JIT back end
(`Line::round`, crates/cubek-quant/src/quantize.rs:27).  Both plausible lowerings exist here: round-half-to-even
(the default library and oracle) and round-half-away-from-zero (`libcubek_quant_b200_half_away.so`,
`liboracle_half_away.so`).  The two oracles are checked against the NumPy restatement and against each other (they
may differ on ties only); on a GPU the half-away library must match the half-away oracle bit for bit."""
import ctypes as C

import numpy as np
import pytest

from cubek_b200 import ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef
from cubek_b200 import _ffi
from oracle import numpy_restatement as NR
from oracle import oracle as O
from tests._cases import FLOATS, adversarial_tensor, random_tensor

SCHEMES = [QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32),
           QuantScheme(value=QuantValue.Q4F, store=QuantStore.U32, level=QuantLevel.block([16])),
           QuantScheme(value=QuantValue.Q2S, store=QuantStore.U32, level=QuantLevel.block([32])),
           QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16])),
           QuantScheme(value=QuantValue.Q8S, store=QuantStore.Native, level=QuantLevel.block([32]))]


def tie_tensor(F, scheme, seed):
    """Quotients on exact halves: integers and half-integers times a power-of-two scale."""
    rng = np.random.default_rng(seed)
    lo, hi = scheme.value.range()
    k = rng.integers(int(lo) - 1, int(hi) + 1, (8, 64)).astype(np.float32)
    x = (k + rng.choice(np.array([0.0, 0.5], dtype=np.float32), k.shape)) * np.float32(0.25)
    return x.astype(F)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", SCHEMES, ids=lambda s: f"{s.value.name}-{s.store.name}")
def test_half_away_oracle_matches_the_numpy_restatement(fname, scheme):
    F = FLOATS[fname]
    for x in (tie_tensor(F, scheme, 3), adversarial_tensor((8, 64), F, scheme, 4)):
        scale = np.full(scheme.scales_shape(x.shape), 0.25, dtype=F)
        for rounding in ("even", "away"):
            codes, out_scale = O.quantize(x, scale, scheme, rounding=rounding)
            n_codes, n_scale = NR.quantize(x, scale, scheme, rounding=rounding)
            assert codes.tobytes() == n_codes.tobytes(), rounding
            assert out_scale.tobytes() == n_scale.tobytes()


def test_the_two_roundings_differ_on_ties_only():
    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.Native)
    x = tie_tensor(np.float32, scheme, 5)
    scale = np.array([0.25], dtype=np.float32)
    even, _ = O.quantize(x, scale, scheme, rounding="even")
    away, _ = O.quantize(x, scale, scheme, rounding="away")
    q = x / np.float32(0.25)
    is_tie = (np.abs(q - np.trunc(q)) == 0.5) & (np.abs(q) < 127)
    differ = even != away
    assert differ.any() and not (differ & ~is_tie).any()
    # half to even and half away agree on ties whose even neighbour is also the farther one from zero
    assert np.array_equal(away[is_tie].astype(np.int32), (np.sign(q[is_tie]) * np.ceil(np.abs(q[is_tie]))).astype(np.int32))
    # no ties, no difference
    y = random_tensor((16, 64), np.float32, 6)
    s = O.compute_scales(y, scheme)
    assert O.quantize(y, s, scheme, rounding="even")[0].tobytes() == O.quantize(y, s, scheme, rounding="away")[0].tobytes()


def test_half_away_library_loads_and_says_so():
    lib = _ffi.load(_ffi.LIB_PATH_HALF_AWAY)
    assert b"half away" in lib.qk_version()
    assert b"half away" not in _ffi.lib().qk_version()


@pytest.mark.gpu
@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("scheme", SCHEMES, ids=lambda s: f"{s.value.name}-{s.store.name}")
def test_half_away_library_matches_half_away_oracle(fname, scheme):
    import torch

    from tests._util import NP_FLOAT, assert_bits_equal, code_dtype, elem_of, empty_device, to_device, to_numpy

    lib = _ffi.load(_ffi.LIB_PATH_HALF_AWAY)
    F = FLOATS[fname]
    for x in (tie_tensor(F, scheme, 7), adversarial_tensor((64, 256), F, scheme, 8), random_tensor((64, 256), F, 9)):
        want_codes, want_scale = O.quantize_dynamic(x, scheme, rounding="away")
        dx = to_device(x)
        dq = empty_device(scheme.packed_shape(x.shape), code_dtype(scheme))
        ds = empty_device(scheme.scales_shape(x.shape), np.float32)
        ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
        ti, tq, ts = _ffi.c_tensors(*(TensorHandleRef.from_torch(t) for t in (dx, dq, ds)))
        rc = lib.qk_quantize_dynamic(ti.ref(), tq.ref(), ts.ref(), _ffi.c_scheme(scheme), int(elem_of(F)), ws.data_ptr(),
                                     ws.numel(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0, _ffi.strerror(rc)
        assert_bits_equal(to_numpy(ds, np.float32), want_scale, "scales")
        assert_bits_equal(to_numpy(dq, code_dtype(scheme)), want_codes, "codes (half away)")
