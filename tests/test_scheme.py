"""Host-side scheme logic against the constants the reference's call sites imply."""
import pytest

from cubek_b200 import BlockSize, QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue


def test_default_scheme_matches_reference_default():
    s = QuantScheme()
    assert (s.value, s.param, s.store, s.level.is_tensor) == (QuantValue.Q8F, QuantParam.F32, QuantStore.U32, True)


@pytest.mark.parametrize("value,bits,nq,rng", [
    (QuantValue.Q8F, 8, 4, (-128, 127)), (QuantValue.Q8S, 8, 4, (-127, 127)),
    (QuantValue.Q4F, 4, 8, (-8, 7)), (QuantValue.Q4S, 4, 8, (-7, 7)),
    (QuantValue.Q2F, 2, 16, (-2, 1)), (QuantValue.Q2S, 2, 16, (-1, 1)),
    (QuantValue.E2M1, 4, 8, (-6, 6)), (QuantValue.E4M3, 8, 4, (-448, 448)),
])
def test_value_constants(value, bits, nq, rng):
    s = QuantScheme().with_value(value).with_store(QuantStore.U32)
    assert value.size_bits() == bits
    assert s.num_quants() == nq          # 32 / 8 = 4 (quantize.rs:305)
    assert value.range() == tuple(float(v) for v in rng)


def test_native_num_quants():
    assert QuantScheme(value=QuantValue.Q8S, store=QuantStore.Native).num_quants() == 1
    assert QuantScheme(value=QuantValue.E4M3, store=QuantStore.Native).num_quants() == 1
    # e2m1 has native packing (e2m1x2): crates/cubek-matmul/src/base.rs:506-512
    assert QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native).num_quants() == 2


def test_builder_is_immutable_and_chained():
    base = QuantScheme()
    s = (base.with_level(QuantLevel.block([32])).with_value(QuantValue.Q4S)
         .with_store(QuantStore.U32).with_param(QuantParam.F32))
    assert base.level.is_tensor and not s.level.is_tensor
    assert s.level.block_size.as_slice() == (32,)


def test_block_size_to_dim_vec_left_pads():
    assert BlockSize((32,)).to_dim_vec(2) == (1, 32)       # layout/scales.rs:239
    assert BlockSize((2, 16)).to_dim_vec(3) == (1, 2, 16)
    with pytest.raises(ValueError):
        BlockSize((2, 16)).to_dim_vec(1)
    with pytest.raises(ValueError):
        BlockSize((256,))                                   # block extents are u8


def test_shapes():
    s = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32]))
    assert s.packed_shape((16, 64)) == (16, 8)              # symmetric.rs:68-69
    assert s.scales_shape((16, 64)) == (16, 2)              # symmetric.rs:158-159
    assert QuantScheme().scales_shape((16, 64)) == (1,)
    with pytest.raises(ValueError):
        s.packed_shape((16, 60))
