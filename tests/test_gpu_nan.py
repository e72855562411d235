"""NaN elements are outside the parity contract (the reference leaves their code to its back end), but they must
stay inside their own code: the scale of a block is the absmax of its other elements, and every other element
of the block, of the stored word and of the tensor gets exactly the code it would get with the NaN replaced by
zero.  Checked for the fused kernels (whose shortcut arithmetic drops the clamp), the given-scale kernels, the
per-tensor routes and the two-blocks-per-unit form."""
import numpy as np
import pytest

from cubek_b200 import QuantLevel, QuantScheme, QuantStore, QuantValue
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import assert_bits_equal, gpu_dequantize, gpu_quantize, gpu_quantize_dynamic

pytestmark = pytest.mark.gpu

VALUES = [(QuantValue.Q8S, QuantStore.U32), (QuantValue.Q4S, QuantStore.U32), (QuantValue.Q2S, QuantStore.U32),
          (QuantValue.Q8S, QuantStore.Native), (QuantValue.E2M1, QuantStore.Native), (QuantValue.E4M3, QuantStore.Native)]


def element_codes(codes, scheme):
    """One integer per element (fields of the stored words / bytes), so that single elements can be masked."""
    bits = scheme.value.size_bits()
    if scheme.store == QuantStore.U32:
        nq = 32 // bits
        shifts = (np.arange(nq, dtype=np.uint32) * bits)
        return ((codes[..., None] >> shifts) & np.uint32((1 << bits) - 1)).reshape(codes.shape[0], -1)
    if bits == 4:
        b = codes.view(np.uint8)
        return np.stack([b & 0xF, b >> 4], axis=-1).reshape(codes.shape[0], -1)
    return codes.view(np.uint8)


@pytest.mark.parametrize("fname", list(FLOATS))
@pytest.mark.parametrize("value,store", VALUES)
@pytest.mark.parametrize("level", ["tensor", "block16", "block32", "block128"])
def test_nan_elements_do_not_disturb_their_neighbours(fname, value, store, level):
    F = FLOATS[fname]
    lvl = QuantLevel.Tensor if level == "tensor" else QuantLevel.block([int(level[5:])])
    scheme = QuantScheme(value=value, store=store, level=lvl)
    if not scheme.level.is_tensor and int(level[5:]) % scheme.num_quants():
        pytest.skip("block not a multiple of num_quants")
    x = random_tensor((96, 512), F, 77, "normal")
    rng = np.random.default_rng(78)
    nan_at = np.zeros(x.shape, dtype=bool)
    nan_at[rng.integers(0, 96, 40), rng.integers(0, 512, 40)] = True
    nan_at[5, 0:3] = True          # neighbours inside one word
    nan_at[9, 511] = True          # last element of a row
    clean = x.copy()
    clean[nan_at] = 0
    dirty = x.copy()
    dirty[nan_at] = np.nan
    want_codes, want_scale = O.quantize_dynamic(clean, scheme)
    keep = ~nan_at
    # fused
    codes, scale = gpu_quantize_dynamic(dirty, scheme)
    assert_bits_equal(scale, want_scale, "scales (fused)")
    assert np.array_equal(element_codes(codes, scheme)[keep], element_codes(want_codes, scheme)[keep]), "codes (fused)"
    # given scales
    given = O.compute_scales(clean, scheme)
    codes, scale = gpu_quantize(dirty, given, scheme)
    assert_bits_equal(scale, want_scale, "scales (given)")
    assert np.array_equal(element_codes(codes, scheme)[keep], element_codes(want_codes, scheme)[keep]), "codes (given)"
