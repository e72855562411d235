"""Seeded random configurations: rank, shape, value type, store, level (per tensor, last-dim blocks, N-d
blocks, tiles), param type, float type and the memory layout of the float tensor (contiguous, transposed,
a slice of a wider tensor, an odd element offset).  Every configuration checks the fused quantize, the
two-call form and dequantize against the oracle, bit for bit."""
import numpy as np
import pytest
import torch

from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue,
                        TensorHandleRef, _ffi, dequantize, quantize)
from oracle import oracle as O
from tests._cases import FLOATS
from tests._util import NP_FLOAT, assert_bits_equal, code_dtype, elem_of, empty_device, to_device, to_numpy

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch

U32_VALUES = [QuantValue.Q8F, QuantValue.Q8S, QuantValue.Q4F, QuantValue.Q4S, QuantValue.Q2F, QuantValue.Q2S]
NATIVE_VALUES = [QuantValue.Q8F, QuantValue.Q8S, QuantValue.E2M1, QuantValue.E4M3, QuantValue.E5M2]


def pick(rng, options):
    return options[int(rng.integers(len(options)))]


def draw(seed):
    rng = np.random.default_rng(1000 + seed)
    fname = pick(rng, list(FLOATS))
    store = QuantStore.U32 if rng.random() < 0.6 else QuantStore.Native
    value = pick(rng, U32_VALUES if store == QuantStore.U32 else NATIVE_VALUES)
    param = pick(rng, [QuantParam.F32, QuantParam.F32, QuantParam.F16, QuantParam.BF16])
    probe = QuantScheme(value=value, store=store)
    nq = probe.num_quants()
    rank = int(rng.integers(1, 5))
    kind = pick(rng, ["tensor", "last", "last", "nd", "tiles"]) if rank >= 2 else pick(rng, ["tensor", "last"])
    # last dim: a multiple of the block (which is a multiple of num_quants)
    b_last = int(nq * pick(rng, [1, 2, 3, 4, 8, 16]))
    while b_last > 255:
        b_last //= 2
    b_last = max(nq, b_last - b_last % nq)
    last = b_last * int(rng.integers(1, 9))
    lead = [int(rng.integers(1, 7)) for _ in range(rank - 1)]
    if rank >= 2 and rng.random() < 0.3:
        lead[-1] = int(rng.integers(30, 200))
    if rng.random() < 0.15:                              # large enough for many CTAs
        last *= 16
        if rank >= 2:
            lead[-1] *= 40
    while int(np.prod(lead + [last], dtype=np.int64)) > (4 << 20) and lead:      # keep the oracle fast
        i = int(np.argmax(lead))
        if lead[i] == 1:
            break
        lead[i] = max(1, lead[i] // 2)
    shape = tuple(lead + [last])
    if kind == "tensor":
        level = QuantLevel.Tensor
    elif kind == "last":
        level = QuantLevel.block([b_last])
    elif kind == "tiles":
        level = QuantLevel.block([pick(rng, [2, 4, 8, 32]), b_last])
    else:
        nb = int(rng.integers(2, rank + 1))
        level = QuantLevel.block([int(rng.integers(1, 5)) for _ in range(nb - 1)] + [b_last])
    scheme = QuantScheme(value=value, store=store, level=level, param=param)
    layout = pick(rng, ["contiguous", "contiguous", "transposed", "slice", "offset"])
    if layout == "transposed" and rank < 2:
        layout = "contiguous"
    F = FLOATS[fname]
    lo, hi = value.range()
    x = (rng.standard_normal(shape) * rng.uniform(0.05, 4.0)).astype(np.float32)
    mask = rng.random(shape) < 0.02
    x[mask] *= 8.0
    if rng.random() < 0.3:
        x.reshape(-1)[: max(1, x.size // 7)] = 0.0       # zero blocks
    return fname, F, scheme, shape, layout, x.astype(F)


def device_view(x, layout):
    """A device tensor with the values of `x` and the requested memory layout."""
    dense = to_device(x)
    if layout == "contiguous":
        return dense
    if layout == "transposed":
        perm = list(range(x.ndim))
        perm[-1], perm[-2] = perm[-2], perm[-1]
        return dense.permute(perm).contiguous().permute(perm)          # same values, last two strides swapped
    if layout == "slice":
        wide = torch.zeros(x.shape[:-1] + (x.shape[-1] + 24,), dtype=dense.dtype, device="cuda")
        wide[..., 8:8 + x.shape[-1]] = dense
        return wide[..., 8:8 + x.shape[-1]]
    flat = torch.zeros(x.size + 3, dtype=dense.dtype, device="cuda")
    flat[1:1 + x.size] = dense.reshape(-1)
    return flat[1:1 + x.size].view(x.shape)                            # base off by one element


@pytest.mark.parametrize("seed", range(400))
def test_random_configuration(seed):
    fname, F, scheme, shape, layout, x = draw(seed)
    elem = elem_of(F)
    pdt = NP_FLOAT[ElemType(int(scheme.param))]
    client = ComputeClient.current()
    dx = device_view(x, layout)
    assert tuple(dx.shape) == shape
    want_codes, want_scale = O.quantize_dynamic(x, scheme)
    want_restored = O.dequantize(want_codes, want_scale, scheme, F)

    # fused
    dq = empty_device(scheme.packed_shape(shape), code_dtype(scheme))
    ds = empty_device(scheme.scales_shape(shape), pdt)
    tin = _ffi.CTensor(H(dx))
    need = int(_ffi.lib().qk_workspace_bytes_for(tin.ref(), _ffi.c_scheme(scheme), int(elem)))
    ws = torch.zeros(max(need, 8192), dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic(client, H(dx), H(dq), H(ds), scheme, elem, H(ws))
    # two calls
    dscale = empty_device(scheme.scales_shape(shape), F)
    quantize.compute_scales(client, H(dx), H(dscale), scheme, elem, H(ws))
    dq2 = empty_device(scheme.packed_shape(shape), code_dtype(scheme))
    ds2 = empty_device(scheme.scales_shape(shape), pdt)
    quantize.launch_ref(client, H(dx), H(dq2), H(dscale), H(ds2), scheme, elem)
    # dequantize into a tensor of the same layout as the input
    dout = torch.zeros_like(dx) if layout == "contiguous" else device_view(np.zeros(shape, dtype=F), layout)
    dequantize.launch_ref(client, H(dq), H(dout), H(ds), scheme, elem)
    torch.cuda.synchronize()

    tag = f"{fname} {scheme.value.name} {scheme.store.name} {scheme.level} {scheme.param.name} {shape} {layout}"
    assert_bits_equal(to_numpy(dq, code_dtype(scheme)), want_codes, "fused codes: " + tag)
    assert_bits_equal(to_numpy(ds, pdt), want_scale, "fused scales: " + tag)
    assert_bits_equal(to_numpy(dscale, F), O.compute_scales(x, scheme), "compute_scales: " + tag)
    assert_bits_equal(to_numpy(dq2, code_dtype(scheme)), want_codes, "two-call codes: " + tag)
    assert_bits_equal(to_numpy(ds2, pdt), want_scale, "two-call scales: " + tag)
    assert_bits_equal(to_numpy(dout.contiguous(), F), want_restored, "restored: " + tag)
