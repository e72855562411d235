"""The benchmark configurations at their full sizes: every element of every configuration is compared bit for
bit with the oracle (codes, scales, restored values), and so are the eight tensors of one batched benchmark
step.  Size-independent properties are checked besides: the fused one-pass result equals the two-call result,
the round-trip error is within half a quantization step of every element, and re-quantizing the restored
tensor with the same scales reproduces the codes (idempotence)."""
import numpy as np
import pytest
import torch

from cubek_b200 import ComputeClient, ElemType, QuantParam, TensorHandleRef, dequantize, quantize
from cubek_b200.synthetic import TORCH_DTYPE, WORKLOADS, generate
from oracle import oracle as O
from tests._util import NP_FLOAT, assert_bits_equal, to_numpy

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch

FULL = ["q8_tensor_f32_4096x4096", "q4_block32_bf16_14336x4096", "e2m1_block16_f16_8192x4096",
        "e2m1_block32_f16_8192x4096", "q2_block64_f32_65536x4096", "q8_block128_bf16_14336x4096",
        "q8_tensor_bf16_14336x4096"]


def run_full(w, x):
    s, elem = w.scheme, w.elem
    client = ComputeClient.current()
    code_t = torch.int32 if s.store.name == "U32" else torch.uint8
    codes = torch.empty(s.packed_shape(x.shape), dtype=code_t, device="cuda")
    out_scale = torch.empty(s.scales_shape(x.shape), dtype=torch.float32, device="cuda")
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic(client, H(x), H(codes), H(out_scale), s, elem, H(ws))
    restored = torch.empty_like(x)
    dequantize.launch_ref(client, H(codes), H(restored), H(out_scale), s, elem)
    torch.cuda.synchronize()
    return codes, out_scale, restored


@pytest.mark.parametrize("name", FULL)
def test_full_size_configuration(name):
    w = WORKLOADS[name]
    s, elem = w.scheme, w.elem
    F = NP_FLOAT[elem]
    x = generate(w, "cuda")
    rows, cols = x.shape
    client = ComputeClient.current()
    codes, out_scale, restored = run_full(w, x)

    # (a) the two-call form gives the same bits as the fused one
    scale = torch.empty(s.scales_shape(x.shape), dtype=TORCH_DTYPE[elem], device="cuda")
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.compute_scales(client, H(x), H(scale), s, elem, H(ws))
    codes2 = torch.empty_like(codes)
    out_scale2 = torch.empty_like(out_scale)
    quantize.launch_ref(client, H(x), H(codes2), H(scale), H(out_scale2), s, elem)
    torch.cuda.synchronize()
    assert torch.equal(codes, codes2) and torch.equal(out_scale.view(torch.int32), out_scale2.view(torch.int32))

    # (b) round trip within half a step (plus the narrowing of the product for 16-bit types)
    if s.level.is_tensor:
        step = out_scale.reshape(1, 1).expand(rows, cols)
    else:
        step = out_scale.repeat_interleave(s.level.block_size.as_slice()[-1], dim=1)
    err = (restored.float() - x.float()).abs()
    if s.value.name == "E2M1":
        bound = step * 1.5                     # round to an integer (0.5), then 5 -> 4 on the fp4 grid (1.0)
    else:
        bound = step * 0.5
    # The quotient and the product are rounded to F: relative 2^-24 (the reference tests allow
    # 1e-4), 2^-11 for f16, 2^-8 for bf16, once on the way in (can move the code by one) and once out.
    rel = {ElemType.F32: 1e-4, ElemType.F16: 2.0 ** -9, ElemType.BF16: 2.0 ** -6}[elem]
    assert bool((err <= bound * (1 + 1e-4) + x.float().abs() * rel + 1e-30).all())

    # (c) idempotence: quantizing the restored tensor with the same scales gives the same codes
    if s.value.name != "E2M1":
        codes3 = torch.empty_like(codes)
        out_scale3 = torch.empty_like(out_scale)
        quantize.launch_ref(client, H(restored), H(codes3), H(out_scale.to(TORCH_DTYPE[elem])), H(out_scale3), s, elem)
        torch.cuda.synchronize()
        if elem == ElemType.F32:
            assert torch.equal(codes, codes3)

    # (d) bit-exact against the oracle on the whole tensor
    o_codes, o_scale = O.quantize_dynamic(to_numpy(x, F), s)
    assert_bits_equal(to_numpy(out_scale, np.float32), o_scale, "scales")
    assert_bits_equal(to_numpy(codes, o_codes.dtype), o_codes, "codes")
    o_restored = O.dequantize(o_codes, o_scale, s, F)
    assert_bits_equal(to_numpy(restored, F), o_restored, "restored")


@pytest.mark.parametrize("name", ["q4_block32_bf16_14336x4096", "q8_tensor_bf16_14336x4096"])
def test_batched_benchmark_step_matches_the_oracle_on_every_tensor(name):
    """The call the benchmark times: eight distinct 14336 x 4096 tensors through qk_quantize_dynamic_batch and
    qk_dequantize_batch (one launch each for the block scheme); all eight compared with the oracle in full."""
    w = WORKLOADS[name]
    s, elem = w.scheme, w.elem
    F = NP_FLOAT[elem]
    client = ComputeClient.current()
    xs = [generate(w, "cuda", seed_offset=i) for i in range(8)]
    codes = [torch.empty(s.packed_shape(x.shape), dtype=torch.int32, device="cuda") for x in xs]
    scales = [torch.empty(s.scales_shape(x.shape), dtype=torch.float32, device="cuda") for x in xs]
    outs = [torch.empty_like(x) for x in xs]
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.PreparedDynamicBatch(client, [H(t) for t in xs], [H(t) for t in codes], [H(t) for t in scales], s, elem, H(ws))()
    dequantize.PreparedBatch(client, [H(t) for t in codes], [H(t) for t in outs], [H(t) for t in scales], s, elem)()
    torch.cuda.synchronize()
    for i in range(8):
        o_codes, o_scale = O.quantize_dynamic(to_numpy(xs[i], F), s)
        assert_bits_equal(to_numpy(scales[i], np.float32), o_scale, f"scales of tensor {i}")
        assert_bits_equal(to_numpy(codes[i], np.uint32), o_codes, f"codes of tensor {i}")
        assert_bits_equal(to_numpy(outs[i], F), O.dequantize(o_codes, o_scale, s, F), f"restored tensor {i}")


def test_embedding_sized_tensor_q8_block128():
    """The largest single tensor of the Llama-3-8B-shaped set (128256 x 4096 bf16, 1 GB)."""
    from dataclasses import replace

    w = replace(WORKLOADS["q8_block128_bf16_14336x4096"], shape=(128256, 4096))
    x = generate(w, "cuda")
    codes, out_scale, restored = run_full(w, x)
    F = NP_FLOAT[w.elem]
    pick = torch.tensor([0, 1, 777, 64000, 128255], device="cuda")
    xs = to_numpy(x[pick].contiguous(), F)
    o_codes, o_scale = O.quantize_dynamic(xs, w.scheme)
    assert_bits_equal(to_numpy(codes[pick].contiguous(), np.uint32), o_codes, "codes")
    assert_bits_equal(to_numpy(restored[pick].contiguous(), F), O.dequantize(o_codes, o_scale, w.scheme, F), "restored")


@pytest.mark.parametrize("level", ["block32", "tensor"])
def test_more_than_2_31_elements(level):
    """A bf16 tensor of 2^31 + 2^20 elements (4.3 GB): unit, element and byte offsets pass 2^31 and 2^32.
    Whole rows at the start, around the 2^31-element boundary and at the very end are compared with the
    oracle; for the per-tensor scheme the largest magnitude is the tensor's last element."""
    from cubek_b200 import QuantLevel, QuantScheme, QuantValue

    rows, cols = (1 << 19) + 256, 4096
    assert rows * cols > 1 << 31
    if level == "block32":
        s = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32]))
    else:
        s = QuantScheme(value=QuantValue.Q8S)
    elem, F = ElemType.BF16, NP_FLOAT[ElemType.BF16]
    x = torch.empty((rows, cols), dtype=torch.bfloat16, device="cuda").normal_(0.0, 0.02, generator=torch.Generator("cuda").manual_seed(31))
    if level == "tensor":
        x[-1, -1] = 3.0
    client = ComputeClient.current()
    codes = torch.empty(s.packed_shape(x.shape), dtype=torch.int32, device="cuda")
    out_scale = torch.empty(s.scales_shape(x.shape), dtype=torch.float32, device="cuda")
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic(client, H(x), H(codes), H(out_scale), s, elem, H(ws))
    restored = torch.empty_like(x)
    dequantize.launch_ref(client, H(codes), H(restored), H(out_scale), s, elem)
    torch.cuda.synchronize()
    half = (1 << 31) // cols
    pick = torch.tensor([0, 1, half - 1, half, half + 1, rows - 2, rows - 1], device="cuda")
    xs = to_numpy(x[pick].contiguous(), F)
    if level == "tensor":
        lo, hi = s.value.range()
        want_scale = np.array([np.float32(2) * np.float32(3.0) / np.float32(hi - lo)], dtype=np.float32).astype(F)
        o_codes, o_scale = O.quantize(xs, want_scale, s)
        assert_bits_equal(to_numpy(out_scale, np.float32), o_scale, "scale")
    else:
        o_codes, o_scale = O.quantize_dynamic(xs, s)
        assert_bits_equal(to_numpy(out_scale[pick].contiguous(), np.float32), o_scale, "scales")
    assert_bits_equal(to_numpy(codes[pick].contiguous(), np.uint32), o_codes, "codes")
    assert_bits_equal(to_numpy(restored[pick].contiguous(), F), O.dequantize(o_codes, o_scale, s, F), "restored")
    # every element took part: the restored tensor is within half a step everywhere
    step = out_scale.reshape(1, 1) if level == "tensor" else None
    if step is not None:
        err = (restored.float() - x.float()).abs().max()
        assert float(err) <= float(step.max()) * 0.5 * (1 + 1e-4) + 3.0 * 2.0 ** -6
