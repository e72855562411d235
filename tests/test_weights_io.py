"""The quantized weight-set container: write / read round trip, shard merging (CPU), and a set
quantized on the GPU surviving save -> load -> dequantize unchanged."""
import numpy as np
import pytest

from cubek_b200 import ElemType, QuantLevel, QuantParam, QuantScheme, QuantStore, QuantValue
from cubek_b200 import weights as W
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor


def make(name, shape, scheme, seed, F=np.float32, rows=None):
    x = random_tensor(shape, F, seed)
    codes, scales = O.quantize_dynamic(x, scheme)
    raw = scales.view(np.uint32) if scales.dtype.itemsize == 4 else scales.view(np.uint16)
    return x, W.QuantizedTensor(name, shape, O.elem_type(F), scheme, codes, raw, rows)


def test_save_load_round_trip(tmp_path):
    schemes = [QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32])),
               QuantScheme(value=QuantValue.Q8S),
               QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16]), param=QuantParam.BF16)]
    items = [make(f"t{i}", (16 + i, 64), s, 70 + i, FLOATS["bf16"])[1] for i, s in enumerate(schemes)]
    path = tmp_path / "set.cubekq"
    W.save(path, items)
    back = W.load(path)
    assert [b.name for b in back] == ["t0", "t1", "t2"]
    for a, b in zip(items, back):
        assert (a.shape, a.elem, a.scheme, a.rows) == (b.shape, b.elem, b.scheme, b.rows)
        assert a.codes.tobytes() == b.codes.tobytes() and a.codes.dtype == b.codes.dtype
        assert a.scales.tobytes() == b.scales.tobytes()
    raw = path.read_bytes()
    assert raw[:8] == W.MAGIC and len(raw) % 256 == 0
    with pytest.raises(ValueError):
        (tmp_path / "bad").write_bytes(b"nonsense" * 4)
        W.load(tmp_path / "bad")


def test_row_shards_merge_to_the_whole_tensor():
    scheme = QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([32]))
    x, whole = make("w", (48, 128), scheme, 80)
    pieces = []
    for start, count in ((32, 16), (0, 16), (16, 16)):
        codes, scales = O.quantize_dynamic(x[start:start + count], scheme)
        pieces.append(W.QuantizedTensor("w", (count, 128), ElemType.F32, scheme, codes, scales.view(np.uint32), (start, count)))
    merged = W.merge_row_shards(pieces)
    assert merged.shape == (48, 128)
    assert merged.codes.tobytes() == whole.codes.tobytes() and merged.scales.tobytes() == whole.scales.tobytes()
    with pytest.raises(ValueError):
        W.merge_row_shards(pieces[:2])


def test_llama_shape_list():
    shapes = W.llama3_8b_shapes()
    assert len(shapes) == 225 and sum(r * c for _, r, c in shapes) == 7504658432


@pytest.mark.gpu
def test_gpu_set_survives_the_container(tmp_path):
    import torch
    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from tests._util import empty_device, to_device, to_numpy

    H = TensorHandleRef.from_torch
    client = ComputeClient.current()
    scheme = QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([128]))
    F = FLOATS["bf16"]
    shapes = [(64, 256), (32, 1024), (128, 128)]
    xs = [random_tensor(s, F, 90 + i, "normal") for i, s in enumerate(shapes)]
    dx = [to_device(x) for x in xs]
    dq = [empty_device(scheme.packed_shape(s), np.uint32) for s in shapes]
    ds = [empty_device(scheme.scales_shape(s), np.float32) for s in shapes]
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    quantize.launch_dynamic_batch(client, [H(t) for t in dx], [H(t) for t in dq], [H(t) for t in ds], scheme, ElemType.BF16, H(ws))
    torch.cuda.synchronize()
    items = [W.QuantizedTensor(f"w{i}", s, ElemType.BF16, scheme, to_numpy(q, np.uint32), to_numpy(sc, np.float32).view(np.uint32))
             for i, (s, q, sc) in enumerate(zip(shapes, dq, ds))]
    W.save(tmp_path / "w.cubekq", items)
    back = W.load(tmp_path / "w.cubekq")
    dq2 = [to_device(b.codes) for b in back]
    ds2 = [to_device(b.scales.view(np.float32)) for b in back]
    do = [empty_device(s, F) for s in shapes]
    dequantize.launch_batch(client, [H(t) for t in dq2], [H(t) for t in do], [H(t) for t in ds2], scheme, ElemType.BF16)
    torch.cuda.synchronize()
    for x, b, o in zip(xs, back, do):
        oc, osc = O.quantize_dynamic(x, scheme)
        assert b.codes.tobytes() == oc.tobytes()
        assert to_numpy(o, F).tobytes() == O.dequantize(oc, osc, scheme, F).tobytes()
