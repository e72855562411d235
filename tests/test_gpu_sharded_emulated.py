"""The row-sharded path on ONE GPU: the ranks of a world of 2, 3 and 8 are played one after the other by this
process, each on its own rows (`shard.plan_rows`), and the only exchange of the path - all-reduce(MAX) of one f32 per
tensor - is replaced by the element-wise maximum of the ranks' absmax vectors, which is what that collective
computes.  Everything else is the code a multi-GPU run executes: `qk_absmax_batch`, `qk_quantize_from_absmax_batch`
(`shard.ShardedPerTensorSet`), the fused batch quantize for per-block schemes, `qk_dequantize_batch`.  The
concatenated shards must equal the oracle's result on the whole tensors bit for bit, and every rank must hold the
same scale bits."""
import numpy as np
import pytest
import torch

from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef,
                        dequantize, quantize)
from cubek_b200.shard import ShardedPerTensorSet, plan_rows
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import NP_FLOAT, assert_bits_equal, to_device, to_numpy

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch
SHAPES = [(4096, 512), (1024, 4096), (37, 256), (3, 128), (1500, 1024)]


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("fname", ["bf16", "f32"])
def test_per_tensor_set_sharded_by_rows(world, fname):
    F = FLOATS[fname]
    elem = {"f32": ElemType.F32, "bf16": ElemType.BF16}[fname]
    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32)
    xs = [random_tensor(sh, F, 600 + i, "normal") for i, sh in enumerate(SHAPES)]
    xs[1][-1, -1] = 11.0          # the largest magnitude of tensor 1 sits in the last rank's rows
    xs[3][0, 0] = -7.5            # tensor 3 has fewer rows than ranks: some ranks hold nothing of it
    client = ComputeClient.current()
    ranks = []
    for r in range(world):
        plan = [plan_rows(x.shape[0], x.shape[1], world, elem, scheme)[r] for x in xs]
        held = [i for i, p in enumerate(plan) if p.rows > 0]
        mine = [to_device(xs[i][plan[i].row_start: plan[i].row_start + plan[i].rows]) for i in held]
        codes = [torch.empty(scheme.packed_shape(t.shape), dtype=torch.int32, device="cuda") for t in mine]
        scales = [torch.empty(1, dtype=torch.float32, device="cuda") for _ in mine]
        cells = torch.zeros(len(mine), dtype=torch.float32, device="cuda")
        sset = ShardedPerTensorSet(client, [H(t) for t in mine], [H(t) for t in codes], [H(t) for t in scales], cells, scheme, elem)
        sset.absmax()
        ranks.append(dict(plan=plan, held=held, mine=mine, codes=codes, scales=scales, cells=cells, sset=sset))
    # the exchange: MAX over the ranks of one f32 per tensor (ranks without rows of a tensor contribute 0)
    glob = torch.zeros(len(xs), dtype=torch.float32, device="cuda")
    for rk in ranks:
        glob[torch.tensor(rk["held"], device="cuda")] = torch.maximum(glob[torch.tensor(rk["held"], device="cuda")], rk["cells"])
    for rk in ranks:
        rk["cells"].copy_(glob[torch.tensor(rk["held"], device="cuda")])
        rk["sset"].quantize()
    torch.cuda.synchronize()
    for i, x in enumerate(xs):
        want_codes, want_scale = O.quantize_dynamic(x, scheme)
        pieces = []
        for rk in ranks:
            if i in rk["held"]:
                k = rk["held"].index(i)
                assert_bits_equal(to_numpy(rk["scales"][k], np.float32), want_scale, f"scale of tensor {i} on a rank")
                pieces.append(to_numpy(rk["codes"][k], np.uint32))
        assert_bits_equal(np.concatenate(pieces, axis=0), want_codes, f"codes of tensor {i}")


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("value,block", [(QuantValue.Q4S, 32), (QuantValue.Q8S, 128), (QuantValue.Q2S, 64)])
def test_per_block_set_sharded_by_rows_needs_no_exchange(world, value, block):
    elem, F = ElemType.BF16, NP_FLOAT[ElemType.BF16]
    scheme = QuantScheme(value=value, store=QuantStore.U32, level=QuantLevel.block([block]))
    xs = [random_tensor(sh, F, 700 + i, "outliers") for i, sh in enumerate(SHAPES)]
    client = ComputeClient.current()
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    got = [dict(codes=[], scales=[], restored=[]) for _ in xs]
    for r in range(world):
        plan = [plan_rows(x.shape[0], x.shape[1], world, elem, scheme)[r] for x in xs]
        held = [i for i, p in enumerate(plan) if p.rows > 0]
        mine = [to_device(xs[i][plan[i].row_start: plan[i].row_start + plan[i].rows]) for i in held]
        codes = [torch.empty(scheme.packed_shape(t.shape), dtype=torch.int32, device="cuda") for t in mine]
        scales = [torch.empty(scheme.scales_shape(t.shape), dtype=torch.float32, device="cuda") for t in mine]
        outs = [torch.empty_like(t) for t in mine]
        quantize.launch_dynamic_batch(client, [H(t) for t in mine], [H(t) for t in codes], [H(t) for t in scales], scheme, elem, H(ws))
        dequantize.launch_batch(client, [H(t) for t in codes], [H(t) for t in outs], [H(t) for t in scales], scheme, elem)
        torch.cuda.synchronize()
        for k, i in enumerate(held):
            got[i]["codes"].append(to_numpy(codes[k], np.uint32))
            got[i]["scales"].append(to_numpy(scales[k], np.float32))
            got[i]["restored"].append(to_numpy(outs[k], F))
    for i, x in enumerate(xs):
        want_codes, want_scale = O.quantize_dynamic(x, scheme)
        assert_bits_equal(np.concatenate(got[i]["codes"], axis=0), want_codes, f"codes of tensor {i}")
        assert_bits_equal(np.concatenate(got[i]["scales"], axis=0), want_scale, f"scales of tensor {i}")
        assert_bits_equal(np.concatenate(got[i]["restored"], axis=0), O.dequantize(want_codes, want_scale, scheme, F),
                          f"restored tensor {i}")
