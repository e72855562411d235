"""Host-side sharding logic, and the N>1 data path on CPU ranks (gloo, world size 2): shards
concatenate to the single-device result and the max-reduced absmax gives every rank the scale
of the whole tensor."""
import os
import socket

import numpy as np
import pytest

from cubek_b200 import ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue
from cubek_b200.shard import assign_round_robin, plan_rows, row_granularity


@pytest.mark.parametrize("rows,cols,world", [(14336, 4096, 8), (65536, 4096, 4), (1024, 4096, 8), (1000, 64, 3),
                                             (5, 4096, 8), (128256, 4096, 8)])
def test_plan_rows_partitions_exactly(rows, cols, world):
    scheme = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32]))
    shards = plan_rows(rows, cols, world, ElemType.BF16, scheme)
    assert len(shards) == world
    assert shards[0].row_start == 0 and sum(s.rows for s in shards) == rows
    g = row_granularity(cols, ElemType.BF16, scheme)
    for a, b in zip(shards, shards[1:]):
        assert a.row_start + a.rows == b.row_start
        assert b.row_start % g == 0 or b.rows == 0
    for s in shards:
        assert (s.row_start * cols * 2) % 256 == 0           # input bytes
        assert (s.row_start * cols // 8 * 4) % 256 == 0 or s.rows == 0      # packed bytes
    sizes = [s.rows for s in shards if s.rows]
    assert max(sizes) - min(sizes) <= g or len(sizes) < world


def test_plan_rows_rejects_blocks_that_straddle_rows():
    with pytest.raises(ValueError):
        plan_rows(64, 96, 2, ElemType.F32, QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([64])))
    with pytest.raises(ValueError):
        plan_rows(64, 128, 2, ElemType.F32, QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([2, 64])))


def test_round_robin_balances_a_llama_layer_set():
    from cubek_b200.synthetic import LLAMA3_8B_EMBEDDING, LLAMA3_8B_LAYER, LLAMA3_8B_LAYERS

    sizes = [r * c for _, r, c in LLAMA3_8B_LAYER] * LLAMA3_8B_LAYERS + [LLAMA3_8B_EMBEDDING[1] * LLAMA3_8B_EMBEDDING[2]]
    assert len(sizes) == 225 and sum(sizes) == 7504658432
    owned = assign_round_robin(sizes, 8)
    assert sorted(i for o in owned for i in o) == list(range(225))
    load = [sum(sizes[i] for i in o) for o in owned]
    assert max(load) / (sum(load) / 8) < 1.08


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, rows, cols, result_dir):
    import torch
    import torch.distributed as dist

    from cubek_b200.shard import allreduce_absmax, plan_rows
    from oracle import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(42)
        full = rng.standard_normal((rows, cols)).astype(np.float32)
        full[rows - 1, cols - 1] = 17.25          # the global absmax sits in the last rank's shard
        tensor_scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32)
        block_scheme = QuantScheme(value=QuantValue.Q4S, store=QuantStore.U32, level=QuantLevel.block([32]))
        shard = plan_rows(rows, cols, world, ElemType.F32, tensor_scheme)[rank]
        mine = full[shard.row_start: shard.row_start + shard.rows]

        # per tensor: local absmax -> all_reduce(MAX) -> scale, identical bits on every rank
        local = np.float32(np.abs(mine).max()) if mine.size else np.float32(0)
        t = torch.tensor([local], dtype=torch.float32)
        allreduce_absmax(t)
        lo, hi = tensor_scheme.value.range()
        scale = np.array([(np.float32(2) * np.float32(t.item())) / np.float32(hi - lo)], dtype=np.float32)
        want_scale = O.compute_scales(full, tensor_scheme)
        assert scale.tobytes() == want_scale.tobytes()
        codes, _ = O.quantize(mine, scale, tensor_scheme)
        want_codes, _ = O.quantize(full, want_scale, tensor_scheme)
        assert codes.tobytes() == want_codes[shard.row_start: shard.row_start + shard.rows].tobytes()

        # the same exchange started and awaited separately
        t2 = torch.tensor([local, np.float32(rank)], dtype=torch.float32)
        pending = allreduce_absmax(t2, async_op=True)
        assert pending is not None
        pending.wait()
        assert t2[0].item() == t.item() and t2[1].item() == world - 1

        # per block: no communication; the shard's result is a slice of the whole tensor's
        bcodes, bscale = O.quantize_dynamic(mine, block_scheme)
        wcodes, wscale = O.quantize_dynamic(full, block_scheme)
        assert bcodes.tobytes() == wcodes[shard.row_start: shard.row_start + shard.rows].tobytes()
        assert bscale.tobytes() == wscale[shard.row_start: shard.row_start + shard.rows].tobytes()
        open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_reproduce_the_single_device_result(tmp_path):
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, 96, 256, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_exchange_without_a_process_group_is_a_no_op():
    import torch

    from cubek_b200.shard import allreduce_absmax

    t = torch.tensor([3.5], dtype=torch.float32)
    assert allreduce_absmax(t) is None and allreduce_absmax(t, async_op=True) is None
    assert t.item() == 3.5
