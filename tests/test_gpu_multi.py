"""Multi-GPU data path on real devices (needs >= 2 GPUs): one process per GPU over NCCL.
Row shards quantized independently concatenate to the single-GPU result bit for bit, and the
per-tensor path (absmax -> all-reduce(MAX) -> quantize) gives every rank the single-GPU scale."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    import torch.distributed as dist

    from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef,
                            quantize)
    from cubek_b200.shard import plan_rows, quantize_per_tensor_sharded

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        H = TensorHandleRef.from_torch
        rows, cols = 4096, 4096
        g = torch.Generator(device="cuda").manual_seed(99)           # same tensor on every rank
        full = torch.randn((rows, cols), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        full[rows - 1, cols - 1] = 9.5                                # global absmax in the last shard
        client = ComputeClient.current()
        ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
        results = {}
        for name, scheme in (("tensor", QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32)),
                             ("block", QuantScheme(value=QuantValue.Q4S, store=QuantStore.U32,
                                                   level=QuantLevel.block([32])))):
            # single-device result
            codes_full = torch.empty(scheme.packed_shape((rows, cols)), dtype=torch.int32, device="cuda")
            scale_full = torch.empty(scheme.scales_shape((rows, cols)), dtype=torch.float32, device="cuda")
            quantize.launch_dynamic(client, H(full), H(codes_full), H(scale_full), scheme, ElemType.BF16, H(ws))
            # this rank's shard
            sh = plan_rows(rows, cols, world, ElemType.BF16, scheme)[rank]
            mine = full[sh.row_start: sh.row_start + sh.rows]
            codes = torch.empty(scheme.packed_shape((sh.rows, cols)), dtype=torch.int32, device="cuda")
            scale = torch.empty(scheme.scales_shape((sh.rows, cols)), dtype=torch.float32, device="cuda")
            if scheme.level.is_tensor:
                absmax = torch.zeros(1, dtype=torch.float32, device="cuda")
                quantize_per_tensor_sharded(client, H(mine), H(codes), H(scale), absmax, scheme, ElemType.BF16)
                torch.cuda.synchronize()
                assert torch.equal(scale.view(torch.int32), scale_full.view(torch.int32)), "scale differs"
            else:
                quantize.launch_dynamic(client, H(mine), H(codes), H(scale), scheme, ElemType.BF16, H(ws))
                torch.cuda.synchronize()
                assert torch.equal(scale, scale_full[sh.row_start: sh.row_start + sh.rows])
            assert torch.equal(codes, codes_full[sh.row_start: sh.row_start + sh.rows]), f"{name} codes differ"
            results[name] = True
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_row_shards_match_single_gpu(tmp_path):
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 8)
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]


def _nccl_rank_main(rank, world, port, out_dir):
    """`qk_allreduce_max_f32` on a communicator the caller owns (created here through ctypes on the
    NCCL library already loaded in the process)."""
    import ctypes as C

    import torch.distributed as dist

    from cubek_b200 import _ffi

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.zeros(1, device="cuda")                      # CUDA context
        nccl = None
        for line in open("/proc/self/maps"):
            if "libnccl.so" in line:
                nccl = C.CDLL(line.split()[-1])
                break
        if nccl is None:
            nccl = C.CDLL("libnccl.so.2")

        class UniqueId(C.Structure):
            _fields_ = [("internal", C.c_char * 128)]

        uid = UniqueId()
        if rank == 0:
            assert nccl.ncclGetUniqueId(C.byref(uid)) == 0
        t = torch.tensor(list(bytes(uid)), dtype=torch.uint8)
        dist.broadcast(t, 0)
        C.memmove(C.byref(uid), bytes(t.tolist()), 128)
        comm = C.c_void_p()
        nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
        assert nccl.ncclCommInitRank(C.byref(comm), world, uid, rank) == 0
        buf = torch.tensor([1.0 + rank, 100.0 - rank, 0.0, float(rank == world - 1) * 7.5], device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        rc = _ffi.lib().qk_allreduce_max_f32(buf.data_ptr(), buf.numel(), comm, stream)
        assert rc == 0, _ffi.strerror(rc)
        torch.cuda.synchronize()
        assert buf.tolist() == [float(world), 100.0, 0.0, 7.5], buf.tolist()
        nccl.ncclCommDestroy.argtypes = [C.c_void_p]
        nccl.ncclCommDestroy(comm)
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_allreduce_max_entry_point_on_a_caller_owned_communicator(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_nccl_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def _set_rank_main(rank, world, port, out_dir):
    """A set of row-sharded tensors, per-tensor scheme: one all-reduce of all absmax scalars; every rank's
    codes equal the single-device codes of its rows and every rank holds the single-device scales."""
    import torch.distributed as dist

    from cubek_b200 import (ComputeClient, ElemType, QuantScheme, QuantStore, QuantValue, TensorHandleRef, quantize)
    from cubek_b200.shard import ShardedPerTensorSet, plan_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        H = TensorHandleRef.from_torch
        client = ComputeClient.current()
        scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32)
        g = torch.Generator(device="cuda").manual_seed(7)
        shapes = [(512, 1024), (64, 4096), (1024, 256), (8, 128)]
        full = [torch.randn(s, generator=g, device="cuda").to(torch.bfloat16) * (1 + i) for i, s in enumerate(shapes)]
        for i, t in enumerate(full):
            t[-1, -1] = 50.0 + i                      # every global absmax sits in the last rank's rows
        ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
        want_codes = [torch.empty(scheme.packed_shape(s), dtype=torch.int32, device="cuda") for s in shapes]
        want_scale = [torch.empty(1, dtype=torch.float32, device="cuda") for _ in shapes]
        quantize.launch_dynamic_batch(client, [H(t) for t in full], [H(t) for t in want_codes], [H(t) for t in want_scale],
                                      scheme, ElemType.BF16, H(ws))
        plans = [plan_rows(s[0], s[1], world, ElemType.BF16, scheme)[rank] for s in shapes]
        keep = [i for i, p in enumerate(plans) if p.rows > 0]
        mine = [full[i][plans[i].row_start: plans[i].row_start + plans[i].rows] for i in keep]
        codes = [torch.empty(scheme.packed_shape(m.shape), dtype=torch.int32, device="cuda") for m in mine]
        scale = [torch.empty(1, dtype=torch.float32, device="cuda") for _ in mine]
        absmax = torch.zeros(len(mine), dtype=torch.float32, device="cuda")
        # ranks may hold different subsets only if a tensor has fewer row granules than ranks; the
        # all-reduce needs equal lengths, which these shapes guarantee
        assert len(mine) == len(shapes)
        ShardedPerTensorSet(client, [H(t) for t in mine], [H(t) for t in codes], [H(t) for t in scale], absmax, scheme,
                            ElemType.BF16)()
        torch.cuda.synchronize()
        for j, i in enumerate(keep):
            p = plans[i]
            assert torch.equal(scale[j].view(torch.int32), want_scale[i].view(torch.int32)), f"scale {i}"
            assert torch.equal(codes[j], want_codes[i][p.row_start: p.row_start + p.rows]), f"codes {i}"
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_row_sharded_set_with_one_allreduce(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_set_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
