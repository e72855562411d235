"""Benchmark of the quantize + dequantize hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--batch B] [--impl reference]

One step = fused dynamic quantize followed by dequantize of a batch of B distinct synthetic
tensors of the workload (B x inputs > L2, so every step streams from HBM).  Prints ONE JSON line.
Under torchrun every rank processes its own batch (weak scaling, no data-path collective for
per-block schemes); time is the max over ranks, measured with CUDA events.

``--impl reference`` times the CPU oracle (a port of the reference's arithmetic; the reference
itself needs a Rust toolchain and a JIT dependency that are not available) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

DEFAULT_WORKLOAD = "q4_block32_bf16_14336x4096"
METRIC = "quantize+dequantize HBM GB/s"
SPEC_PEAK_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch and per tensor from one ncu capture of each kernel
# on a reduced number of rows (still larger than L2), scaled by rows to the bench tensor; summaries of those
# captures are kept under profiles/.  Reads equal the algorithmic reads; writes come out lower than the
# algorithmic writes because part of the output is still dirty in L2 when the kernel ends.
NCU_TRAFFIC_BYTES = {
    "q4_block32_bf16_14336x4096": {"quantize_dynamic": 145.2e6, "dequantize": 130.4e6},
    "e2m1_block16_f16_8192x4096": {"quantize_dynamic": 84.6e6, "dequantize": 78.3e6},
    "q2_block64_f32_65536x4096": {"quantize_dynamic": 1145.0e6, "dequantize": 941.9e6},
    "q8_block128_bf16_14336x4096": {"quantize_dynamic": 164.9e6, "dequantize": 154.5e6},
    "q8_tensor_bf16_14336x4096": {"quantize_dynamic": 281.3e6},        # absmax pass + quantize pass
}


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_PEAK_GBS, "fallback"


def algorithmic_bytes(workload, rows=None):
    """Bytes one quantize and one dequantize must move for a tensor of this workload."""
    r, c = workload.shape
    if rows is not None:
        r = rows
    n = r * c
    s = workload.scheme
    nscales = 1 if s.level.is_tensor else n // s.level.block_size.as_slice()[-1]
    code_bytes = n * s.value.size_bits() // 8
    in_bytes = n * workload.elem.size
    quant = in_bytes * (2 if s.level.is_tensor else 1) + code_bytes + nscales * s.param.size
    dequant = code_bytes + nscales * s.param.size + in_bytes
    return quant, dequant


class ClockSampler:
    """Samples SM clocks and throttle reasons (read-only NVML queries) while the timed region
    runs.  The timed region lasts milliseconds, so a thread polls NVML every ~2 ms instead of
    going through nvidia-smi's 100 ms loop."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.samples, self.reason_bits, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self.thread = None
        self.nvml = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.gpu_index
            if visible:
                try:
                    index = int(visible.split(",")[self.gpu_index])
                except ValueError:
                    pass
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    def _poll(self):
        nv = self.nvml
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        if not self.nvml:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self._stop.set()
        self.thread.join(timeout=2)
        reasons = sorted(name for name, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_sample_rows(workload, seconds_target=12.0):
    """Rows of the workload tensor the oracle processes in about ``seconds_target`` seconds."""
    import numpy as np
    from oracle import oracle as O

    probe_rows = min(256, workload.shape[0])
    x = cpu_input(workload, probe_rows)
    t0 = time.perf_counter()
    codes, scale = O.quantize_dynamic(x, workload.scheme)
    O.dequantize(codes, scale, workload.scheme, x.dtype)
    dt = max(time.perf_counter() - t0, 1e-6)
    rows = int(probe_rows * seconds_target / dt / 6)   # ~6 passes: warm-up + best of 5
    rows = max(probe_rows, min(rows, workload.shape[0]))
    return rows - rows % 8 if rows >= 8 else rows


def cpu_input(workload, rows):
    import numpy as np
    from cubek_b200.synthetic import generate
    from tests._util import NP_FLOAT, bfloat16
    import torch

    t = generate(workload, "cpu", rows=rows)
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(bfloat16)
    return t.numpy()


def time_cpu(workload, rows, repeats=5):
    """Best-of-``repeats`` seconds of oracle quantize_dynamic + dequantize on ``rows`` rows."""
    from oracle import oracle as O

    x = cpu_input(workload, rows)
    step = cpu_step(workload, x)
    best = float("inf")
    for i in range(repeats + 1):
        t0 = time.perf_counter()
        step()
        dt = time.perf_counter() - t0
        if i > 0:
            best = min(best, dt)
    return best


def cpu_step(workload, x):
    """One oracle round trip (scales, quantize, dequantize) on ``x`` with every output buffer allocated once, as a
    caller of the reference keeps its tensors across iterations."""
    from oracle import oracle as O

    s = workload.scheme
    scale = O.compute_scales(x, s)
    codes, out_scale = O.quantize(x, scale, s)
    restored = O.dequantize(codes, out_scale, s, x.dtype)

    def step():
        O.compute_scales(x, s, out=scale)
        O.quantize(x, scale, s, out=codes, out_scale=out_scale)
        O.dequantize(codes, out_scale, s, x.dtype, out=restored)

    return step


def cpu_baseline(workload):
    from oracle import oracle as O

    O.set_threads(len(os.sched_getaffinity(0)))
    rows = cpu_sample_rows(workload)
    secs = time_cpu(workload, rows)
    q, d = algorithmic_bytes(workload, rows)
    return {"value": round((q + d) / secs / 1e9, 3), "unit": "GB/s", "cores": O.max_threads(), "kind": "port",
            "sample": f"{rows} of {workload.shape[0]} rows of one {workload.name} tensor, best of 5, "
                      f"OpenMP over {O.max_threads()} threads"}


def run_reference(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O

    # torchrun exports OMP_NUM_THREADS=1 to every rank; this arm is the only CPU work of the job and takes
    # every core the process may run on.
    O.set_threads(len(os.sched_getaffinity(0)))
    rows = cpu_sample_rows(workload, seconds_target=max(2.0, 60.0 / max(args.steps + args.warmup, 1)))
    x = cpu_input(workload, rows)
    q, d = algorithmic_bytes(workload, rows)
    step = cpu_step(workload, x)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        step()
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    secs = sum(times) / len(times)
    value = round((q + d) / secs / 1e9, 3)
    sample = (f"{rows} of {workload.shape[0]} rows of one {workload.name} tensor per step "
              f"(one of the {args.batch} tensors of a step of the GPU arm)")
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(secs * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": workload.elem.name.lower(),
        "data": "synthetic", "config": config_of(workload, args),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": O.max_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU port of the reference arithmetic (the oracle); the reference's own CubeCL CPU runtime "
                "cannot be built here (no Rust toolchain, un-vendored JIT dependency)",
    })


def config_of(workload, args):
    s = workload.scheme
    return {"workload": workload.name, "shape": list(workload.shape),
            "batch_tensors_per_step": args.batch,
            "value": s.value.name, "store": s.store.name, "param": s.param.name,
            "level": "tensor" if s.level.is_tensor else f"block{list(s.level.block_size.as_slice())}",
            "distribution": workload.distribution,
            "api": "qk_quantize_dynamic_batch + qk_dequantize_batch (one launch per batch each)",
            "l2": "batch of distinct tensors larger than L2; no flush needed"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_gpu(args, workload):
    import torch
    import torch.distributed as dist

    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from cubek_b200 import _ffi
    from cubek_b200.synthetic import TORCH_DTYPE, generate

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    lib = _ffi.lib()      # raises if the CUDA library is missing: there is no fallback
    if args.no_pdl:
        lib.qk_set_tuning(_ffi.TUNE_PDL, 0)
    for kv in filter(None, args.tune.split(",")):
        key, value = kv.split("=")
        lib.qk_set_tuning(int(key), int(value))
    scheme, elem = workload.scheme, workload.elem
    r, c = workload.shape
    B = args.batch
    tdt = TORCH_DTYPE[elem]
    code_torch = torch.int32 if scheme.store.name == "U32" else torch.uint8
    pdt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[int(scheme.param)]

    xs = [generate(workload, dev, seed_offset=rank * 1000 + i) for i in range(B)]
    codes = [torch.empty(scheme.packed_shape((r, c)), dtype=code_torch, device=dev) for _ in range(B)]
    scales = [torch.empty(scheme.scales_shape((r, c)), dtype=pdt, device=dev) for _ in range(B)]
    outs = [torch.empty((r, c), dtype=tdt, device=dev) for _ in range(B)]
    ws = torch.zeros(4096, dtype=torch.uint8, device=dev)
    H = TensorHandleRef.from_torch
    hx, hc, hs, ho, hws = [H(t) for t in xs], [H(t) for t in codes], [H(t) for t in scales], [H(t) for t in outs], H(ws)
    client = ComputeClient.current()
    # Argument marshalling is done once.  A step is two calls into the C ABI: the fused quantize
    # of the whole batch and the dequantize of the whole batch (one launch each for up to 64
    # tensors).  The same work as one call per tensor is timed afterwards for comparison.
    quant_batch = quantize.PreparedDynamicBatch(client, hx, hc, hs, scheme, elem, hws)
    dequant_batch = dequantize.PreparedBatch(client, hc, ho, hs, scheme, elem)
    quant_calls = [quantize.PreparedDynamic(client, hx[i], hc[i], hs[i], scheme, elem, hws) for i in range(B)]
    dequant_calls = [dequantize.Prepared(client, hc[i], ho[i], hs[i], scheme, elem) for i in range(B)]

    def step():
        quant_batch()
        dequant_batch()

    def step_single():
        for i in range(B):
            quant_calls[i]()
            dequant_calls[i]()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = lib.qk_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    launches = lib.qk_launch_count() - launches_before
    elapsed_ms = start.elapsed_time(stop)

    # Per-kernel durations for the roofline: the same launches, one kind at a time, again
    # bracketed by events on the launch stream (an event between every pair of kernels would
    # serialise launch and execution and time the gap, not the kernel).
    q_avg = timed(quant_batch, args.steps)
    d_avg = timed(dequant_batch, args.steps)
    # Distribution over single steps (an event pair per step; the gaps they add are part of these figures).
    per_step = []
    for _ in range(min(args.steps, 50)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        per_step.append((a, b))
    torch.cuda.synchronize()
    per_step = sorted(a.elapsed_time(b) for a, b in per_step)
    single_ms = timed(step_single, max(args.steps // 2, 1))
    single_q = timed(lambda: [c() for c in quant_calls], max(args.steps // 2, 1)) / B
    single_d = timed(lambda: [c() for c in dequant_calls], max(args.steps // 2, 1)) / B
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())

    # sanity: the last round trip must be within half a quantization step (cheap, outside timing)
    err_ok = bool(torch.isfinite(outs[-1].float()).all().item())

    # ---- end to end through host buffers (pinned), copies inside the timed region ---------------
    e2e = run_e2e(args, workload, dev, local_rank, rank, world, xs)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    q_bytes, d_bytes = algorithmic_bytes(workload)
    total_bytes = (q_bytes + d_bytes) * B * args.steps * world
    value = total_bytes / (elapsed_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    kernels = {
        "quantize_dynamic": {"avg_ms": round(q_avg, 5), "bytes": q_bytes * B, "gbs": round(q_bytes * B / q_avg / 1e6, 1),
                             "tensors_per_launch": B},
        "dequantize": {"avg_ms": round(d_avg, 5), "bytes": d_bytes * B, "gbs": round(d_bytes * B / d_avg / 1e6, 1),
                       "tensors_per_launch": B},
    }
    dom = "quantize_dynamic" if q_avg >= d_avg else "dequantize"
    achieved = kernels[dom]["gbs"]
    traffic = NCU_TRAFFIC_BYTES.get(workload.name, {}).get(dom)
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(elapsed_ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": elem.name.lower(), "data": "synthetic",
        "config": config_of(workload, args),
        "pct_of_spec_peak": round(100 * value / world / SPEC_PEAK_GBS, 1),
        "pct_of_measured_peak": round(100 * value / world / peak, 1),
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic * B if traffic else None,
                     "peak_source": f"{peak_kind} copy bandwidth", "kernels": kernels},
        "single_tensor_calls": {
            "value": round((q_bytes + d_bytes) * B / single_ms / 1e6, 1), "unit": "GB/s (this rank)",
            "ms_per_step": round(single_ms, 4),
            "quantize_dynamic": {"avg_ms": round(single_q, 5), "gbs": round(q_bytes / single_q / 1e6, 1)},
            "dequantize": {"avg_ms": round(single_d, 5), "gbs": round(d_bytes / single_d / 1e6, 1)}},
        "step_ms": {"median": round(per_step[len(per_step) // 2], 4), "best": round(per_step[0], 4),
                    "worst": round(per_step[-1], 4), "samples": len(per_step)},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "finite_output": err_ok,
    }
    if world == 1:
        out["cpu_baseline"] = cpu_baseline(workload)
    emit(out)
    if world > 1:
        dist.destroy_process_group()


def run_weight_set(args, per_tensor: bool, row_sharded: bool = False):
    """BASELINE config 5: the 225 bf16 matrices of a Llama-3-8B-shaped model (15 GB), q8 with
    block-128 scales or per-tensor scales, whole tensors placed round-robin over the ranks (strong
    scaling: the set is fixed).  One step = fused quantize + dequantize of every tensor a rank owns."""
    import torch
    import torch.distributed as dist

    from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef,
                            dequantize, quantize)
    from cubek_b200 import _ffi
    from cubek_b200.shard import assign_round_robin
    from cubek_b200.weights import llama3_8b_shapes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _ffi.lib()
    level = QuantLevel.Tensor if per_tensor else QuantLevel.block([128])
    scheme = QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32, level=level)
    shapes = llama3_8b_shapes()
    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED0004 + rank)
    if row_sharded:
        # every tensor is split by rows over the ranks; the per-tensor absmax needs one all-reduce(MAX)
        from cubek_b200.shard import ShardedPerTensorSet, plan_rows

        my_shapes = [(plan_rows(r, c, world, ElemType.BF16, scheme)[rank].rows, c) for _, r, c in shapes]
        my_shapes = [sh for sh in my_shapes if sh[0] > 0]
    else:
        owned = assign_round_robin([r * c for _, r, c in shapes], world)[rank]
        my_shapes = [(shapes[i][1], shapes[i][2]) for i in owned]
    xs = [(torch.randn(sh, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16) for sh in my_shapes]
    codes = [torch.empty(scheme.packed_shape(x.shape), dtype=torch.int32, device=dev) for x in xs]
    scales = [torch.empty(scheme.scales_shape(x.shape), dtype=torch.float32, device=dev) for x in xs]
    outs = [torch.empty_like(x) for x in xs]
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device=dev)
    H = TensorHandleRef.from_torch
    client = ComputeClient.current()
    if row_sharded:
        absmax = torch.zeros(len(xs), dtype=torch.float32, device=dev)
        qb = ShardedPerTensorSet(client, [H(t) for t in xs], [H(t) for t in codes], [H(t) for t in scales], absmax, scheme,
                                 ElemType.BF16)
    else:
        qb = quantize.PreparedDynamicBatch(client, [H(t) for t in xs], [H(t) for t in codes], [H(t) for t in scales],
                                           scheme, ElemType.BF16, H(ws))
    db = dequantize.PreparedBatch(client, [H(t) for t in codes], [H(t) for t in outs], [H(t) for t in scales], scheme,
                                  ElemType.BF16)

    def step():
        qb()
        db()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    before = lib.qk_launch_count()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    barrier()
    launches = lib.qk_launch_count() - before
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        n = sum(r * c for _, r, c in shapes)
        nscales = len(shapes) if per_tensor else n // 128
        q_bytes = n * 2 * (2 if per_tensor else 1) + n + nscales * 4
        d_bytes = n + nscales * 4 + n * 2
        ms = float(t.item()) / args.steps
        value = (q_bytes + d_bytes) / ms / 1e6
        peak, kind = measured_peak()
        emit({
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "tensors": len(shapes), "elements": n,
                       "level": "tensor" if per_tensor else "block[128]", "value": "Q8S", "store": "U32",
                       "placement": ("every tensor split by rows over the ranks; one all-reduce(MAX) of 225 floats per step"
                                     if row_sharded else "whole tensors, largest first onto the least loaded rank"),
                       "api": "qk_quantize_dynamic_batch + qk_dequantize_batch", "distribution": "normal(0,0.02)"},
            "pct_of_measured_peak": round(100 * value / world / peak, 1), "peak_source": f"{kind} copy bandwidth",
            "gpu_launches": int(launches)})
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, workload, dev, local_rank, rank, world, xs):
    """Same metric through ``qk_roundtrip_host``: inputs in pinned host memory, codes + scales +
    restored tensor read back to pinned host memory, every step."""
    import torch
    import torch.distributed as dist

    from cubek_b200 import TensorHandleRef
    from cubek_b200 import _ffi
    from cubek_b200.synthetic import TORCH_DTYPE

    lib = _ffi.lib()
    scheme, elem = workload.scheme, workload.elem
    r, c = workload.shape
    nb = min(args.batch, args.e2e_batch)
    steps = max(1, min(args.steps, args.e2e_steps))
    tdt = TORCH_DTYPE[elem]
    code_torch = torch.int32 if scheme.store.name == "U32" else torch.uint8
    pdt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[int(scheme.param)]
    h_in = [xs[i].cpu().pin_memory() for i in range(nb)]
    h_codes = [torch.empty(scheme.packed_shape((r, c)), dtype=code_torch).pin_memory() for _ in range(nb)]
    h_scales = [torch.empty(scheme.scales_shape((r, c)), dtype=pdt).pin_memory() for _ in range(nb)]
    h_out = [torch.empty((r, c), dtype=tdt).pin_memory() for _ in range(nb)]
    H = TensorHandleRef.from_torch
    cin = [_ffi.CTensor(H(t)) for t in h_in]
    ccodes = [_ffi.CTensor(H(t)) for t in h_codes]
    cscales = [_ffi.CTensor(H(t)) for t in h_scales]
    cout = [_ffi.CTensor(H(t)) for t in h_out]
    sch = _ffi.c_scheme(scheme)
    need = lib.qk_host_roundtrip_staging_bytes(cin[0].ref(), sch, int(elem))
    staging = torch.empty(int(need), dtype=torch.uint8, device=dev)

    def step():
        for i in range(nb):
            _ffi.check(lib.qk_roundtrip_host(cin[i].ref(), ccodes[i].ref(), cscales[i].ref(), cout[i].ref(), sch,
                                             int(elem), staging.data_ptr(), int(need), local_rank))

    step()   # warm-up (creates the internal streams)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    t = torch.tensor([secs], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs = float(t.item())
    q_bytes, d_bytes = algorithmic_bytes(workload)
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d2h = sum(t.numel() * t.element_size() for ts in (h_codes, h_scales, h_out) for t in ts)
    # the restored tensor must be what the device path produced
    return {"value": round((q_bytes + d_bytes) * nb * steps * world / secs / 1e9, 2), "unit": "GB/s",
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": steps,
            "tensors_per_step": nb, "ms_per_step": round(secs / steps * 1e3, 3),
            "api": "qk_roundtrip_host (pinned host buffers, 4-slot pipelined copies)"}


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Library chatter on stdout (NCCL prints its version there when NCCL_DEBUG asks for it) would sit next to
    the result line: from here on file descriptor 1 goes to stderr, and the one JSON line is written to the
    original stdout by emit()."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(result) -> None:
    line = (json.dumps(result) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, line)


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--batch", type=int, default=8, help="distinct tensors per step")
    ap.add_argument("--e2e-batch", type=int, default=2)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch (A/B runs)")
    ap.add_argument("--tune", default="", help="library tuning keys for A/B runs, e.g. 11=2,8=1 (see qk_set_tuning)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from cubek_b200.synthetic import WORKLOADS

    if args.workload.startswith("llama3_8b_q8_") and args.impl != "reference":
        run_weight_set(args, per_tensor="tensor" in args.workload, row_sharded=args.workload.endswith("_sharded"))
        return
    workload = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, workload)
    else:
        run_gpu(args, workload)


if __name__ == "__main__":
    main()
