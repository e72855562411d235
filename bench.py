"""Benchmark of the quantize + dequantize hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload ``llama3_8b_q8``: the 225 bf16 matrices of a Llama-3-8B-shaped model (7.5 G elements, 15 GB).
One step quantizes and dequantizes the whole set twice: with q8 codes and one scale per block of 128
(``block128``: no communication) and with q8 codes and one scale per tensor (``tensor``: absmax of the local
shards, ONE all-reduce(MAX) of 225 floats, quantize with the scales every rank derives from the reduced
values).  Under torchrun every tensor is split into contiguous row ranges, one per rank (strong scaling: the
set is fixed); the time of a run is the maximum over the ranks, measured with CUDA events.

The line also carries, under ``configs``, a record for each of the single-tensor configurations (f32 q8 per
tensor, bf16 q4 block 32, f16 fp4 block 16 / 32, f32 q2 block 64), timed the same way on tensors that are
row-sharded over the ranks, as one batched launch per phase and as one call per tensor.

``--workload NAME`` with a name from ``cubek_b200.synthetic.WORKLOADS`` makes that configuration the headline
instead.  ``--case NAME --rows R --iters I [--layout L]`` runs a few launches of one configuration on R rows and
exits: the small case a profiler captures.  ``--impl reference`` times the CPU oracle (a port of the
reference's arithmetic; the reference itself needs a Rust toolchain and a JIT dependency that are not
available) on the host cores.  Prints ONE JSON line on stdout.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

DEFAULT_WORKLOAD = "llama3_8b_q8"
METRIC = "quantize+dequantize HBM GB/s"
SPEC_PEAK_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0
L2_BYTES = 126 << 20
SUB_CONFIGS = ("q8_tensor_f32_4096x4096", "q4_block32_bf16_14336x4096", "e2m1_block16_f16_8192x4096",
               "e2m1_block32_f16_8192x4096", "q2_block64_f32_65536x4096")

# dram__bytes_read.sum + dram__bytes_write.sum of one step of the default workload on ONE GPU, per kernel, from an ncu
# capture of the full-size step (the two counters take one pass per launch; summary and command in the file named
# here).  Row-sharded over N ranks every launch moves 1/N of it.  Reads equal the algorithmic reads; writes fall
# short by the 50-60 MB per launch that are still dirty in L2 when a kernel ends.
NCU_STEP_DRAM_BYTES = {
    "llama3_8b_q8": {"dequantize": 44812.2e6, "quantize_dynamic": 22629.6e6, "absmax": 15010.1e6,
                     "quantize_from_absmax": 22394.0e6},
}
NCU_STEP_DRAM_SOURCE = "profiles/bench_dram_traffic_llama3_8b_q8.md"
# Single-tensor configurations: modelled from a capture of each kernel on a reduced number of rows (still larger than
# L2): traffic(launch) = algorithmic bytes - the write residue still dirty in L2 at kernel end.
NCU_WRITE_RESIDUE_BYTES = {
    ("dequantize", "q8_block128_bf16"): (268.4e6 - 215.1e6, "profiles/dequantize_kernel_q8_block128_bf16.md"),
    ("quantize_dynamic", "q8_block128_bf16"): (138.4e6 - 108.7e6, "profiles/quantize_kernel_q8_block128_bf16.md"),
    ("dequantize", "q4_block32_bf16"): (268.4e6 - 215.0e6, "profiles/dequantize_kernel_q4_block32_bf16.md"),
    ("quantize_dynamic", "q4_block32_bf16"): (83.9e6 - 62.5e6, "profiles/quantize_kernel_q4_block32_bf16.md"),
}


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_PEAK_GBS, "fallback"


def tensor_bytes(n, esize, scheme):
    """Algorithmic bytes (quantize, dequantize) of one tensor of ``n`` elements: the fused quantize reads the
    input once per block scheme and twice per tensor scheme (absmax pass, quantize pass), writes codes and
    scales; the dequantize reads codes and scales and writes the floats."""
    per_tensor = scheme.level.is_tensor
    nscales = 1 if per_tensor else n // math.prod(scheme.level.block_size.as_slice())
    code_bytes = n * scheme.value.size_bits() // 8
    quant = n * esize * (2 if per_tensor else 1) + code_bytes + nscales * scheme.param.size
    dequant = code_bytes + nscales * scheme.param.size + n * esize
    return quant, dequant


def algorithmic_bytes(workload, rows=None):
    r, c = workload.shape
    return tensor_bytes((rows if rows is not None else r) * c, workload.elem.size, workload.scheme)


_SAMPLER_SOURCE = r"""
import os, sys, time
import pynvml
pynvml.nvmlInit()
handle = pynvml.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
out = open(sys.argv[2], "w", buffering=1)
out.write("max %d\n" % pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
parent, born = os.getppid(), time.time()
while os.getppid() == parent and time.time() - born < 1800:   # never outlives the benchmark process
    try:
        out.write("%.6f %d %d\n" % (time.time(), pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM),
                                     int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))))
    except Exception:
        pass
    time.sleep(0.002)
"""


class ClockSampler:
    """Samples SM clocks and throttle reasons (read-only NVML queries) while the timed region runs.  The timed
    region lasts milliseconds, so NVML is polled every ~2 ms instead of going through nvidia-smi's 100 ms loop -
    from a child process: a polling thread inside the benchmark process shares its interpreter lock and its driver
    locks with the thread that launches the kernels, and starved it once steps were down to 2 ms (8 GPUs)."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = self.path = None
        self.t0 = None

    def start(self):
        """Starts the child and waits (a few seconds at most) until it is sampling."""
        import subprocess
        import tempfile

        index = self.gpu_index
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            try:
                index = int(visible.split(",")[self.gpu_index])
            except ValueError:
                pass
        try:
            fd, self.path = tempfile.mkstemp(prefix="qk_clocks_", suffix=".txt")
            os.close(fd)
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_SOURCE, str(index), self.path],
                                         stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
            return
        deadline = time.time() + 10.0
        while time.time() < deadline and self.proc.poll() is None:
            try:
                if os.path.getsize(self.path) > 40:
                    break
            except OSError:
                pass
            time.sleep(0.01)

    def begin(self):
        """Call when the timed region starts: samples taken before are dropped."""
        self.t0 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        t1 = time.time()
        time.sleep(0.005)
        self.proc.terminate()          # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        samples, bits, max_mhz = [], 0, None
        try:
            for line in open(self.path):
                f = line.split()
                if len(f) == 2 and f[0] == "max":
                    max_mhz = float(f[1])
                elif len(f) == 3 and (self.t0 is None or self.t0 <= float(f[0]) <= t1):
                    samples.append(float(f[1]))
                    bits |= int(f[2])
            os.unlink(self.path)
        except (OSError, ValueError):
            pass
        reasons = sorted(name for name, bit in self.REASONS.items() if bits & bit)
        return {"sm_mhz": statistics.median(samples) if samples else None, "sm_max_mhz": max_mhz,
                "reasons": reasons, "samples": len(samples)}


def torch_to_numpy(t):
    """Host NumPy view of a torch tensor, bf16 included (as ml_dtypes.bfloat16)."""
    import ml_dtypes
    import numpy as np
    import torch

    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    if t.dtype == torch.int32:
        return t.numpy().view(np.uint32)
    return t.numpy()


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_workloads(name):
    """The single-tensor configurations whose round trips make one CPU step of workload ``name``: for the
    weight set, the largest layer matrix (gate / up projection, 14336 x 4096 bf16) under both of its schemes."""
    from cubek_b200.synthetic import WORKLOADS

    if name.startswith("llama3_8b_q8"):
        parts = []
        if not name.endswith("_tensor"):
            parts.append(WORKLOADS["q8_block128_bf16_14336x4096"])
        if not name.endswith("_block128"):
            parts.append(WORKLOADS["q8_tensor_bf16_14336x4096"])
        return parts
    return [WORKLOADS[name]]


def cpu_input(workload, rows):
    from cubek_b200.synthetic import generate

    return torch_to_numpy(generate(workload, "cpu", rows=rows))


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


def cpu_plan(name, seconds_per_step):
    """(steps, bytes): the oracle round trips of one CPU step, on as many rows of each tensor as fit the time."""
    parts = cpu_workloads(name)
    steps, total, sample = [], 0, []
    for w in parts:
        probe_rows = min(256, w.shape[0])
        x = cpu_input(w, probe_rows)
        probe = cpu_step(w, x)
        probe()
        t0 = time.perf_counter()
        probe()
        dt = max(time.perf_counter() - t0, 1e-6)
        rows = int(probe_rows * seconds_per_step / len(parts) / dt)
        rows = max(probe_rows, min(rows, w.shape[0]))
        rows -= rows % 8
        steps.append(cpu_step(w, cpu_input(w, rows)))
        q, d = algorithmic_bytes(w, rows)
        total += q + d
        sample.append(f"{rows} of {w.shape[0]} rows of one {w.name} tensor")
    return steps, total, " + ".join(sample)


def cpu_baseline(name):
    from oracle import oracle as O

    O.set_threads(len(os.sched_getaffinity(0)))
    steps, total, sample = cpu_plan(name, seconds_per_step=2.5)
    best = float("inf")
    for i in range(6):
        t0 = time.perf_counter()
        for s in steps:
            s()
        dt = time.perf_counter() - t0
        if i > 0:
            best = min(best, dt)
    return {"value": round(total / best / 1e9, 3), "unit": "GB/s", "cores": O.max_threads(), "kind": "port",
            "sample": f"{sample}; best of 5; OpenMP over {O.max_threads()} threads"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O

    # torchrun exports OMP_NUM_THREADS=1 to every rank; this arm is the only CPU work of the job and takes
    # every core the process may run on.
    O.set_threads(len(os.sched_getaffinity(0)))
    steps, total, sample = cpu_plan(args.workload, seconds_per_step=max(0.5, 60.0 / max(args.steps + args.warmup, 1)))
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        for s in steps:
            s()
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    secs = sum(times) / len(times)
    value = round(total / secs / 1e9, 3)
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(secs * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": reference_dtype(args.workload),
        "data": "synthetic", "config": config_of(args.workload, args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": O.max_threads(), "kind": "port",
                         "sample": sample + " per step"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU port of the reference arithmetic (the oracle); the reference's own CubeCL CPU runtime "
                "cannot be built here (no Rust toolchain, un-vendored JIT dependency)",
    })


def reference_dtype(name):
    return cpu_workloads(name)[0].elem.name.lower()


def config_of(name, world):
    from cubek_b200.synthetic import WORKLOADS
    from cubek_b200.weights import llama3_8b_shapes

    if name.startswith("llama3_8b_q8"):
        shapes = llama3_8b_shapes()
        schemes = [k for k in ("block128", "tensor") if name in ("llama3_8b_q8", "llama3_8b_q8_" + k)]
        return {"workload": name, "tensors": len(shapes), "elements": sum(r * c for _, r, c in shapes),
                "value": "Q8S", "store": "U32", "param": "F32", "schemes_per_step": schemes,
                "distribution": "normal(0,0.02)",
                "placement": (f"every tensor split into contiguous row ranges over {world} ranks" if world > 1
                              else "one GPU holds the whole set"),
                "collective": ("tensor: one all-reduce(MAX) of 225 f32 per step (NCCL); block128: none" if world > 1
                               else "none (one rank)") if "tensor" in schemes else "none",
                "api": "qk_quantize_dynamic_batch, qk_absmax_batch + qk_quantize_from_absmax_batch, qk_dequantize_batch "
                       "(up to 64 tensors per launch)",
                "l2": "per-rank inputs of a step are far larger than L2; no flush needed"}
    w = WORKLOADS[name]
    s = w.scheme
    return {"workload": w.name, "shape": list(w.shape), "value": s.value.name, "store": s.store.name,
            "param": s.param.name, "level": "tensor" if s.level.is_tensor else f"block{list(s.level.block_size.as_slice())}",
            "distribution": w.distribution,
            "placement": f"rows split over {world} ranks" if world > 1 else "one GPU",
            "api": "qk_quantize_dynamic_batch + qk_dequantize_batch (one launch per batch each)"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class Ctx:
    """Process-wide state of the GPU arm: rank, device, library, stream helpers."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        from cubek_b200 import ComputeClient, _ffi

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.lib = _ffi.lib()      # raises if the CUDA library is missing: there is no fallback
        if args.no_pdl:
            self.lib.qk_set_tuning(_ffi.TUNE_PDL, 0)
        for kv in filter(None, args.tune.split(",")):
            key, value = kv.split("=")
            self.lib.qk_set_tuning(int(key), int(value))
        self.client = ComputeClient.current()
        self.flush_buf = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return float(value)
        t = self.torch.tensor([value], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def flush_l2(self):
        """Evicts the step's tensors from L2 with a read-only pass over a 512 MB buffer (reads leave no dirty
        lines behind that the next step would have to write back)."""
        from cubek_b200 import ElemType, TensorHandleRef, quantize

        torch = self.torch
        if self.flush_buf is None:
            self.flush_buf = torch.ones(128 << 20, dtype=torch.float32, device=self.dev)
            self.flush_cell = torch.zeros(1, dtype=torch.float32, device=self.dev)
            self.flush_handle = TensorHandleRef.from_torch(self.flush_buf)
        quantize.absmax(self.client, self.flush_handle, ElemType.F32, self.flush_cell.data_ptr())

    def time_steps(self, fn, steps, flush=False):
        """Milliseconds per call of ``fn`` over ``steps`` calls (device time, this rank).  Without a flush the
        calls run back to back between two events; with one, every call has its own event pair and the
        flush runs between the pairs."""
        torch = self.torch
        if not flush:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / steps
        pairs = []
        for _ in range(steps):
            self.flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            pairs.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in pairs) / steps


class ShardedSet:
    """A set of 2-D tensors of one float type under one scheme, every tensor row-sharded over the ranks; this
    rank's shards with their code, scale and restored buffers, and the prepared calls on them."""

    def __init__(self, ctx: Ctx, shapes, elem, scheme, make_input, seed, codes=None, outs=None):
        from cubek_b200 import TensorHandleRef, dequantize, quantize
        from cubek_b200.shard import ShardedPerTensorSet, plan_rows
        from cubek_b200.synthetic import TORCH_DTYPE

        torch = ctx.torch
        self.ctx, self.scheme, self.elem, self.global_shapes = ctx, scheme, elem, list(shapes)
        self.per_tensor = scheme.level.is_tensor
        plans = [plan_rows(r, c, ctx.world, elem, scheme) for r, c in shapes]
        self.shards = [p[ctx.rank] for p in plans]
        # Tensors every rank holds rows of come first (single-row tensors stay whole on one rank): the same order on
        # every rank, and a rank without the others works on a prefix of it.
        everyone = [all(sh.rows > 0 for sh in p) for p in plans]
        order = sorted(range(len(shapes)), key=lambda i: (not everyone[i], i))
        self.cell_pos = {i: k for k, i in enumerate(order)}                  # cell of tensor i in the absmax vector
        self.index = [i for i in order if self.shards[i].rows > 0]           # tensors this rank holds rows of
        local = [(self.shards[i].rows, shapes[i][1]) for i in self.index]
        tdt = TORCH_DTYPE[elem]
        code_torch = torch.int32 if scheme.store.name == "U32" else torch.uint8
        pdt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[int(scheme.param)]
        self.xs = [make_input(i, sh, seed) for i, sh in zip(self.index, local)]
        self.codes = codes if codes is not None else [torch.empty(scheme.packed_shape(sh), dtype=code_torch, device=ctx.dev)
                                                      for sh in local]
        self.scales = [torch.empty(scheme.scales_shape(sh), dtype=pdt, device=ctx.dev) for sh in local]
        self.outs = outs if outs is not None else [torch.empty(sh, dtype=tdt, device=ctx.dev) for sh in local]
        self.ws = torch.zeros(1 << 16, dtype=torch.uint8, device=ctx.dev)
        H = TensorHandleRef.from_torch
        hx, hc, hs, ho = ([H(t) for t in ts] for ts in (self.xs, self.codes, self.scales, self.outs))
        self.handles = (hx, hc, hs, ho)
        if self.per_tensor:
            # One cell per tensor of the SET, reduced over the ranks in one all-reduce.  A rank whose tensors are a
            # prefix of the vector reduces straight into it (and clears the rest, which only the all-reduce writes);
            # otherwise its cells are scattered into it first.
            self.absmax = torch.zeros(len(shapes), dtype=torch.float32, device=ctx.dev)
            cells_at = [self.cell_pos[i] for i in self.index]
            self.holds_prefix = cells_at == list(range(len(self.index)))
            self.cells = (self.absmax[:len(self.index)] if self.holds_prefix
                          else torch.zeros(len(self.index), dtype=torch.float32, device=ctx.dev))
            self.rest = self.absmax[len(self.index):] if self.holds_prefix and len(self.index) < len(shapes) else None
            self.index_t = torch.tensor(cells_at, dtype=torch.int64, device=ctx.dev)
            self.pending = None
            self.quant_set = ShardedPerTensorSet(ctx.client, hx, hc, hs, self.cells, scheme, elem)
            self.quant = self._quant_per_tensor
        else:
            self.quant = quantize.PreparedDynamicBatch(ctx.client, hx, hc, hs, scheme, elem, H(self.ws))
        self.dequant = dequantize.PreparedBatch(ctx.client, hc, ho, hs, scheme, elem)
        q = d = 0
        for r, c in shapes:
            tq, td = tensor_bytes(r * c, elem.size, scheme)
            q, d = q + tq, d + td
        self.quant_bytes, self.dequant_bytes = q, d          # whole set, all ranks
        self.local_input_bytes = sum(t.numel() * t.element_size() for t in self.xs)

    def quant_begin(self):
        """Per tensor, first half: this rank's absmax cells, then the all-reduce(MAX) is started."""
        from cubek_b200.shard import allreduce_absmax

        self.quant_set.absmax()
        if self.holds_prefix:
            if self.rest is not None:
                self.rest.zero_()
        else:
            self.absmax.zero_()
            self.absmax.index_copy_(0, self.index_t, self.cells)
        self.pending = allreduce_absmax(self.absmax, async_op=True)

    def quant_end(self):
        """Per tensor, second half: the stream waits for the exchange, then the shards are quantized."""
        pending, self.pending = self.pending, None
        if pending is not None:
            pending.wait()
        if not self.holds_prefix:
            self.cells.copy_(self.absmax.index_select(0, self.index_t))
        self.quant_set.quantize()

    def _quant_per_tensor(self):
        self.quant_begin()
        self.quant_end()

    def step(self):
        self.quant()
        self.dequant()

    def phases(self):
        """(name, callable, whole-set algorithmic bytes) of the kernels of one step, in order."""
        if not self.per_tensor:
            return [("quantize_dynamic", self.quant, self.quant_bytes), ("dequantize", self.dequant, self.dequant_bytes)]
        n_in = sum(r * c for r, c in self.global_shapes) * self.elem.size
        return [("absmax", self.quant_set.absmax, n_in),
                ("quantize_from_absmax", self.quant_set.quantize, self.quant_bytes - n_in),
                ("dequantize", self.dequant, self.dequant_bytes)]

    def per_call(self):
        """The same work as one call per tensor (the reference's calling pattern)."""
        from cubek_b200 import TensorHandleRef, dequantize, quantize
        from cubek_b200.shard import quantize_per_tensor_sharded

        ctx, H = self.ctx, TensorHandleRef.from_torch
        hx, hc, hs, ho = self.handles
        n = len(hx)
        deq = [dequantize.Prepared(ctx.client, hc[i], ho[i], hs[i], self.scheme, self.elem) for i in range(n)]
        if self.per_tensor and ctx.world > 1:
            cells = [self.absmax[self.cell_pos[j]: self.cell_pos[j] + 1] for j in self.index]

            def quant_one(i):
                quantize_per_tensor_sharded(ctx.client, hx[i], hc[i], hs[i], cells[i], self.scheme, self.elem)
        else:
            calls = [quantize.PreparedDynamic(ctx.client, hx[i], hc[i], hs[i], self.scheme, self.elem, H(self.ws))
                     for i in range(n)]

            def quant_one(i):
                calls[i]()

        def run():
            for i in range(n):
                quant_one(i)
                deq[i]()

        return run

    def two_call(self):
        """The reference-shaped flow, one tensor per call: ``compute_scales`` (the caller's half: absmax and the
        scale formula, scales typed like the input) then ``launch_ref`` with those scales.  Returns the two
        phases as callables over all local tensors, with their algorithmic bytes over all ranks.  One rank only
        (a sharded per-tensor scale needs the exchange, which ``quantize_per_tensor_sharded`` does)."""
        from cubek_b200 import TensorHandleRef, quantize
        from cubek_b200.synthetic import TORCH_DTYPE

        ctx, H = self.ctx, TensorHandleRef.from_torch
        hx, hc, hs, _ = self.handles
        given = [ctx.torch.empty(self.scheme.scales_shape(x.shape), dtype=TORCH_DTYPE[self.elem], device=ctx.dev) for x in self.xs]
        hg = [H(t) for t in given]
        self._given = given
        scales = [quantize.PreparedScales(ctx.client, hx[i], hg[i], self.scheme, self.elem, H(self.ws)) for i in range(len(hx))]
        quant = [quantize.PreparedRef(ctx.client, hx[i], hc[i], hg[i], hs[i], self.scheme, self.elem) for i in range(len(hx))]
        n_in = sum(r * c for r, c in self.global_shapes) * self.elem.size
        nscales = sum(t.numel() for t in given) * ctx.world
        code_bytes = sum(r * c for r, c in self.global_shapes) * self.scheme.value.size_bits() // 8
        return [("compute_scales", lambda: [c() for c in scales], n_in + nscales * self.elem.size),
                ("quantize_given_scales", lambda: [c() for c in quant],
                 n_in + nscales * self.elem.size + code_bytes + nscales * self.scheme.param.size)]


def check_against_oracle(ctx: Ctx, sset: ShardedSet, rows_per_tensor=4, max_tensors=None):
    """Outside the timed region: whole rows of this rank's shards (first, last and random ones of every tensor)
    are compared bit for bit with the oracle - codes, scales and restored values.  Per tensor, the oracle is
    given the scale that follows from the all-reduced torch absmax, and the ranks compare their scale bits."""
    import numpy as np
    from oracle import oracle as O

    torch = ctx.torch
    s = sset.scheme
    F = O.np_dtype(int(sset.elem))
    lo, hi = s.value.range()
    gen = torch.Generator().manual_seed(1234 + ctx.rank)
    checked_rows = mismatches = 0
    picked = list(range(len(sset.xs)))
    if max_tensors is not None and len(picked) > max_tensors:
        picked = picked[:: max(1, len(picked) // max_tensors)][:max_tensors]
    if sset.per_tensor:
        want_amax = torch.zeros(len(sset.global_shapes), dtype=torch.float32, device=ctx.dev)
        for j, x in zip(sset.index, sset.xs):
            want_amax[j] = x.float().abs().max()
        if ctx.world > 1:
            ctx.dist.all_reduce(want_amax, op=ctx.dist.ReduceOp.MAX)
        want_amax = want_amax.cpu().numpy()
    for k in picked:
        x, codes, scales, out = sset.xs[k], sset.codes[k], sset.scales[k], sset.outs[k]
        rows = x.shape[0]
        extra = torch.randint(0, rows, (max(rows_per_tensor - 2, 0),), generator=gen).tolist()
        pick = torch.tensor(sorted(set([0, rows - 1] + extra)), device=ctx.dev)
        xs = torch_to_numpy(x[pick])
        if sset.per_tensor:
            amax = np.float32(want_amax[sset.index[k]])
            want_scale = np.array([np.float32(2) * amax / np.float32(hi - lo)], dtype=np.float32).astype(F)
            o_codes, o_scale = O.quantize(xs, want_scale, s)
            got_scale = torch_to_numpy(scales).reshape(-1)
        else:
            o_codes, o_scale = O.quantize_dynamic(xs, s)
            got_scale = torch_to_numpy(scales[pick])
        o_restored = O.dequantize(o_codes, o_scale, s, F)
        ok = (got_scale.tobytes() == o_scale.reshape(got_scale.shape).tobytes()
              and torch_to_numpy(codes[pick]).tobytes() == o_codes.tobytes()
              and torch_to_numpy(out[pick]).tobytes() == o_restored.tobytes())
        mismatches += 0 if ok else 1
        checked_rows += int(pick.numel())
    scales_agree = True
    if sset.per_tensor and ctx.world > 1:
        # every rank that holds rows of a tensor must have written the same scale bits
        mine = torch.full((len(sset.global_shapes),), -1, dtype=torch.int64, device=ctx.dev)
        for j, sc in zip(sset.index, sset.scales):
            mine[j] = sc.view(torch.int32).reshape(-1)[0].to(torch.int64)
        gathered = [torch.empty_like(mine) for _ in range(ctx.world)]
        ctx.dist.all_gather(gathered, mine)
        g = torch.stack(gathered)
        held = g >= 0
        ref = torch.where(held, g, torch.full_like(g, -1)).max(dim=0).values
        scales_agree = bool((~held | (g == ref.unsqueeze(0))).all().item())
    t = torch.tensor([mismatches, checked_rows, 0 if scales_agree else 1], dtype=torch.int64, device=ctx.dev)
    if ctx.world > 1:
        ctx.dist.all_reduce(t)
    return {"ok": int(t[0]) == 0 and int(t[2]) == 0, "rows_compared": int(t[1]), "tensors_with_mismatch": int(t[0]),
            "scale_bits_agree_across_ranks": int(t[2]) == 0}


def count_ties(ctx: Ctx, sset: ShardedSet, max_elements=1 << 27):
    """How many quotients x / scale, rounded to the input type as the kernels do, fall on an exact half: the only
    inputs on which the rounding rule of the reference's back end (half to even here, half away from zero in the
    alternative build) changes a code.  Counted with torch on the first tensors of this rank, after a step."""
    torch = ctx.torch
    ties = seen = 0
    for x, sc in zip(sset.xs, sset.scales):
        if seen >= max_elements:
            break
        s = sc.to(x.dtype)
        if not sset.per_tensor:
            s = s.repeat_interleave(sset.scheme.level.block_size.as_slice()[-1], dim=-1)
        q = (x / s).float().abs()
        ties += int(((q - q.floor()) == 0.5).sum().item())
        seen += x.numel()
        del q, s
    t = torch.tensor([ties, seen], dtype=torch.int64, device=ctx.dev)
    if ctx.world > 1:
        ctx.dist.all_reduce(t)
    return {"ties": int(t[0]), "elements_examined": int(t[1]), "fraction": float(t[0]) / max(int(t[1]), 1)}


def llama_input(ctx):
    torch = ctx.torch

    def make(i, shape, seed):
        g = torch.Generator(device=ctx.dev)
        g.manual_seed(0x5EED0004 + 1000003 * (seed + i) + 7919 * ctx.rank)
        return (torch.randn(shape, generator=g, device=ctx.dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    return make


def workload_input(ctx, workload):
    from dataclasses import replace

    from cubek_b200.synthetic import generate

    def make(i, shape, seed):
        return generate(replace(workload, shape=tuple(shape)), ctx.dev, seed_offset=seed + i + 100 * ctx.rank)

    return make


def timed_region(ctx, step, args):
    """Warm-up, barrier, K timed steps between two events, barrier; returns (ms per step as the maximum over the
    ranks, kernel launches of this rank inside the region, clocks sampled on rank 0)."""
    torch = ctx.torch
    # The sampler starts before the warm-up: whatever a rank does between the barrier and its first launch is
    # waited for by every other rank at the first collective of the timed region.
    sampler = ClockSampler(ctx.local_rank)
    if ctx.rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    ctx.barrier()
    sampler.begin()
    before = ctx.lib.qk_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    ctx.barrier()
    launches = ctx.lib.qk_launch_count() - before
    clocks = sampler.stop() if ctx.rank == 0 else None
    ms = ctx.max_over_ranks(start.elapsed_time(stop)) / args.steps
    return ms, int(launches), clocks


def phase_table(ctx, sets, steps):
    """Per kernel kind: launches per call, average launch duration (this rank's events, maximum over the ranks)
    and algorithmic GB/s over all ranks.  One kind at a time between two events (an event between every pair
    of kernels would time the launch gap, not the kernel)."""
    table = {}
    for label, sset in sets:
        for name, fn, nbytes in sset.phases():
            fn()
            ctx.torch.cuda.synchronize()
            before = ctx.lib.qk_launch_count()
            fn()
            launches = int(ctx.lib.qk_launch_count() - before)
            ctx.barrier()
            ms = ctx.max_over_ranks(ctx.time_steps(fn, steps))
            kernels = launches - (1 if name == "absmax" else 0)    # the absmax call counts its memset as a launch
            table[f"{label}.{name}"] = {
                "kernel_launches_per_step": kernels, "avg_launch_ms": round(ms / max(kernels, 1), 5),
                "ms_per_step": round(ms, 5), "bytes_per_step": int(nbytes),
                "bytes_per_launch": int(nbytes / ctx.world / max(kernels, 1)),
                "gbs": round(nbytes / ms / 1e6, 1), "gbs_per_gpu": round(nbytes / ms / 1e6 / ctx.world, 1)}
    return table


def run_weight_set(ctx: Ctx, args):
    from cubek_b200 import ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue
    from cubek_b200.weights import llama3_8b_shapes

    shapes = [(r, c) for _, r, c in llama3_8b_shapes()]
    make = llama_input(ctx)
    sets = []
    block = tensor = None
    if not args.workload.endswith("_tensor"):
        block = ShardedSet(ctx, shapes, ElemType.BF16,
                           QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32, level=QuantLevel.block([128])), make, 0)
        sets.append(("block128", block))
    if not args.workload.endswith("_block128"):
        # the two schemes share inputs, codes and restored buffers (same sizes); only the scales differ
        shared = block
        tensor = ShardedSet(ctx, shapes, ElemType.BF16, QuantScheme(value=QuantValue.Q8S, store=QuantStore.U32),
                            (lambda i, sh, seed, xs=shared.xs: xs[shared.index.index(i)]) if shared else make, 0,
                            codes=shared.codes if shared else None, outs=shared.outs if shared else None)
        sets.append(("tensor", tensor))

    def step():
        # One scheme after the other.  Starting the per-tensor exchange first and running the block scheme's kernels
        # while it is in flight was measured on two GPUs and lost 23 % (10.15 instead of 8.2 ms per step): the
        # collective's resident CTAs take SM slots from the one-wave persistent grids, whose displaced CTAs then run
        # as a second wave.
        for _, s in sets:
            s.step()

    ms, launches, clocks = timed_region(ctx, step, args)
    total_bytes = sum(s.quant_bytes + s.dequant_bytes for _, s in sets)
    # parity right after the timed region: the buffers hold the last step's results of the LAST scheme run on them
    parity = {}
    for label, s in sets:
        s.step()
        ctx.torch.cuda.synchronize()
        parity[label] = check_against_oracle(ctx, s, rows_per_tensor=4)
        parity[label]["rounding_ties"] = count_ties(ctx, s)
    table = phase_table(ctx, sets, max(args.steps // 2, 2))
    per_scheme = {}
    for label, s in sets:
        t = ctx.max_over_ranks(ctx.time_steps(s.step, max(args.steps // 2, 2)))
        per_scheme[label] = {"ms_per_step": round(t, 4), "gbs": round((s.quant_bytes + s.dequant_bytes) / t / 1e6, 1)}
    return {"ms": ms, "launches": launches, "clocks": clocks, "bytes": total_bytes, "parity": parity, "kernels": table,
            "per_scheme": per_scheme, "sets": sets, "dtype": "bf16",
            "traffic_key": "q8_block128_bf16"}


def run_single_config(ctx: Ctx, args, workload, batch, headline):
    """One of the single-tensor configurations: ``batch`` distinct tensors, each row-sharded over the ranks."""
    sset = ShardedSet(ctx, [workload.shape] * batch, workload.elem, workload.scheme, workload_input(ctx, workload),
                      seed=workload.index * 17)
    flush = sset.local_input_bytes < 2 * L2_BYTES
    total = sset.quant_bytes + sset.dequant_bytes
    rec = {}
    if headline:
        ms, launches, clocks = timed_region(ctx, sset.step, args)
        rec.update(ms=ms, launches=launches, clocks=clocks, bytes=total, dtype=workload.elem.name.lower(),
                   traffic_key=workload.name.rsplit("_", 1)[0])
    steps = args.steps if headline else max(args.steps // 2, 3)
    for _ in range(3):
        sset.step()
    ctx.barrier()
    batch_ms = ctx.max_over_ranks(ctx.time_steps(sset.step, steps, flush))
    sset.step()
    ctx.torch.cuda.synchronize()
    parity = check_against_oracle(ctx, sset, rows_per_tensor=6, max_tensors=2)
    parity["rounding_ties"] = count_ties(ctx, sset)
    table = phase_table(ctx, [("batch", sset)], steps) if not flush else {}
    if flush:
        for name, fn, nbytes in sset.phases():
            t = ctx.max_over_ranks(ctx.time_steps(fn, steps, True))
            table[f"batch.{name}"] = {"ms_per_step": round(t, 5), "bytes_per_step": int(nbytes), "gbs": round(nbytes / t / 1e6, 1),
                                      "gbs_per_gpu": round(nbytes / t / 1e6 / ctx.world, 1)}
    per_call = sset.per_call()
    per_call()
    ctx.barrier()
    call_ms = ctx.max_over_ranks(ctx.time_steps(per_call, steps, flush))
    two_call = {}
    if ctx.world == 1:
        for name, fn, nbytes in sset.two_call():
            fn()
            t = ctx.time_steps(fn, steps, flush)
            two_call[name] = {"gbs_per_gpu": round(nbytes / t / 1e6, 1), "ms_per_step": round(t, 5)}
    peak, _ = measured_peak()
    summary = {
        "tensors_per_step": batch, "shape": list(workload.shape),
        "batch": {"gbs": round(total / batch_ms / 1e6, 1), "ms_per_step": round(batch_ms, 4),
                  "frac_of_measured_per_gpu": round(total / batch_ms / 1e6 / ctx.world / peak, 4),
                  "frac_of_spec_per_gpu": round(total / batch_ms / 1e6 / ctx.world / SPEC_PEAK_GBS, 4)},
        "per_call": {"gbs": round(total / call_ms / 1e6, 1), "ms_per_step": round(call_ms, 4),
                     "frac_of_measured_per_gpu": round(total / call_ms / 1e6 / ctx.world / peak, 4),
                     "frac_of_spec_per_gpu": round(total / call_ms / 1e6 / ctx.world / SPEC_PEAK_GBS, 4)},
        "kernels": {k.split(".", 1)[1]: {"gbs_per_gpu": v["gbs_per_gpu"], "ms_per_step": v["ms_per_step"]} for k, v in table.items()},
        "two_call_flow_per_tensor": two_call,
        "l2": "flushed between steps (read-only pass over 512 MB, outside the event pairs)" if flush
              else "per-rank inputs of a step exceed twice the L2",
        "parity_checked": parity["ok"], "rounding_ties": parity["rounding_ties"],
    }
    rec.update(summary=summary, kernels=table, parity={"batch": parity}, sets=[("batch", sset)])
    return rec


def run_e2e(ctx: Ctx, args, sset: ShardedSet, what: str):
    """Same metric through ``qk_roundtrip_host``: this rank's shards in pinned host memory; codes, scales and the
    restored tensor read back to pinned host memory, every step.  Also times the same copies alone (both
    directions at once on two streams, no kernels): the ceiling the host link and host memory set."""
    import ctypes as C

    from cubek_b200 import TensorHandleRef, _ffi

    torch, lib = ctx.torch, ctx.lib
    scheme, elem = sset.scheme, sset.elem
    take = list(range(min(len(sset.xs), args.e2e_tensors)))
    steps = max(1, min(args.steps, args.e2e_steps))
    h_in = [sset.xs[i].cpu().pin_memory() for i in take]
    h_codes = [torch.empty_like(sset.codes[i], device="cpu").pin_memory() for i in take]
    h_scales = [torch.empty_like(sset.scales[i], device="cpu").pin_memory() for i in take]
    h_out = [torch.empty_like(sset.outs[i], device="cpu").pin_memory() for i in take]
    H = TensorHandleRef.from_torch
    cin, ccodes, cscales, cout = (_ffi.CTensorArray([H(t) for t in ts]) for ts in (h_in, h_codes, h_scales, h_out))
    sch = _ffi.c_scheme(scheme)
    need = int(lib.qk_host_roundtrip_staging_bytes_batch(cin.count, cin.array, sch, int(elem)))
    staging = torch.empty(need, dtype=torch.uint8, device=ctx.dev)

    def step():
        _ffi.check(lib.qk_roundtrip_host_batch(cin.count, cin.array, ccodes.array, cscales.array, cout.array, sch,
                                               int(elem), staging.data_ptr(), need, ctx.local_rank))

    def wall(fn, reps):
        fn()
        ctx.barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        torch.cuda.synchronize()
        return ctx.max_over_ranks(time.perf_counter() - t0) / reps

    secs = wall(step, steps)
    # copies alone
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    d_in = [sset.xs[i] for i in take]

    def copies():
        with torch.cuda.stream(up):
            for h, d in zip(h_in, d_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(down):
            for i, k in enumerate(take):
                h_codes[i].copy_(sset.codes[k], non_blocking=True)
                h_scales[i].copy_(sset.scales[k], non_blocking=True)
                h_out[i].copy_(sset.outs[k], non_blocking=True)
        up.synchronize()
        down.synchronize()

    copy_secs = wall(copies, steps)
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d2h = sum(t.numel() * t.element_size() for ts in (h_codes, h_scales, h_out) for t in ts)
    # bytes of the metric for the tensors taken, all ranks
    nbytes = 0
    for i in take:
        r, c = sset.global_shapes[sset.index[i]]
        q, d = tensor_bytes(r * c, elem.size, scheme)
        nbytes += q + d
    return {"value": round(nbytes / secs / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
            "steps": steps, "ms_per_step": round(secs * 1e3, 3), "sample": what,
            "copies_only": {"ms_per_step": round(copy_secs * 1e3, 3), "h2d_gbs_per_rank": round(h2d / copy_secs / 1e9, 1),
                            "d2h_gbs_per_rank": round(d2h / copy_secs / 1e9, 1),
                            "note": "the same host<->device copies with no kernels, both directions at once: the "
                                    "ceiling set by the host link and, with several ranks, by host memory"},
            "fraction_of_copy_ceiling": round(copy_secs / secs, 3),
            "api": "qk_roundtrip_host_batch (pinned host buffers; the slices of all tensors pass through one ring of 4 "
                   "staging slots, copies in both directions overlapping the kernels); bytes per step are this rank's"}


def run_reduce_record(ctx: Ctx, steps):
    """Axis reductions (the caller-side absmax / range step) on a 64 x 4096 x 4096 tensor: algorithmic GB/s (the
    input is read once, the output is small) along the first axis (the contiguous axis is kept and vectorised) and
    along the last, contiguous one."""
    from cubek_b200 import ElemType, TensorHandleRef
    from cubek_b200.reduce import ReduceInst, reduce

    torch, H = ctx.torch, TensorHandleRef.from_torch
    peak, _ = measured_peak()
    out = {}
    for name, tdt, elem in (("f32", torch.float32, ElemType.F32), ("bf16", torch.bfloat16, ElemType.BF16)):
        x = torch.empty((64, 4096, 4096), dtype=tdt, device=ctx.dev).normal_(0.0, 1.0)
        for axis in (0, 2):
            shape = list(x.shape)
            shape[axis] = 1
            y = torch.empty(shape, dtype=tdt, device=ctx.dev)
            for inst in ReduceInst:
                fn = lambda: reduce(ctx.client, H(x), H(y), axis, None, inst, elem)
                fn()
                ms = ctx.time_steps(fn, steps)
                nbytes = x.numel() * x.element_size() + y.numel() * y.element_size()
                out[f"{inst.name}_{name}_axis{axis}"] = {"gbs": round(nbytes / ms / 1e6, 1), "frac_of_measured": round(nbytes / ms / 1e6 / peak, 4)}
        del x
        torch.cuda.empty_cache()
    return {"shape": [64, 4096, 4096], "results": out}


def run_gpu(args):
    from cubek_b200.synthetic import WORKLOADS
    from cubek_b200.weights import llama3_8b_shapes

    ctx = Ctx(args)
    torch = ctx.torch
    peak, peak_kind = measured_peak()
    is_set = args.workload.startswith("llama3_8b_q8")
    if is_set:
        main = run_weight_set(ctx, args)
        shapes = llama3_8b_shapes()[:args.e2e_tensors]
        e2e_set, e2e_what = main["sets"][0][1], (f"the first {len(shapes)} tensors of the set ({len(shapes) / 7:g} layers of q, k, v, o, gate, up, "
                                                 f"down = {sum(r * c for _, r, c in shapes) / 1e6:.0f} M of the 7505 M elements), scheme "
                                                 + main["sets"][0][0])
    else:
        w = WORKLOADS[args.workload]
        main = run_single_config(ctx, args, w, args.batch, headline=True)
        e2e_set, e2e_what = main["sets"][0][1], f"{min(args.e2e_tensors, args.batch)} of the {args.batch} tensors of a step"
    e2e = None if args.no_e2e else run_e2e(ctx, args, e2e_set, e2e_what)

    configs = {}
    if is_set and not args.no_configs:
        del main["sets"]
        e2e_set = None
        torch.cuda.empty_cache()
        for name in SUB_CONFIGS:
            w = WORKLOADS[name]
            rec = run_single_config(ctx, args, w, 2 if w.shape[0] * w.shape[1] >= 1 << 28 else 8, headline=False)
            configs[name] = rec["summary"]
            del rec
            torch.cuda.empty_cache()
        if ctx.world == 1:
            configs["reduce_64x4096x4096"] = run_reduce_record(ctx, 5)

    if ctx.rank == 0:
        value = main["bytes"] / main["ms"] / 1e6
        kernels = main["kernels"]
        # The dominant kernel: phases that run the same kernel (the dequantize of both schemes) count together.
        groups = {}
        for name, rec in kernels.items():
            g = groups.setdefault(name.split(".", 1)[1], {"ms": 0.0, "bytes": 0, "launches": 0, "phases": []})
            g["ms"] += rec["ms_per_step"]
            g["bytes"] += rec["bytes_per_step"]
            g["launches"] += rec.get("kernel_launches_per_step", 0)
            g["phases"].append(name)
        dom = max(groups, key=lambda k: groups[k]["ms"])
        g = groups[dom]
        achieved = round(g["bytes"] / g["ms"] / 1e6 / ctx.world, 1)
        d = {"avg_launch_ms": round(g["ms"] / max(g["launches"], 1), 5) if g["launches"] else None,
             "bytes_per_launch": int(g["bytes"] / ctx.world / max(g["launches"], 1)) if g["launches"] else None}
        traffic, traffic_source = None, None
        step_dram = NCU_STEP_DRAM_BYTES.get(args.workload, {}).get(dom)
        tk = NCU_WRITE_RESIDUE_BYTES.get((dom, main.get("traffic_key", "")))
        if step_dram and g["launches"]:
            traffic, traffic_source = int(step_dram / ctx.world / g["launches"]), NCU_STEP_DRAM_SOURCE
        elif tk and d["bytes_per_launch"]:
            traffic, traffic_source = int(max(d["bytes_per_launch"] - tk[0], 0)), tk[1]
        dom = f"{dom} ({' + '.join(g['phases'])})"
        parity_ok = all(p["ok"] for p in main["parity"].values())
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": ctx.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(main["ms"], 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": main["dtype"], "data": "synthetic",
            "config": config_of(args.workload, ctx.world),
            "pct_of_spec_peak_per_gpu": round(100 * value / ctx.world / SPEC_PEAK_GBS, 1),
            "pct_of_measured_peak_per_gpu": round(100 * value / ctx.world / peak, 1),
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "frac_of_spec": round(achieved / SPEC_PEAK_GBS, 4),
                         "traffic": traffic, "traffic_source": traffic_source,
                         "avg_launch_ms": d.get("avg_launch_ms"), "bytes_per_launch": d.get("bytes_per_launch"),
                         "peak_source": f"{peak_kind} copy bandwidth (a plain copy: a lower bound of the peak, so a "
                                        "fraction may read slightly above 1)",
                         "kernels": kernels},
            "parity_checked": parity_ok, "parity": main["parity"],
            "e2e": e2e, "gpu_launches": main["launches"], "clocks": main["clocks"],
        }
        if "per_scheme" in main:
            out["per_scheme"] = main["per_scheme"]
        if "summary" in main:
            out["headline_config"] = main["summary"]
        if configs:
            out["configs"] = configs
        if ctx.world == 1:
            out["cpu_baseline"] = cpu_baseline(args.workload)
        if ctx.world > 1 and is_set:
            out["limits"] = ("per-rank shards shrink with N while launches per step stay (5 batched launches per scheme "
                             "of up to 64 tensors) and the tensor scheme adds one all-reduce of 225 floats")
        emit(out)
    if ctx.world > 1:
        ctx.dist.destroy_process_group()


def run_case(args):
    """A few fused quantize + dequantize launches of one configuration on a reduced number of rows: the small
    case a profiler captures.  Layouts: contiguous, transposed (`.t()` views of [cols, rows] matrices), slice
    (column slices of matrices 256 columns wider), twocall (compute_scales, quantize with given scales,
    dequantize on contiguous tensors)."""
    import torch

    from cubek_b200 import ComputeClient, TensorHandleRef, dequantize, quantize
    from cubek_b200.synthetic import WORKLOADS, generate

    w = WORKLOADS[args.case]
    rows = args.rows or w.shape[0]
    layout = args.layout
    s, cols = w.scheme, w.shape[1]
    x = generate(w, "cuda", rows=rows)

    def like(t):
        if layout == "transposed":
            return torch.empty((cols, rows), dtype=t.dtype, device="cuda").t()
        if layout == "slice":
            return torch.empty((rows, cols + 256), dtype=t.dtype, device="cuda")[:, 128:128 + cols]
        return torch.empty_like(t)

    if layout in ("transposed", "slice"):
        view = like(x)
        view.copy_(x)
        x = view
    code_dtype = torch.int32 if s.store.name == "U32" else torch.uint8
    codes = torch.empty(s.packed_shape((rows, cols)), dtype=code_dtype, device="cuda")
    scales = torch.empty(s.scales_shape((rows, cols)), dtype=torch.float32, device="cuda")
    out = like(x)
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    H, client = TensorHandleRef.from_torch, ComputeClient.current()
    given = torch.empty(s.scales_shape((rows, cols)), dtype=x.dtype, device="cuda")
    if args.case_tensors > 1:
        # the batched entry points on several tensors of that size (contiguous only): what the set benchmarks launch
        xs = [x] + [generate(w, "cuda", rows=rows, seed_offset=i) for i in range(1, args.case_tensors)]
        cs = [codes] + [torch.empty_like(codes) for _ in xs[1:]]
        ss = [scales] + [torch.empty_like(scales) for _ in xs[1:]]
        os_ = [out] + [torch.empty_like(out) for _ in xs[1:]]
        q = quantize.PreparedDynamicBatch(client, [H(t) for t in xs], [H(t) for t in cs], [H(t) for t in ss], s, w.elem, H(ws))
        d = dequantize.PreparedBatch(client, [H(t) for t in cs], [H(t) for t in os_], [H(t) for t in ss], s, w.elem)
        for _ in range(args.iters):
            q()
            d()
        torch.cuda.synchronize()
        emit({"case": w.name, "rows": rows, "iters": args.iters, "layout": layout, "tensors": args.case_tensors,
              "max_abs_restored": float(os_[-1].float().abs().max())})
        return
    for _ in range(args.iters):
        if layout == "twocall":
            quantize.compute_scales(client, H(x), H(given), s, w.elem, H(ws))
            quantize.launch_ref(client, H(x), H(codes), H(given), H(scales), s, w.elem)
        else:
            quantize.launch_dynamic(client, H(x), H(codes), H(scales), s, w.elem, H(ws))
        dequantize.launch_ref(client, H(codes), H(out), H(scales), s, w.elem)
    torch.cuda.synchronize()
    emit({"case": w.name, "rows": rows, "iters": args.iters, "layout": layout, "max_abs_restored": float(out.float().abs().max())})


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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD,
                    help="llama3_8b_q8 (both schemes), llama3_8b_q8_block128, llama3_8b_q8_tensor, or a single-tensor configuration")
    ap.add_argument("--case-tensors", type=int, default=1, help="with --case: tensors per batched call (1 = the single-tensor calls)")
    ap.add_argument("--batch", type=int, default=8, help="distinct tensors per step of a single-tensor configuration")
    ap.add_argument("--e2e-tensors", type=int, default=28)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-configs", action="store_true", help="skip the records of the single-tensor configurations")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host round trip (launch lists of the device steps only)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch (A/B runs)")
    ap.add_argument("--tune", default="", help="library tuning keys for A/B runs, e.g. 11=2,8=1")
    ap.add_argument("--case", default="", help="run a few launches of this configuration and exit (profiler case)")
    ap.add_argument("--rows", type=int, default=0, help="rows of the --case tensor (default: the configuration's)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--layout", default="contiguous", choices=["contiguous", "transposed", "slice", "twocall"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
