#!/usr/bin/env python
"""Benchmark of the native-provider hot path on B200.

Default workload (the configuration the headline metric is quoted on): GEMM + bias + ReLU,
A[8192,8192] @ W[8192,8192] + bias[8192], BF16 in / FP32 accumulate / BF16 out, captured once
in a CUDA Graph; one step = one graph replay.  Inputs are synthetic and seeded.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gemm_relu|gemm_bias_1024|rmsnorm|softmax|mla|mla_batch_sharded|
                                gemm_decode_square|gemm_decode_up|gemm_decode_down|
                                tp_mlp|tp_mlp_unfused|tp_mlp_noreduce]

Prints one JSON line (rank 0).  With N > 1 (launched under torch.distributed.run) the GEMM,
RMSNorm and softmax workloads run an independent replica on every GPU ("replicas only": the
path has no exchange step); `mla` shards the heads and `mla_batch_sharded` the sequences over
the ranks, again without an exchange; the `tp_mlp*` workloads shard a SwiGLU MLP N ways with
the sum all-reduce over NVLink peer memory.  Timing is the maximum over ranks and `value` is
the aggregate.
"""
import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REPO / "trinity-be_b200"))

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024

# DRAM bytes per launch of the dominant kernel from an ncu capture (profiles/), per workload.
# None until a capture exists for that workload.  Sources: profiles/*.md.
NCU_TRAFFIC_BYTES = {
    "gemm_relu": 1.127e9,
    "gemm_bias_1024": None,
    "rmsnorm": 4.84e8,
    "softmax": 4.83e8,
    "mla": 3.15e8,
    "mla_batch_sharded": None,
    "gemm_decode_square": None,
    "gemm_decode_up": None,
    "gemm_decode_down": None,
    "tp_mlp": None,
    "tp_mlp_unfused": None,
    "tp_mlp_noreduce": None,
}


def peaks():
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"],
                "bf16_tflops_sustained": data["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: clocks are reported as unknown
            self.nvml = None

    def _loop(self):
        n = self.nvml
        names = {
            getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nvml:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        ordered = sorted(self.samples)
        return {"sm_mhz": ordered[len(ordered) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(ordered)}


# ---------------------------------------------------------------- workloads
class Workload:
    """name, metric, unit, bound, work per step, device step, end-to-end step, CPU sample."""


def make_workload(name, device, world=None):
    from oracle import workloads as wl  # seeded input generators only (no oracle math here)
    from trinity_lowering import kernels as k

    w = Workload()
    w.name = name
    w.world = world
    w.strong = False
    w.no_graph = False
    on_gpu = device.type == "cuda"

    def pin(t):
        return t.pin_memory() if on_gpu else t
    if name in ("gemm_relu", "gemm_bias_1024"):
        if name == "gemm_relu":
            m = n = kk = 8192
            a, wt, bias = wl.gemm_inputs(m, n, kk, 1235, "normal")
            act = k.ACT_RELU
            w.label = "gemm_bias_relu A[8192,8192]@W[8192,8192]+bias[8192], CUDA-Graph replay"
        else:
            m = n = kk = 1024
            a, wt, bias = wl.gemm_inputs(m, n, kk, 1234, "uniform")
            act = k.ACT_NONE
            w.label = ("gemm_bias A[1024,1024]@B[1024,1024]+bias[1024], CUDA-Graph replay of 32 launches "
                       "over 32 operand sets")
        w.metric, w.unit, w.bound, w.dtype = "bf16_gemm_epilogue_tflops", "TFLOP/s", "tensor", "bf16"
        w.work = 2.0 * m * n * kk / 1e12                       # TFLOP per step
        w.alg_bytes = (m * kk + kk * n + n + m * n) * 2
        host = [pin(t) for t in (a, wt, bias)]
        host_out = pin(torch.empty((m, n), dtype=torch.bfloat16))
        dev = [t.to(device) for t in (a, wt, bias)]
        out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        w.kernels_per_step = 1
        w.l2_note, w.flush = "inputs larger than L2", False
        # A single small GEMM would be timed with one event pair per launch, which measures the
        # launch path rather than the kernel.  The small configuration therefore runs 32 launches
        # per step over 32 operand sets (32 x 6.3 MB > L2), back to back.
        sets = 1 if (m * kk + kk * n) * 2 > L2_BYTES or not on_gpu else 32
        rotating = [(dev[0].clone(), dev[1].clone(), torch.empty_like(out)) for _ in range(sets - 1)]
        rotating.append((dev[0], dev[1], out))
        w.kernels_per_step = sets
        w.work *= sets
        w.e2e_work = w.work / sets
        w.alg_bytes *= sets

        def device_step():
            for a_i, w_i, out_i in rotating:
                k.gemm(a_i, w_i, bias=dev[2], bias_mode=k.BIAS_COL_VECTOR, activation=act, out=out_i)

        # End to end goes through the public path: plan -> emit -> compile -> load -> prepare,
        # then per step host->device copies, execution.run(), device->host copy.
        api = {}

        def e2e_step():
            if not api:
                import trinity_lowering as tl
                from trinity_lowering import plans
                artifact = tl.compile(tl.emit(plans.gemm_bias(m, n, kk, "relu" if act else None)))
                api["module"] = tl.load(artifact, device)
                artifact.close()
                api["execution"] = api["module"].prepare({"A": dev[0], "W": dev[1], "bias": dev[2]}, out=out)
            for src, dst in zip(host, dev):
                dst.copy_(src, non_blocking=True)
            api["execution"].run()
            host_out.copy_(out, non_blocking=True)

        w.h2d = sum(t.numel() * 2 for t in host)
        w.d2h = host_out.numel() * 2
        # host cost of one launch through the public API (runtime checks + trinity_launch), no copies
        w.host_launch = lambda: api["execution"].run()

        def cpu_sample(threads, budget_s):
            torch.set_num_threads(threads)
            af, wf, bf = a.float(), wt.float(), bias.float()
            rows = min(m, 256)
            t0 = time.perf_counter()
            torch.relu(torch.addmm(bf, af[:rows], wf)) if act else torch.addmm(bf, af[:rows], wf)
            probe = max(time.perf_counter() - t0, 1e-4)
            rows = int(min(m, max(256, rows * budget_s / probe / 2)))
            t0 = time.perf_counter()
            y = torch.addmm(bf, af[:rows], wf)
            if act:
                y = torch.relu(y)
            y = y.bfloat16()
            dt = time.perf_counter() - t0
            return 2.0 * rows * n * kk / 1e12 / dt, f"{rows} of {m} rows, torch CPU FP32 addmm" + \
                ("+relu" if act else ""), dt

    elif name in ("rmsnorm", "softmax"):
        rows, cols = 32768, 4096
        x, g = wl.rownorm_inputs(rows, cols, 1236)
        w.label = f"{name} X[32768,4096] bf16" + (", gain[4096], eps 1e-6" if name == "rmsnorm" else "")
        w.metric, w.unit, w.bound, w.dtype = f"{name}_hbm_gbs", "GB/s", "hbm", "bf16"
        w.alg_bytes = rows * cols * 4 + (cols * 2 if name == "rmsnorm" else 0)
        w.work = w.alg_bytes / 1e9
        host_x = pin(x)
        host_y = pin(torch.empty_like(x))
        xd, gd = x.to(device), g.to(device)
        yd = torch.empty_like(xd)
        w.kernels_per_step = 1
        w.l2_note, w.flush = "inputs larger than L2", False

        def device_step():
            if name == "rmsnorm":
                k.rmsnorm(xd, gd, 1e-6, out=yd)
            else:
                k.softmax(xd, out=yd)

        def e2e_step():
            xd.copy_(host_x, non_blocking=True)
            device_step()
            host_y.copy_(yd, non_blocking=True)

        w.h2d, w.d2h = x.numel() * 2, x.numel() * 2

        def cpu_sample(threads, budget_s):
            torch.set_num_threads(threads)
            sample = x[:4096]
            t0 = time.perf_counter()
            if name == "rmsnorm":
                wl.rmsnorm_oracle(sample, g, 1e-6)
            else:
                wl.softmax_oracle(sample)
            dt = time.perf_counter() - t0
            return sample.numel() * 4 / 1e9 / dt, "4096 of 32768 rows, CPU oracle (FP32 torch)", dt

    elif name in ("gemm_decode_square", "gemm_decode_up", "gemm_decode_down"):
        # Decode-time GEMMs: 16 tokens against a large weight, which the kernel streams once.
        m = 16
        kk, n = {"gemm_decode_square": (8192, 8192), "gemm_decode_up": (8192, 28672),
                 "gemm_decode_down": (28672, 8192)}[name]
        a, wt, _ = wl.gemm_inputs(m, n, kk, 1240, "normal")
        w.label = f"gemm A[16,{kk}]@W[{kk},{n}] bf16 (decode-time shape)"
        w.metric, w.unit, w.bound, w.dtype = "gemm_decode_hbm_gbs", "GB/s", "hbm", "bf16"
        w.alg_bytes = (m * kk + kk * n + m * n) * 2
        w.work = w.alg_bytes / 1e9
        host_a, host_w = pin(a), pin(wt)
        ad, wd = a.to(device), wt.to(device)
        out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        host_out = pin(torch.empty((m, n), dtype=torch.bfloat16))
        w.kernels_per_step = 1
        w.l2_note, w.flush = "inputs larger than L2", False

        def device_step():
            k.gemm(ad, wd, out=out)

        def e2e_step():
            ad.copy_(host_a, non_blocking=True)
            wd.copy_(host_w, non_blocking=True)
            device_step()
            host_out.copy_(out, non_blocking=True)

        w.h2d, w.d2h = (a.numel() + wt.numel()) * 2, out.numel() * 2

        def cpu_sample(threads, budget_s):
            torch.set_num_threads(threads)
            af, wf = a.float(), wt.float()
            t0 = time.perf_counter()
            (af @ wf).bfloat16()
            dt = time.perf_counter() - t0
            return w.alg_bytes / 1e9 / dt, "whole GEMM, torch CPU FP32 matmul", dt

    elif name in ("mla", "mla_batch_sharded"):
        batch, heads, seq, d_qk, d_v = 64, 128, 4096, 576, 512
        # On N GPUs "mla" shards the heads N ways and every rank holds the whole cache (the cache
        # is shared by all heads, so tensor-parallel ranks replicate it); "mla_batch_sharded"
        # gives each rank batch/N sequences with all their heads.  Neither has a collective.
        ranks = int(os.environ.get("WORLD_SIZE", "1")) if on_gpu else 1
        mine = int(os.environ.get("RANK", "0")) if on_gpu else 0
        q, cache = wl.mla_inputs(batch, heads, seq, d_qk, 1237)
        if ranks > 1 and name == "mla":
            share = heads // ranks
            q = q[:, mine * share:(mine + 1) * share].contiguous()
            heads = share
            w.parallelism = f"{ranks}-way head sharding, cache replicated, no collective"
        elif ranks > 1:
            share = batch // ranks
            q = q[mine * share:(mine + 1) * share].contiguous()
            cache = cache[mine * share:(mine + 1) * share].contiguous()
            batch = share
            w.parallelism = f"{ranks}-way batch sharding, no collective"
            w.strong = True
        scale = 1.0 / math.sqrt(192.0)
        w.label = f"mla_decode batch{batch} x {heads} heads per GPU, cache[{batch},4096,576] bf16"
        w.metric, w.unit, w.bound, w.dtype = "mla_decode_hbm_gbs", "GB/s", "hbm", "bf16"
        w.alg_bytes = (q.numel() + cache.numel() + batch * heads * d_v) * 2
        w.work = w.alg_bytes / 1e9
        host_q, host_c = pin(q), pin(cache)
        qd, cd = q.to(device), cache.to(device)
        od = torch.empty((batch, heads, d_v), dtype=torch.bfloat16, device=device)
        host_o = pin(torch.empty_like(od, device="cpu"))
        splits = k.mla_default_splits(batch, seq) if on_gpu else 1
        scratch = torch.empty(max(256, k.mla_scratch_bytes(batch, heads, d_v, splits)) if on_gpu
                              else 256, dtype=torch.uint8, device=device)
        w.kernels_per_step = 1 if splits == 1 else 2
        w.l2_note, w.flush = "inputs larger than L2", False

        def device_step():
            k.mla_decode(qd, cd, scale, kv_splits=0, out=od, scratch=scratch)

        def e2e_step():
            qd.copy_(host_q, non_blocking=True)
            cd.copy_(host_c, non_blocking=True)
            device_step()
            host_o.copy_(od, non_blocking=True)

        w.h2d, w.d2h = (q.numel() + cache.numel()) * 2, od.numel() * 2

        def cpu_sample(threads, budget_s):
            torch.set_num_threads(threads)
            t0 = time.perf_counter()
            wl.mla_oracle(q, cache, scale, d_v, batches=[0, 1])
            dt = time.perf_counter() - t0
            return (w.alg_bytes * 2 / batch) / 1e9 / dt, "2 of 64 sequences, CPU oracle", dt
    elif name in ("tp_mlp", "tp_mlp_unfused", "tp_mlp_noreduce"):
        # Tensor-parallel SwiGLU MLP: total work fixed, sharded over the ranks (strong scaling).
        m, d_model, d_ff = 16384, 8192, 28672
        w.label = ("tp_swiglu_mlp X[16384,8192], W_gate/W_up[8192,28672] column-sharded, "
                   "W_down[28672,8192] row-sharded" + {
                       "tp_mlp": ", all-reduce fused into the down GEMM",
                       "tp_mlp_unfused": ", separate all-reduce kernel",
                       "tp_mlp_noreduce": ", NO all-reduce (timing baseline, result incomplete)"}[name])
        w.metric, w.unit, w.bound, w.dtype = "tp_mlp_tflops", "TFLOP/s", "tensor", "bf16"
        w.total_work = 3 * 2.0 * m * d_model * d_ff / 1e12
        w.alg_bytes = (m * d_model * 2 + 3 * d_model * d_ff + m * d_ff * 2) * 2
        w.flush, w.l2_note = False, "inputs larger than L2"
        w.strong = True
        w.no_graph = True     # the all-reduce epoch is a launch argument
        if on_gpu:
            from trinity_lowering.tp_mlp import TensorParallelMLP
            world = w.world
            size = world.size if world is not None else 1
            rank = world.rank if world is not None else 0
            shard = d_ff // size
            g = torch.Generator(device=device)
            g.manual_seed(1238 + rank)
            def normal(shape, std):
                return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).bfloat16()
            gx = torch.Generator(device=device)
            gx.manual_seed(1238)
            xd = (torch.randn((m, d_model), generator=gx, device=device)).bfloat16()
            wg = normal((d_model, shard), 1.0 / math.sqrt(d_model))
            wu = normal((d_model, shard), 1.0 / math.sqrt(d_model))
            wd = normal((shard, d_model), 1.0 / math.sqrt(d_ff))
            mlp = TensorParallelMLP(world, m, d_model, d_ff, wg, wu, wd,
                                    fused={"tp_mlp": True, "tp_mlp_unfused": False}.get(name))
            host_x = xd.cpu().pin_memory()
            host_y = torch.empty((m, d_model), dtype=torch.bfloat16).pin_memory()
            w.work = w.total_work / size
            w.kernels_per_step = 2 if (size == 1 or name == "tp_mlp") else 3

            def device_step():
                mlp.forward(xd)

            def e2e_step():
                xd.copy_(host_x, non_blocking=True)
                mlp.forward(xd)
                host_y.copy_(mlp.output, non_blocking=True)

            w.h2d, w.d2h = xd.numel() * 2, m * d_model * 2
        else:
            device_step = e2e_step = None

        def cpu_sample(threads, budget_s):
            torch.set_num_threads(threads)
            rows = 128
            gcpu = torch.Generator().manual_seed(7)
            xs = torch.randn((rows, d_model), generator=gcpu)
            a = torch.randn((d_model, d_ff), generator=gcpu) / math.sqrt(d_model)
            bm = torch.randn((d_model, d_ff), generator=gcpu) / math.sqrt(d_model)
            c = torch.randn((d_ff, d_model), generator=gcpu) / math.sqrt(d_ff)
            t0 = time.perf_counter()
            gate = xs @ a
            h = (xs @ bm) * (gate * torch.sigmoid(gate))
            (h.bfloat16().float() @ c).bfloat16()
            dt = time.perf_counter() - t0
            return 3 * 2.0 * rows * d_model * d_ff / 1e12 / dt, f"{rows} of {m} rows, torch CPU FP32", dt
    else:
        raise SystemExit(f"unknown workload {name}")
    w.device_step, w.e2e_step, w.cpu_sample = device_step, e2e_step, cpu_sample
    return w


def flush_l2(buffer):
    buffer.zero_()


def timed(step, steps, flush_buffer, stream):
    """CUDA-event time (ms) of `steps` calls on `stream`; L2 flushes are excluded from the sum."""
    if flush_buffer is None:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(steps):
            step()
        stop.record(stream)
        stop.synchronize()
        return start.elapsed_time(stop)
    total = 0.0
    events = []
    for _ in range(steps):
        flush_l2(flush_buffer)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        step()
        b.record(stream)
        events.append((a, b))
    torch.cuda.synchronize()
    for a, b in events:
        total += a.elapsed_time(b)
    return total


def run_reference(args, rank, world):
    """The reference's CPU evaluation of the path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    w = make_workload(args.workload, torch.device("cpu"))
    values = []
    sample = ""
    for i in range(args.warmup + args.steps):
        value, sample, _ = w.cpu_sample(threads, budget_s=2.0)
        if i >= args.warmup:
            values.append(value)
    value = sum(values) / len(values)
    line = {
        "impl": "reference", "metric": w.metric, "value": value, "unit": w.unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": w.label, "note": "reference plan evaluation on host cores"},
        "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="gemm_relu")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-graph", action="store_true",
                        help="launch directly instead of replaying a CUDA Graph (for profilers)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        # The CPU workload construction needs no GPU; ranks other than 0 do no work.
        if rank == 0:
            run_reference(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    from trinity_lowering import kernels as k
    k.library()
    world_obj = None
    if distributed and args.workload.startswith("tp_mlp"):
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        from trinity_lowering.world import World
        world_obj = World.from_torchrun(timeout=120.0)
    w = make_workload(args.workload, device, world_obj)
    if w.no_graph:
        args.no_graph = True
    stream = torch.cuda.Stream(device=device)
    flush_buffer = (torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device) if w.flush else None)

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
            torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        # Capture one step (all launches of the hot path) in a CUDA Graph, as the configuration asks.
        w.device_step()
        torch.cuda.synchronize()
        if args.no_graph:
            replay = w.device_step
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                w.device_step()
            replay = graph.replay
        for _ in range(args.warmup):
            replay()
        barrier()
        launches_before = k.launch_count()
        with ClockSampler(local_rank) as clocks:
            ms = timed(replay, args.steps, flush_buffer, stream)
        barrier()
        # end to end: host buffers in, result out, every step
        for _ in range(3):
            w.e2e_step()
        barrier()
        e2e_steps = max(3, min(args.steps, 10))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(e2e_steps):
            w.e2e_step()
        stop.record(stream)
        stop.synchronize()
        e2e_ms = start.elapsed_time(stop)
        barrier()
        launches_after = k.launch_count()
        host_launch_us = None
        if getattr(w, "host_launch", None) is not None:
            calls = 100
            t0 = time.perf_counter()
            for _ in range(calls):
                w.host_launch()
            host_launch_us = (time.perf_counter() - t0) / calls * 1e6
            barrier()
    launches = launches_after - launches_before
    if not args.no_graph:
        launches += args.steps * w.kernels_per_step  # replays do not pass through the library

    if distributed:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()

    status = k.device_status()
    if status:
        raise SystemExit(f"device status word {status:#x}: a bounded in-kernel wait gave up")

    pk = peaks()
    per_step_ms = ms / args.steps
    value = world * w.work * args.steps / (ms / 1e3)
    e2e_value = world * (getattr(w, "e2e_work", None) or w.work) * e2e_steps / (e2e_ms / 1e3)
    scaling = "strong" if w.strong else "weak"
    achieved = w.work / (per_step_ms / 1e3)            # per GPU, dominant kernel
    if w.bound == "tensor":
        long_run = ms > 1000.0
        peak = pk["bf16_tflops_sustained"] if long_run else pk["bf16_tflops"]
        peak_note = ("sustained" if long_run else "burst") + " cuBLAS bf16, " + pk["source"]
        roof_unit = "TFLOP/s"
    else:
        peak, peak_note, roof_unit = pk["hbm_gbs"], "copy bandwidth, " + pk["source"], "GB/s"
    line = {
        "metric": w.metric, "value": value, "unit": w.unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step_ms, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": w.label, "l2": w.l2_note,
                   "parallelism": (getattr(w, "parallelism", None) or
                                   ("single GPU" if world == 1 else
                                    f"tp{world} over NVLink peer memory" if w.strong else "replicas only")),
                   "launch": "direct" if args.no_graph else "CUDA Graph replay"},
        "roofline": {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": roof_unit,
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(w.name),
                     "algorithmic_bytes": w.alg_bytes, "peak_kind": peak_note},
        "e2e": {"value": e2e_value, "unit": w.unit, "h2d_bytes_per_step": w.h2d,
                "d2h_bytes_per_step": w.d2h, "steps": e2e_steps},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
    }
    if host_launch_us is not None:
        line["host_launch_us"] = host_launch_us   # public-API launch, host side only
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, sample, _ = w.cpu_sample(threads, budget_s=10.0)
        line["cpu_baseline"] = {"value": v, "unit": w.unit, "cores": threads, "kind": "port",
                                "sample": sample}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
