#!/usr/bin/env python
"""Benchmark of the native-provider hot path on B200.

Default workload at every GPU count: the tensor-parallel SwiGLU MLP
Y = (silu(X Wg) * (X Wu)) Wd with X[16384,8192], Wg/Wu[8192,28672] column-sharded and
Wd[28672,8192] row-sharded over the GPUs, BF16 in / FP32 accumulate / BF16 out.  One step = one
forward pass: the gated GEMM and the row-parallel down GEMM whose epilogue sums the partial
outputs across GPUs over NVLink peer memory (one GPU: the same two GEMMs without an exchange).
Total work is fixed, so the scaling is strong.  Inputs are synthetic and seeded.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload tp_mlp|tp_mlp_unfused|tp_mlp_noreduce|gemm_relu|gemm_bias_1024|
                                rmsnorm|softmax|mla|mla_batch_sharded|
                                gemm_decode_square|gemm_decode_up|gemm_decode_down|ffn_block_decode|
                                gemm_shape --shape M,N,K --epilogue none|relu|gated]
                    [--no-configs] [--no-cpu-baseline] [--no-graph]

Prints one JSON line (rank 0).  With the default workload the line also carries a "configs" block:
on one GPU the other benchmark configurations (GEMM+bias 1024^3, GEMM+bias+ReLU 8192^3 over 100
graph replays, RMSNorm, softmax, MLA decode, the three decode-time GEMMs of 16 rows and the whole
decode-time feed-forward block as one plan through the public API), on N GPUs the
head-sharded and the batch-sharded MLA decode.  Every workload's result is checked once, outside the timed region, on sampled rows
against a float64 evaluation on the host ("parity").  Timing is by CUDA events, the maximum over
ranks, and `value` is the aggregate over all GPUs.
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
SHAPE, EPILOGUE = (4096, 4096, 4096), "none"   # of the gemm_shape workload (--shape, --epilogue)
REL_L2_BOUND, MAX_ABS_BOUND = 1e-2, 2e-2   # the path's stated floating-point bar

# DRAM bytes per launch of the dominant kernel from an ncu capture (profiles/), per workload.
# None where no capture exists for that workload.  Sources: profiles/*.md.
NCU_TRAFFIC_BYTES = {
    "gemm_relu": 1.206e9,
    "gemm_bias_1024": None,
    "rmsnorm": 4.84e8,
    "softmax": 4.83e8,
    "mla": 3.16e8,
    "mla_batch_sharded": None,
    "gemm_decode_square": 1.39e8,
    "gemm_decode_up": None,
    "gemm_decode_down": None,
    "tp_mlp": 1.34e10,     # the gated GEMM (two thirds of the step), scaled from a quarter-size capture
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
                "sm_mhz_min": ordered[0], "reasons": sorted(self.reasons), "samples": len(ordered)}


# ---------------------------------------------------------------- parity (float64 on the host)
def error_figures(actual, expected, rows, ulps=1):
    """rel-L2 and max-abs of a BF16 result against a float64 expectation of the same rows.  The
    max-abs bound is 2e-2 for outputs of order one; where outputs exceed |y| = 4 the rounding of
    the BF16 result alone is larger than that, and the bound is one BF16 ulp of the largest
    output (stated in the line as max_abs_bound).  A chain of kernels with BF16 intermediates
    passes `ulps` = 2: a one-ulp flip of an intermediate moves the next product's result."""
    a, e = actual.double(), expected.double()
    rel = ((a - e).norm() / e.norm().clamp_min(1e-300)).item()
    worst = (a - e).abs().max().item()
    top = e.abs().max().item()
    bound = max(MAX_ABS_BOUND, ulps * 2.0 ** (math.floor(math.log2(top)) - 7) if top > 0 else 0.0)
    return {"rel_l2": rel, "max_abs": worst, "max_abs_bound": bound, "rows": int(rows),
            "ok": bool(rel <= REL_L2_BOUND and worst <= bound)}


def sampled_rows(total, count):
    step = max(1, total // count)
    rows = list(range(0, total, step))[:count]
    if rows[-1] != total - 1:
        rows.append(total - 1)
    return torch.tensor(rows, dtype=torch.long)


def swiglu_partial_float64(xs, w_gate, w_up, w_down, block=4096):
    """(silu(xs Wg) * (xs Wu)) Wd for a few rows in float64, the hidden activation rounded to
    BF16 once as the plan stores it.  Weights are device tensors; they are brought over in
    column blocks so the host never holds a float64 copy of a whole weight."""
    xs = xs.double()
    y = torch.zeros((xs.shape[0], w_down.shape[1]), dtype=torch.float64)
    for c0 in range(0, w_gate.shape[1], block):
        c1 = min(c0 + block, w_gate.shape[1])
        gate = xs @ w_gate[:, c0:c1].cpu().double()
        up = xs @ w_up[:, c0:c1].cpu().double()
        hidden = (up * (gate * torch.sigmoid(gate))).float().bfloat16().double()
        y += hidden @ w_down[c0:c1].cpu().double()
    return y


# ---------------------------------------------------------------- workloads
class Workload:
    """name, metric, unit, bound, work per step, device step, end-to-end slots, checks."""

    parallelism = None
    strong = False
    no_graph = False
    replays_graph = False      # the device step itself replays a graph captured by the package
    host_launch = None
    e2e_work = None


def workload_label(name):
    """Description of a workload that does not depend on the arm or on the GPU count."""
    mlp = ("tp_swiglu_mlp X[16384,8192], W_gate/W_up[8192,28672] column-sharded, "
           "W_down[28672,8192] row-sharded")
    return {
        "gemm_relu": "gemm_bias_relu A[8192,8192]@W[8192,8192]+bias[8192], CUDA-Graph replay",
        "gemm_bias_1024": ("gemm_bias A[1024,1024]@B[1024,1024]+bias[1024], CUDA-Graph replay of 32 "
                           "launches over 32 operand sets"),
        "rmsnorm": "rmsnorm X[32768,4096] bf16, gain[4096], eps 1e-6",
        "softmax": "softmax X[32768,4096] bf16",
        "gemm_decode_square": "gemm A[16,8192]@W[8192,8192] bf16 (decode-time shape)",
        "gemm_decode_up": "gemm A[16,8192]@W[8192,28672] bf16 (decode-time shape)",
        "gemm_decode_down": "gemm A[16,28672]@W[28672,8192] bf16 (decode-time shape)",
        "ffn_block_decode": ("decode-time feed-forward block, 16 tokens: attn@Wo+R, RMSNorm, SwiGLU, @Wd+X1 with "
                             "Wo[8192,8192], Wg/Wu[8192,28672], Wd[28672,8192]; one four-launch plan through the "
                             "public API, CUDA-Graph replay"),
        "mla": "mla_decode batch 64 x 128 heads, cache[64,4096,576] bf16, heads sharded over the GPUs",
        "mla_batch_sharded": "mla_decode batch 64 x 128 heads, cache[64,4096,576] bf16, sequences sharded over the GPUs",
        "gemm_shape": "gemm A[%d,%d]@W[%d,%d] bf16, epilogue %s" % (SHAPE[0], SHAPE[2], SHAPE[2], SHAPE[1], EPILOGUE),
        "tp_mlp": mlp + ", all-reduce fused into the down GEMM",
        "tp_mlp_unfused": mlp + ", separate all-reduce kernel",
        "tp_mlp_noreduce": mlp + ", NO all-reduce (timing baseline, result incomplete)",
    }[name]


def workload_parallelism(name, ranks):
    if ranks == 1:
        return "single GPU"
    if name.startswith("tp_mlp"):
        return f"tp{ranks} over NVLink peer memory"
    if name == "mla":
        return f"{ranks}-way head sharding, cache replicated, no collective"
    if name == "mla_batch_sharded":
        return f"{ranks}-way batch sharding, no collective"
    return "replicas only"


def make_workload(name, device, world=None, ranks=1, rank=0):
    from trinity_lowering import kernels as k
    from trinity_lowering import synthetic as syn

    w = Workload()
    w.name = name
    w.label = workload_label(name)
    w.parallelism = workload_parallelism(name, ranks)
    on_gpu = device.type == "cuda"

    def pin(t):
        return t.pin_memory() if on_gpu else t

    if name in ("gemm_relu", "gemm_bias_1024"):
        if name == "gemm_relu":
            m = n = kk = 8192
            a, wt, bias = syn.gemm_inputs(m, n, kk, 1235, "normal")
            act = k.ACT_RELU
        else:
            m = n = kk = 1024
            a, wt, bias = syn.gemm_inputs(m, n, kk, 1234, "uniform")
            act = k.ACT_NONE
        w.metric, w.unit, w.bound, w.dtype = "bf16_gemm_epilogue_tflops", "TFLOP/s", "tensor", "bf16"
        w.work = 2.0 * m * n * kk / 1e12                       # TFLOP per step
        w.alg_bytes = (m * kk + kk * n + n + m * n) * 2
        w.l2_note = "inputs larger than L2"
        if on_gpu:
            dev = [t.to(device) for t in (a, wt, bias)]
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            # A single small GEMM would be timed with one event pair per launch, which measures the
            # launch path rather than the kernel.  The small configuration therefore runs 32 launches
            # per step over 32 operand sets (32 x 6.3 MB > L2), back to back.
            sets = 1 if (m * kk + kk * n) * 2 > L2_BYTES else 32
            rotating = [(dev[0].clone(), dev[1].clone(), torch.empty_like(out)) for _ in range(sets - 1)]
            rotating.append((dev[0], dev[1], out))
            w.kernels_per_step = sets
            w.e2e_work = w.work
            w.work *= sets
            w.alg_bytes *= sets

            def device_step():
                for a_i, w_i, out_i in rotating:
                    k.gemm(a_i, w_i, bias=dev[2], bias_mode=k.BIAS_COL_VECTOR, activation=act, out=out_i)

            # End to end goes through the public path: plan -> emit -> compile -> load -> prepare,
            # then per step host->device copies, execution.run(), device->host copy.
            host = [pin(t) for t in (a, wt, bias)]
            api = {}

            def make_slot(index):
                import trinity_lowering as tl
                from trinity_lowering import plans
                if not api:
                    artifact = tl.compile(tl.emit(plans.gemm_bias(m, n, kk, "relu" if act else None)))
                    api["module"] = tl.load(artifact, device)
                    artifact.close()
                mine = dev if index == 0 else [torch.empty_like(t) for t in dev]
                mine_out = out if index == 0 else torch.empty_like(out)
                host_out = pin(torch.empty((m, n), dtype=torch.bfloat16))
                execution = api["module"].prepare({"A": mine[0], "W": mine[1], "bias": mine[2]}, out=mine_out)
                if index == 0:
                    w.host_launch = execution.run

                def h2d():
                    for src, dst in zip(host, mine):
                        dst.copy_(src, non_blocking=True)

                def d2h():
                    host_out.copy_(mine_out, non_blocking=True)
                return h2d, execution.run, d2h

            w.make_slot = make_slot
            w.h2d = sum(t.numel() * 2 for t in host)
            w.d2h = m * n * 2

            def check():
                rows = sampled_rows(m, 64)
                expected = a[rows].double() @ wt.double() + bias.double()
                if act:
                    expected = torch.relu(expected)
                return error_figures(out[rows.to(device)].cpu(), expected, len(rows))
            w.check = check
            w.device_step = device_step

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
        x, g = syn.rownorm_inputs(rows, cols, 1236)
        w.metric, w.unit, w.bound, w.dtype = f"{name}_hbm_gbs", "GB/s", "hbm", "bf16"
        w.alg_bytes = rows * cols * 4 + (cols * 2 if name == "rmsnorm" else 0)
        w.work = w.alg_bytes / 1e9
        w.kernels_per_step = 1
        w.l2_note = "inputs larger than L2"
        if on_gpu:
            host_x = pin(x)
            xd, gd = x.to(device), g.to(device)
            yd = torch.empty_like(xd)

            def run(src, dst):
                if name == "rmsnorm":
                    k.rmsnorm(src, gd, 1e-6, out=dst)
                else:
                    k.softmax(src, out=dst)

            def make_slot(index):
                xs = xd if index == 0 else torch.empty_like(xd)
                ys = yd if index == 0 else torch.empty_like(yd)
                host_y = pin(torch.empty_like(x))
                return (lambda: xs.copy_(host_x, non_blocking=True), lambda: run(xs, ys),
                        lambda: host_y.copy_(ys, non_blocking=True))

            w.make_slot = make_slot
            w.device_step = lambda: run(xd, yd)
            w.h2d, w.d2h = x.numel() * 2, x.numel() * 2

            def check():
                picks = sampled_rows(rows, 64)
                xs = x[picks].double()
                if name == "rmsnorm":
                    expected = xs / torch.sqrt(xs.square().mean(dim=1, keepdim=True) + 1e-6) * g.double()
                else:
                    expected = torch.softmax(xs, dim=1)
                return error_figures(yd[picks.to(device)].cpu(), expected, len(picks))
            w.check = check

        def cpu_sample(threads, budget_s):
            from oracle import workloads as wl   # the CPU baseline times the oracle
            torch.set_num_threads(threads)
            sample = x[:4096]
            t0 = time.perf_counter()
            if name == "rmsnorm":
                wl.rmsnorm_oracle(sample, g, 1e-6)
            else:
                wl.softmax_oracle(sample)
            dt = time.perf_counter() - t0
            return sample.numel() * 4 / 1e9 / dt, "4096 of 32768 rows, CPU oracle (FP32 torch)", dt

    elif name == "gemm_shape":
        # One GEMM of a free shape (profiler captures of small cases, tile-shape sweeps):
        # --shape M,N,K --epilogue none|relu|gated.  Operands are drawn on the device.
        m, n, kk = SHAPE
        w.metric, w.unit, w.bound, w.dtype = "bf16_gemm_epilogue_tflops", "TFLOP/s", "tensor", "bf16"
        gated = EPILOGUE == "gated"
        w.work = (4.0 if gated else 2.0) * m * n * kk / 1e12
        w.alg_bytes = (m * kk + (2 if gated else 1) * kk * n + m * n) * 2
        w.kernels_per_step = 1
        w.l2_note = "inputs larger than L2" if w.alg_bytes > L2_BYTES else "inputs fit in L2"
        if on_gpu:
            g = torch.Generator(device=device)
            g.manual_seed(1241)
            ad = torch.randn((m, kk), generator=g, device=device).bfloat16()
            wd = (torch.randn((kk, n), generator=g, device=device) / math.sqrt(kk)).bfloat16()
            w2 = (torch.randn((kk, n), generator=g, device=device) / math.sqrt(kk)).bfloat16() if gated else None
            bias = (torch.randn((n,), generator=g, device=device) * 0.1).bfloat16()
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            host_a = ad.cpu().pin_memory()

            def run(a_s, o_s):
                if gated:
                    k.gemm(a_s, wd, b2=w2, activation=k.ACT_SILU_GATE, out=o_s)
                elif EPILOGUE == "relu":
                    k.gemm(a_s, wd, bias=bias, bias_mode=k.BIAS_COL_VECTOR, activation=k.ACT_RELU, out=o_s)
                else:
                    k.gemm(a_s, wd, out=o_s)

            def make_slot(index):
                a_s = ad if index == 0 else torch.empty_like(ad)
                o_s = out if index == 0 else torch.empty_like(out)
                host_out = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
                return (lambda: a_s.copy_(host_a, non_blocking=True), lambda: run(a_s, o_s),
                        lambda: host_out.copy_(o_s, non_blocking=True))

            w.make_slot = make_slot
            w.device_step = lambda: run(ad, out)
            w.h2d, w.d2h = m * kk * 2, m * n * 2

            def check():
                rows = sampled_rows(m, 32)
                xs = host_a[rows].double()
                up = xs @ wd.cpu().double()
                if gated:
                    gate = xs @ w2.cpu().double()
                    expected = up * (gate * torch.sigmoid(gate))
                elif EPILOGUE == "relu":
                    expected = torch.relu(up + bias.cpu().double())
                else:
                    expected = up
                return error_figures(out[rows.to(device)].cpu(), expected, len(rows))
            w.check = check

        def cpu_sample(threads, budget_s):
            torch.set_num_threads(threads)
            rows = min(m, 256)
            xs, ws = torch.randn(rows, kk), torch.randn(kk, n)
            t0 = time.perf_counter()
            (xs @ ws).bfloat16()
            dt = time.perf_counter() - t0
            return 2.0 * rows * n * kk / 1e12 / dt, f"{rows} of {m} rows, torch CPU FP32 matmul", dt

    elif name in ("gemm_decode_square", "gemm_decode_up", "gemm_decode_down"):
        # Decode-time GEMMs: 16 tokens against a large weight, which the kernel streams once.
        m = 16
        kk, n = {"gemm_decode_square": (8192, 8192), "gemm_decode_up": (8192, 28672),
                 "gemm_decode_down": (28672, 8192)}[name]
        a, wt, _ = syn.gemm_inputs(m, n, kk, 1240, "normal")
        w.metric, w.unit, w.bound, w.dtype = "gemm_decode_hbm_gbs", "GB/s", "hbm", "bf16"
        w.alg_bytes = (m * kk + kk * n + m * n) * 2
        w.work = w.alg_bytes / 1e9
        w.kernels_per_step = 1
        w.l2_note = "inputs larger than L2"
        if on_gpu:
            host_a, host_w = pin(a), pin(wt)
            ad, wd = a.to(device), wt.to(device)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)

            def make_slot(index):
                a_s = ad if index == 0 else torch.empty_like(ad)
                w_s = wd if index == 0 else torch.empty_like(wd)
                o_s = out if index == 0 else torch.empty_like(out)
                host_out = pin(torch.empty((m, n), dtype=torch.bfloat16))

                def h2d():
                    a_s.copy_(host_a, non_blocking=True)
                    w_s.copy_(host_w, non_blocking=True)
                return h2d, lambda: k.gemm(a_s, w_s, out=o_s), lambda: host_out.copy_(o_s, non_blocking=True)

            w.make_slot = make_slot
            w.device_step = lambda: k.gemm(ad, wd, out=out)
            w.h2d, w.d2h = (a.numel() + wt.numel()) * 2, out.numel() * 2
            w.check = lambda: error_figures(out.cpu(), a.double() @ wt.double(), m)

        def cpu_sample(threads, budget_s):
            torch.set_num_threads(threads)
            af, wf = a.float(), wt.float()
            t0 = time.perf_counter()
            (af @ wf).bfloat16()
            dt = time.perf_counter() - t0
            return w.alg_bytes / 1e9 / dt, "whole GEMM, torch CPU FP32 matmul", dt

    elif name == "ffn_block_decode":
        # The whole decode-time feed-forward block as one plan (output projection + residual,
        # RMSNorm, gated GEMM, down projection + residual): plan -> emit -> compile -> load ->
        # prepare -> run.  At 16 tokens the block streams its 1.54 GB of weights once per step;
        # the weights are parameters and stay on the device, a step's host inputs are the
        # attention output and the residual.
        m, d_model, d_ff = 16, 8192, 28672
        w.metric, w.unit, w.bound, w.dtype = "ffn_block_decode_hbm_gbs", "GB/s", "hbm", "bf16"
        weights = d_model * d_model + 3 * d_model * d_ff
        w.alg_bytes = (weights + d_model + 7 * m * d_model + 2 * m * d_ff) * 2   # + intermediates written and read
        w.work = w.alg_bytes / 1e9
        w.kernels_per_step = 4
        w.l2_note = "inputs larger than L2"
        if on_gpu:
            import trinity_lowering as tl
            from trinity_lowering import plans
            wg, wu, wd = syn.mlp_shard_on_device(0, d_model, d_ff, d_ff, device, seed=1243)
            g = torch.Generator(device=device)
            g.manual_seed(1244)
            wo = (torch.randn((d_model, d_model), generator=g, device=device) / math.sqrt(d_model)).bfloat16()
            attn = torch.randn((m, d_model), generator=g, device=device).bfloat16()
            resid = torch.randn((m, d_model), generator=g, device=device).bfloat16()
            gain = (1.0 + 0.02 * torch.randn((d_model,), generator=g, device=device)).bfloat16()
            out = torch.empty((m, d_model), dtype=torch.bfloat16, device=device)
            host_attn, host_resid = pin(attn.cpu()), pin(resid.cpu())
            artifact = tl.compile(tl.emit(plans.ffn_block(m, d_model, d_ff, 1e-6)))
            module = tl.load(artifact, device)
            artifact.close()
            fixed = {"Wo": wo, "g": gain, "Wg": wg, "Wu": wu, "Wd": wd}
            first = module.prepare(dict(fixed, attn=attn, R=resid), out=out)
            # device-timed: replays of the package's own graph of the four launches
            torch.cuda.synchronize(device)   # the operands were drawn on another stream
            captured = tl.Graph.capture(first.run, executions=[first], stream=torch.cuda.Stream(device=device))
            torch.cuda.synchronize(device)
            w.no_graph = w.replays_graph = True
            w.device_step = captured.replay

            def make_slot(index):
                a_s = attn if index == 0 else torch.empty_like(attn)
                r_s = resid if index == 0 else torch.empty_like(resid)
                o_s = out if index == 0 else torch.empty_like(out)
                host_out = pin(torch.empty((m, d_model), dtype=torch.bfloat16))
                execution = module.prepare(dict(fixed, attn=a_s, R=r_s), out=o_s)   # `first` belongs to the graph
                if index == 0:
                    w.host_launch = execution.run

                def h2d():
                    a_s.copy_(host_attn, non_blocking=True)
                    r_s.copy_(host_resid, non_blocking=True)
                return h2d, execution.run, lambda: host_out.copy_(o_s, non_blocking=True)

            w.make_slot = make_slot
            w.h2d, w.d2h = 2 * m * d_model * 2, m * d_model * 2

            def check():
                # float64 on the host, rounded to BF16 where the plan stores an intermediate
                x1 = (attn.cpu().double() @ wo.cpu().double() + resid.cpu().double()).float().bfloat16().double()
                xn = x1 / torch.sqrt((x1 * x1).mean(dim=1, keepdim=True) + 1e-6) * gain.cpu().double()
                xn = xn.float().bfloat16()
                expected = swiglu_partial_float64(xn, wg, wu, wd) + x1
                return error_figures(out.cpu(), expected, m, ulps=2)
            w.check = check

        def cpu_sample(threads, budget_s):
            # the block's four products on a bounded share of the hidden columns, FP32 torch
            torch.set_num_threads(threads)
            g = torch.Generator().manual_seed(1245)
            share = 2048
            a = torch.randn((m, d_model), generator=g)
            wo_c = torch.randn((d_model, d_model), generator=g)
            wg_c, wu_c = torch.randn((d_model, share), generator=g), torch.randn((d_model, share), generator=g)
            wd_c = torch.randn((share, d_model), generator=g)
            t0 = time.perf_counter()
            x1 = a @ wo_c + a
            xn = x1 * torch.rsqrt((x1 * x1).mean(dim=1, keepdim=True) + 1e-6)
            gate = xn @ wg_c
            h = (xn @ wu_c) * (gate * torch.sigmoid(gate))
            (h @ wd_c + x1).bfloat16()
            dt = time.perf_counter() - t0
            streamed = (d_model * d_model + 3 * d_model * share) * 2
            return streamed / 1e9 / dt, f"{share} of {d_ff} hidden columns, torch CPU FP32", dt

    elif name in ("mla", "mla_batch_sharded"):
        batch, heads, seq, d_qk, d_v = 64, 128, 4096, 576, 512
        # On N GPUs "mla" shards the heads N ways and every rank holds the whole cache (the cache
        # is shared by all heads, so tensor-parallel ranks replicate it); "mla_batch_sharded"
        # gives each rank batch/N sequences with all their heads.  Neither has a collective.
        q, cache = syn.mla_inputs(batch, heads, seq, d_qk, 1237)
        if ranks > 1 and name == "mla":
            share = heads // ranks
            q = q[:, rank * share:(rank + 1) * share].contiguous()
            heads = share
        elif ranks > 1:
            share = batch // ranks
            q = q[rank * share:(rank + 1) * share].contiguous()
            cache = cache[rank * share:(rank + 1) * share].contiguous()
            batch = share
            w.strong = True
        scale = 1.0 / math.sqrt(192.0)
        w.metric, w.unit, w.bound, w.dtype = "mla_decode_hbm_gbs", "GB/s", "hbm", "bf16"
        w.alg_bytes = (q.numel() + cache.numel() + batch * heads * d_v) * 2
        w.work = w.alg_bytes / 1e9
        w.l2_note = "inputs larger than L2"
        if on_gpu:
            host_q, host_c = pin(q), pin(cache)
            qd, cd = q.to(device), cache.to(device)
            od = torch.empty((batch, heads, d_v), dtype=torch.bfloat16, device=device)
            splits = k.mla_default_splits(batch, seq)
            scratch = torch.empty(max(256, k.mla_scratch_bytes(batch, heads, d_v, splits)),
                                  dtype=torch.uint8, device=device)
            w.kernels_per_step = 1 if splits == 1 else 2

            def make_slot(index):
                q_s = qd if index == 0 else torch.empty_like(qd)
                c_s = cd if index == 0 else torch.empty_like(cd)
                o_s = od if index == 0 else torch.empty_like(od)
                host_o = pin(torch.empty_like(od, device="cpu"))

                def h2d():
                    q_s.copy_(host_q, non_blocking=True)
                    c_s.copy_(host_c, non_blocking=True)
                return (h2d, lambda: k.mla_decode(q_s, c_s, scale, kv_splits=0, out=o_s, scratch=scratch),
                        lambda: host_o.copy_(o_s, non_blocking=True))

            w.make_slot = make_slot
            w.device_step = lambda: k.mla_decode(qd, cd, scale, kv_splits=0, out=od, scratch=scratch)
            w.h2d, w.d2h = (q.numel() + cache.numel()) * 2, od.numel() * 2

            def check():
                picks = sorted({0, batch - 1})
                got = od[picks].cpu()
                scores = torch.einsum("bhd,bsd->bhs", q[picks].double(), cache[picks].double()) * scale
                expected = torch.softmax(scores, dim=2) @ cache[picks][:, :, :d_v].double()
                return error_figures(got, expected, len(picks) * heads)
            w.check = check

        def cpu_sample(threads, budget_s):
            from oracle import workloads as wl   # the CPU baseline times the oracle
            torch.set_num_threads(threads)
            t0 = time.perf_counter()
            wl.mla_oracle(q, cache, scale, d_v, batches=[0, 1])
            dt = time.perf_counter() - t0
            return (w.alg_bytes * 2 / batch) / 1e9 / dt, f"2 of {batch} sequences, CPU oracle", dt

    elif name in ("tp_mlp", "tp_mlp_unfused", "tp_mlp_noreduce"):
        # Tensor-parallel SwiGLU MLP: total work fixed, sharded over the ranks (strong scaling).
        m, d_model, d_ff = 16384, 8192, 28672
        w.metric, w.unit, w.bound, w.dtype = "tp_mlp_tflops", "TFLOP/s", "tensor", "bf16"
        w.total_work = 3 * 2.0 * m * d_model * d_ff / 1e12
        w.alg_bytes = (m * d_model * 2 + 3 * d_model * d_ff // ranks + m * (d_ff // ranks) * 2) * 2
        w.l2_note = "inputs larger than L2"
        w.strong = True
        w.no_graph = True     # the all-reduce epoch is a launch argument
        w.work = w.total_work / ranks
        if on_gpu:
            from trinity_lowering.tp_mlp import TensorParallelMLP
            shard = d_ff // ranks
            xd = syn.mlp_activations_on_device(m, d_model, device)
            wg, wu, wd = syn.mlp_shard_on_device(rank, d_model, shard, d_ff, device)
            fused = {"tp_mlp": True, "tp_mlp_unfused": False}.get(name)
            mlp = TensorParallelMLP(world, m, d_model, d_ff, wg, wu, wd, fused=fused)
            host_x = xd.cpu().pin_memory()
            w.kernels_per_step = 2 if (ranks == 1 or name != "tp_mlp_unfused") else 3

            def make_slot(index):
                layer = mlp if index == 0 else TensorParallelMLP(world, m, d_model, d_ff, wg, wu, wd, fused=fused)
                xs = xd if index == 0 else torch.empty_like(xd)
                host_y = torch.empty((m, d_model), dtype=torch.bfloat16).pin_memory()
                return (lambda: xs.copy_(host_x, non_blocking=True), lambda: layer.forward(xs),
                        lambda: host_y.copy_(layer.output, non_blocking=True))

            w.make_slot = make_slot
            w.device_step = lambda: mlp.forward(xd)
            w.h2d, w.d2h = xd.numel() * 2, m * d_model * 2

            def check():
                # Every rank evaluates its own partial product for the sampled rows in float64 and
                # rounds it to BF16 (the partials cross NVLink in BF16); rank 0 adds the partials in
                # rank order in FP32, as the kernel does, and compares.
                rows = sampled_rows(m, 32)
                partial = swiglu_partial_float64(host_x[rows], wg, wu, wd).float().bfloat16()
                if ranks > 1 and name != "tp_mlp_noreduce":
                    import torch.distributed as dist
                    parts = [torch.empty_like(partial, device=device) for _ in range(ranks)]
                    dist.all_gather(parts, partial.to(device))
                    total = torch.zeros(partial.shape, dtype=torch.float32)
                    for part in parts:
                        total += part.cpu().float()
                    expected = total
                else:
                    expected = partial.float()
                return error_figures(mlp.output[rows.to(device)].cpu(), expected, len(rows))
            w.check = check

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
    w.cpu_sample = cpu_sample
    return w


def config_of(w, graph):
    return {"workload": w.label, "l2": w.l2_note, "parallelism": w.parallelism,
            "launch": "CUDA Graph replay" if graph or w.replays_graph else "direct"}


# ---------------------------------------------------------------- timing
def timed(step, steps, stream):
    """CUDA-event time (ms) of `steps` calls on `stream`."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        step()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop)


def end_to_end(w, steps, device):
    """The step through the public call with host buffers: the host->device copy of step i+1, the
    kernels of step i and the device->host copy of step i-1 run on three streams over two sets
    of device buffers; every step's copies are inside the timed region.  Returns ms."""
    slots = [w.make_slot(0), w.make_slot(1)]
    s_in, s_run, s_out = (torch.cuda.Stream(device=device) for _ in range(3))
    copied = [torch.cuda.Event() for _ in range(2)]
    ran = [torch.cuda.Event() for _ in range(2)]
    read = [torch.cuda.Event() for _ in range(2)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def pipeline(count, timing):
        torch.cuda.synchronize()
        if timing:
            start.record(s_in)
        for i in range(count):
            j = i % 2
            h2d, run, d2h = slots[j]
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ran[j])       # the kernels of step i-2 have consumed this input
                h2d()
                copied[j].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(copied[j])
                if i >= 2:
                    s_run.wait_event(read[j])     # the result of step i-2 has left this buffer
                run()
                ran[j].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ran[j])
                d2h()
                read[j].record(s_out)
        if timing:
            stop.record(s_out)
        torch.cuda.synchronize()

    pipeline(3, False)
    pipeline(steps, True)
    return start.elapsed_time(stop)


def measure(w, steps, warmup, stream, device, use_graph, barrier, clock_index=None):
    """Device-timed steps of one workload; returns (ms, launches through the library, clocks)."""
    from trinity_lowering import kernels as k
    with torch.cuda.stream(stream):
        w.device_step()
        torch.cuda.synchronize()
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                w.device_step()
            replay = graph.replay
        else:
            replay = w.device_step
        for _ in range(warmup):
            replay()
        barrier()
        before = k.launch_count()
        if clock_index is None:
            ms, clocks = timed(replay, steps, stream), None
        else:
            with ClockSampler(clock_index) as sampler:
                ms = timed(replay, steps, stream)
            clocks = sampler.summary()
        barrier()
        launches = k.launch_count() - before
        if use_graph or w.replays_graph:
            launches += steps * w.kernels_per_step   # replays do not pass through the library
    return ms, launches, clocks


def roofline_of(w, per_step_ms, long_run):
    pk = peaks()
    achieved = w.work / (per_step_ms / 1e3)            # per GPU
    extra = {}
    if w.bound == "tensor":
        # The burst figure is the denominator for a kernel timed alone over a few milliseconds;
        # a region that keeps the tensor cores busy for longer runs under the 1 kW power cap, as
        # the sustained cuBLAS figure does.  Both fractions are in the line.
        peak = pk["bf16_tflops_sustained"] if long_run else pk["bf16_tflops"]
        note = ("sustained" if long_run else "burst") + " cuBLAS bf16, " + pk["source"]
        unit = "TFLOP/s"
        extra = {"frac_of_burst": achieved / pk["bf16_tflops"],
                 "frac_of_sustained": achieved / pk["bf16_tflops_sustained"]}
    else:
        peak, note, unit = pk["hbm_gbs"], "copy bandwidth, " + pk["source"], "GB/s"
    return {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "traffic": NCU_TRAFFIC_BYTES.get(w.name), "algorithmic_bytes": w.alg_bytes, "peak_kind": note, **extra}


def run_reference(args, rank, world):
    """The reference's CPU evaluation of the path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    w = make_workload(args.workload, torch.device("cpu"), ranks=world)
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
        "ms_per_step": None, "higher_is_better": True, "scaling": "strong" if w.strong else "weak",
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": config_of(w, not (w.no_graph or args.no_graph)),
        "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="tp_mlp")
    parser.add_argument("--shape", default=None, help="M,N,K of --workload gemm_shape")
    parser.add_argument("--epilogue", default="none", choices=["none", "relu", "gated"],
                        help="epilogue of --workload gemm_shape")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-configs", action="store_true",
                        help="skip the block with the other benchmark configurations")
    parser.add_argument("--no-graph", action="store_true",
                        help="launch directly instead of replaying a CUDA Graph (for profilers)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    global SHAPE, EPILOGUE
    if args.shape:
        SHAPE = tuple(int(v) for v in args.shape.split(","))
    EPILOGUE = args.epilogue

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
        # the kernels use plain peer loads and stores; nothing here needs a multicast binding
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=device)

    from trinity_lowering import kernels as k
    k.library()
    world_obj = None
    if distributed and args.workload.startswith("tp_mlp"):
        from trinity_lowering.world import World
        world_obj = World.from_torchrun(timeout=120.0)
    stream = torch.cuda.Stream(device=device)

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
            torch.cuda.synchronize()

    def maximum(*values):
        if not distributed:
            return list(values)
        t = torch.tensor(values, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def worst_parity(figures):
        """The largest errors over the ranks (every rank checks its own shard)."""
        rel, worst, bound = maximum(figures["rel_l2"], figures["max_abs"], figures["max_abs_bound"])
        return {"rel_l2": rel, "max_abs": worst, "max_abs_bound": bound, "rows": figures["rows"],
                "ok": bool(rel <= REL_L2_BOUND and worst <= bound)}

    w = make_workload(args.workload, device, world_obj, world, rank)
    use_graph = not (w.no_graph or args.no_graph)
    ms, launches, clocks = measure(w, args.steps, args.warmup, stream, device, use_graph, barrier, local_rank)
    # milestones of the last device-timed fused launch (read before the end-to-end phase, whose
    # launches wait for each rank's own copies and therefore start at different times)
    stamps = k.gemm_allreduce_stamps() if distributed and args.workload == "tp_mlp" else None
    parity = w.check()
    if not (args.workload.startswith("tp_mlp") and distributed):
        parity = worst_parity(parity)       # the MLP's check already gathers over the ranks
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = end_to_end(w, e2e_steps, device)
    barrier()
    host_launch_us = None
    if w.host_launch is not None:
        calls = 100
        with torch.cuda.stream(stream):
            t0 = time.perf_counter()
            for _ in range(calls):
                w.host_launch()
            host_launch_us = (time.perf_counter() - t0) / calls * 1e6
        barrier()
    ms, e2e_ms = maximum(ms, e2e_ms)

    status = k.device_status()
    if status:
        raise SystemExit(f"device status word {status:#x}: a bounded in-kernel wait gave up")

    per_step_ms = ms / args.steps
    line = {
        "metric": w.metric, "value": world * w.work * args.steps / (ms / 1e3), "unit": w.unit,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step_ms,
        "higher_is_better": True, "scaling": "strong" if w.strong else "weak", "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic", "config": config_of(w, use_graph),
        # more than 100 ms of back-to-back tensor work: the power cap is what the clocks follow
        "roofline": roofline_of(w, per_step_ms, ms > 100.0),
        "e2e": {"value": world * (w.e2e_work or w.work) * e2e_steps / (e2e_ms / 1e3), "unit": w.unit,
                "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h, "steps": e2e_steps,
                "overlap": "copies of neighbouring steps overlap the kernels (three streams, two buffer sets)"},
        "parity": parity,
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if host_launch_us is not None:
        line["host_launch_us"] = host_launch_us   # public-API launch, host side only
    if distributed and args.workload == "tp_mlp":
        # milestones of the last fused down-projection launch on every rank (its first thread block),
        # microseconds after its start: last MMA committed, last partial tile handed over, last
        # owned rows reduced, all ranks retired
        t = stamps
        mine = [round((v - t[0]) / 1e3, 1) for v in t[1:]]
        every = [None] * world
        dist.all_gather_object(every, mine)
        line["fused_gemm_milestones_us"] = every      # one list per rank

    # The other benchmark configurations, each device-timed and checked the same way.
    if args.workload == "tp_mlp" and not args.no_configs:
        del w
        torch.cuda.empty_cache()
        names = (["gemm_bias_1024", "gemm_relu", "rmsnorm", "softmax", "mla", "gemm_decode_square",
                  "gemm_decode_up", "gemm_decode_down", "ffn_block_decode"] if world == 1
                 else ["mla", "mla_batch_sharded"])
        block = {}
        for name in names:
            other = make_workload(name, device, None, world, rank)
            steps = 100 if name == "gemm_relu" else 30
            other_ms, other_launches, _ = measure(other, steps, 5, stream, device, not other.no_graph, barrier)
            figures = worst_parity(other.check())
            (other_ms,) = maximum(other_ms)
            roof = roofline_of(other, other_ms / steps, False)
            block[name] = {"workload": other.label, "parallelism": other.parallelism, "steps": steps,
                           "ms_per_step": other_ms / steps,
                           "value": world * other.work * steps / (other_ms / 1e3), "unit": other.unit,
                           "roofline": roof, "parity": figures, "gpu_launches": other_launches}
            line["gpu_launches"] += other_launches
            del other
            torch.cuda.empty_cache()
        line["configs"] = block
        status = k.device_status()
        if status:
            raise SystemExit(f"device status word {status:#x}: a bounded in-kernel wait gave up")

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        w_cpu = make_workload(args.workload, torch.device("cpu"))
        v, sample, _ = w_cpu.cpu_sample(threads, budget_s=10.0)
        line["cpu_baseline"] = {"value": v, "unit": line["unit"], "cores": threads, "kind": "port",
                                "sample": sample}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()
    checks = [line["parity"]] + [c["parity"] for c in line.get("configs", {}).values()]
    if not all(c["ok"] for c in checks):
        print("bench.py: a result is outside the stated tolerance (see \"parity\")", file=sys.stderr)
        sys.exit(3)


if __name__ == "__main__":
    main()
