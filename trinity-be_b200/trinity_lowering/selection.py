"""Correctness-then-timing choice between implementations of one operation.

Takes the role of the reference's candidate comparison (src/emit/wrapper/selection.py:6-40 and
the Python harness around ``kernel_candidates``, src/emit/candidate.rs:64-71), which leaves
native kernels out; here the native sm_100a kernels are the candidates and library kernels
(cuBLAS through ``torch.matmul``) are the baselines they are compared with.

The rules are the reference's: a candidate only gets timed after it produced the right answer on
private copies of the sample tensors (output pre-filled with NaN, inputs verified untouched), a
timing must be finite and positive, every candidate leaves a report, and an error that poisons
the CUDA context stops the comparison instead of trying the next candidate.
"""
import math
import time
from dataclasses import dataclass, field

import torch

_FATAL = ("illegal memory access", "device-side assert", "illegal instruction", "misaligned address")


@dataclass
class Candidate:
    """``run(tensors)`` writes ``tensors[output]`` from the other entries of the dict."""
    key: str
    run: callable
    provider: str = "sm100"
    details: dict = field(default_factory=dict)


@dataclass
class Report:
    key: str
    provider: str
    status: str            # "load" | "correctness" | "benchmark" | "passed"
    reason: str = ""
    execution_time_ms: float = float("nan")


class NoCandidate(RuntimeError):
    def __init__(self, reports):
        super().__init__("no candidate passed correctness and timing")
        self.reports = reports


def cuda_event_benchmark(warmup=3, iterations=20):
    """Milliseconds per call with CUDA events on the current stream; wall clock without a GPU."""
    def measure(call):
        for _ in range(warmup):
            call()
        if not torch.cuda.is_available():
            t0 = time.perf_counter()
            for _ in range(iterations):
                call()
            return (time.perf_counter() - t0) * 1e3 / iterations
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(iterations):
            call()
        stop.record()
        stop.synchronize()
        return start.elapsed_time(stop) / iterations
    return measure


def select(candidates, tensors, output, expected, compare=None, benchmark=None):
    """Returns (winner, reports).  ``tensors`` maps names to sample tensors (the entry ``output``
    gives shape and dtype of the result), ``expected`` is the oracle's result, ``compare(actual,
    expected)`` raises on a mismatch (default: the path's BF16 bar, rel-L2 <= 1e-2)."""
    compare = compare or _default_compare
    benchmark = benchmark or cuda_event_benchmark()
    reports, passed = [], []
    for candidate in candidates:
        report = Report(candidate.key, candidate.provider, "load")
        reports.append(report)
        try:
            trial = {name: t.clone() for name, t in tensors.items()}
            trial[output].fill_(float("nan"))
            candidate.run(trial)           # lazy initialisation happens before any timing
            report.status = "correctness"
            compare(trial[output], expected)
            for name, original in tensors.items():
                if name != output and not torch.equal(trial[name], original):
                    raise AssertionError(f"input {name} was modified")
            report.status = "benchmark"
            elapsed = float(benchmark(lambda: candidate.run(trial)))
            if not math.isfinite(elapsed) or elapsed <= 0:
                raise ValueError("benchmark must return finite, positive milliseconds")
            report.status, report.execution_time_ms = "passed", elapsed
            passed.append((elapsed, candidate))
        except Exception as error:  # reported per candidate; fatal CUDA errors end the comparison
            text = str(error).lower()
            if any(marker in text for marker in _FATAL):
                raise RuntimeError("fatal CUDA failure while evaluating a candidate") from error
            report.reason = f"{type(error).__name__}: {error}"
    if not passed:
        raise NoCandidate(reports)
    return min(passed, key=lambda item: item[0])[1], reports


def _default_compare(actual, expected):
    a, e = actual.float(), expected.float().to(actual.device)
    if not torch.equal(torch.isnan(a), torch.isnan(e)):
        raise AssertionError("NaN pattern differs")
    finite = torch.isfinite(e)
    err = (a[finite] - e[finite]).norm() / e[finite].norm().clamp_min(1e-30)
    if not err <= 1e-2:
        raise AssertionError(f"rel-L2 {err.item():.3e} above 1e-2")


def gemm_candidates(activation=None):
    """The native GEMM (+ bias, activation) against the cuBLAS baseline for the same equation.
    Tensors: A [m,k], W [k,n], optional bias [n], Y [m,n]."""
    from . import kernels

    act = {None: kernels.ACT_NONE, "relu": kernels.ACT_RELU, "silu": kernels.ACT_SILU}[activation]

    def native(t):
        bias = t.get("bias")
        kernels.gemm(t["A"], t["W"], bias=bias, bias_mode=kernels.BIAS_COL_VECTOR if bias is not None else None,
                     activation=act, out=t["Y"])

    def library(t):
        y = torch.matmul(t["A"], t["W"]).float()
        if t.get("bias") is not None:
            y = y + t["bias"].float()
        if activation == "relu":
            y = torch.relu(y)
        elif activation == "silu":
            y = y * torch.sigmoid(y)
        t["Y"].copy_(y)

    return [Candidate("sm100.gemm_bf16_tcgen05", native, "sm100"),
            Candidate("cublas.matmul+epilogue", library, "library", {"note": "baseline, not shipped"})]
