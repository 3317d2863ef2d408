"""The candidate comparison harness: correctness gates timing (rules of the reference's
src/emit/wrapper/selection.py:6-40), on CPU with stand-in candidates and on a B200 with the
native GEMM against the cuBLAS baseline."""
import time

import pytest
import torch

from trinity_lowering import selection


def _tensors():
    g = torch.Generator().manual_seed(3)
    a = torch.randn(8, 16, generator=g)
    w = torch.randn(16, 4, generator=g)
    return {"A": a, "W": w, "Y": torch.empty(8, 4)}, a @ w


def test_only_correct_candidates_are_timed_and_the_fastest_wins():
    tensors, expected = _tensors()
    timed = []

    def good(delay):
        def run(t):
            time.sleep(delay)
            t["Y"].copy_(t["A"] @ t["W"])
        return run

    def wrong(t):
        t["Y"].copy_(t["A"] @ t["W"] + 1.0)

    def leaves_nan(t):
        pass

    def clobbers_input(t):
        t["Y"].copy_(t["A"] @ t["W"])
        t["A"].zero_()

    def raises(t):
        raise ValueError("unsupported shape")

    def benchmark(call):
        t0 = time.perf_counter()
        call()
        timed.append(1)
        return (time.perf_counter() - t0) * 1e3

    candidates = [selection.Candidate("slow", good(0.02)), selection.Candidate("wrong", wrong),
                  selection.Candidate("nan", leaves_nan), selection.Candidate("clobber", clobbers_input),
                  selection.Candidate("raises", raises), selection.Candidate("fast", good(0.0))]
    winner, reports = selection.select(candidates, tensors, "Y", expected, benchmark=benchmark)
    assert winner.key == "fast"
    assert len(timed) == 2                       # only the two correct candidates were timed
    status = {r.key: r.status for r in reports}
    assert status == {"slow": "passed", "wrong": "correctness", "nan": "correctness", "clobber": "correctness",
                      "raises": "load", "fast": "passed"}
    assert "modified" in next(r.reason for r in reports if r.key == "clobber")
    # the caller's sample tensors are untouched
    fresh, _ = _tensors()
    assert torch.equal(tensors["A"], fresh["A"])


def test_no_valid_candidate_and_bad_timings():
    tensors, expected = _tensors()
    ok = selection.Candidate("ok", lambda t: t["Y"].copy_(t["A"] @ t["W"]))
    with pytest.raises(selection.NoCandidate) as info:
        selection.select([ok], tensors, "Y", expected, benchmark=lambda call: float("nan"))
    assert info.value.reports[0].status == "benchmark"
    with pytest.raises(selection.NoCandidate):
        selection.select([], tensors, "Y", expected)

    def poisoned(t):
        raise RuntimeError("CUDA error: an illegal memory access was encountered")
    with pytest.raises(RuntimeError, match="fatal CUDA failure"):
        selection.select([selection.Candidate("bad", poisoned), ok], tensors, "Y", expected)


@pytest.mark.gpu
def test_native_gemm_against_the_library_baseline():
    from oracle import workloads as wl
    a, w, bias = wl.gemm_inputs(512, 768, 1024, 5, "normal")
    dev = "cuda:0"
    tensors = {"A": a.to(dev), "W": w.to(dev), "bias": bias.to(dev),
               "Y": torch.empty(512, 768, dtype=torch.bfloat16, device=dev)}
    expected = wl.gemm_oracle(a, w, bias, "relu")
    winner, reports = selection.select(selection.gemm_candidates("relu"), tensors, "Y", expected)
    assert [r.status for r in reports] == ["passed", "passed"], reports
    assert winner.key in ("sm100.gemm_bf16_tcgen05", "cublas.matmul+epilogue")
    assert all(r.execution_time_ms > 0 for r in reports)
