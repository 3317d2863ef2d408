"""Regenerates tests/golden/reference_eval.pt from the reference's own evaluator.

Run where the reference tree is available:  python tests/golden/make_golden.py <reference root>
(or set TRINITY_REFERENCE_ROOT).
It imports ``_reference`` from <reference>/src/emit/wrapper/reference.py, evaluates the
workload equations of ``oracle.workloads`` on small seeded inputs and stores inputs' seeds,
shapes and the reference's results (BF16 bit patterns).  The committed fixture lets the oracle
be checked where the reference tree is absent.
"""
import importlib.util
import math
import sys
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
from oracle import evaluator as ev  # noqa: E402
from oracle import workloads as wl  # noqa: E402


def reference_evaluator(root):
    path = Path(root) / "src" / "emit" / "wrapper" / "reference.py"
    spec = importlib.util.spec_from_file_location("trinity_reference_eval", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module._reference


def bits(t):
    return t.contiguous().view(torch.int16).clone()


def main():
    import os
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRINITY_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_golden.py <reference root>")
    ref = reference_evaluator(root)

    def stored(equation, env, shape, dtype="bf16"):
        out = ref(ev.store_root(equation, shape, dtype), dict(env))
        return out.to(ev.DTYPES[dtype])

    cases = {}
    for name, (m, n, k, act, bias_mode, dist, seed) in {
        "gemm_bias": (96, 80, 72, None, "col", "uniform", 1234),
        "gemm_bias_relu": (160, 136, 200, "relu", "col", "normal", 1235),
        "gemm_matrix_bias": (64, 128, 64, None, "matrix", "normal", 1236),
        "gemm_silu": (48, 64, 128, "silu", "col", "normal", 1237),
    }.items():
        a, w, bias = wl.gemm_inputs(m, n, k, seed, dist)
        if bias_mode == "matrix":
            bias = wl._normal((m, n), 0.5, wl._gen(seed + 100))
        out = stored(wl.gemm_equation(act, bias_mode), {"A": a, "W": w, "bias": bias}, [m, n])
        cases[name] = {"kind": "gemm", "m": m, "n": n, "k": k, "activation": act,
                       "bias_mode": bias_mode, "distribution": dist, "seed": seed,
                       "expected": bits(out)}
    a, wg, wu, _ = wl.mlp_inputs(40, 64, 96, 1238)
    out = stored(wl.gated_equation(), {"A": a, "Wu": wu, "Wg": wg}, [40, 96])
    cases["gated"] = {"kind": "gated", "m": 40, "d_model": 64, "d_ff": 96, "seed": 1238,
                      "expected": bits(out)}
    for name, (rows, cols, eps, gain, seed) in {
        "rmsnorm_eps_gain": (12, 512, 1e-6, True, 1240),
        "rmsnorm_plain": (5, 136, 0.0, False, 1241),
    }.items():
        x, g = wl.rownorm_inputs(rows, cols, seed)
        if name == "rmsnorm_plain":
            x[0].zero_()  # eps-free form keeps 0/0 -> NaN (python/tests/test_tensor_ops.py:205)
        out = stored(wl.rmsnorm_equation(cols, eps, gain), {"X": x, "g": g}, [rows, cols])
        cases[name] = {"kind": "rmsnorm", "rows": rows, "cols": cols, "eps": eps, "gain": gain,
                       "seed": seed, "expected": bits(out)}
    x, _ = wl.rownorm_inputs(9, 264, 1242)
    out = stored(wl.softmax_equation(), {"X": x}, [9, 264])
    cases["softmax"] = {"kind": "softmax", "rows": 9, "cols": 264, "seed": 1242,
                        "expected": bits(out)}
    # MLA at reduced geometry: same equation, evaluated by the reference evaluator per batch.
    batch, heads, seq, d_qk, d_v = 2, 16, 96, 576, 512
    q, cache = wl.mla_inputs(batch, heads, seq, d_qk, 1243)
    scale = 1.0 / math.sqrt(192.0)
    outs = []
    for b in range(batch):
        env = {"Q": q[b], "Kt": cache[b].t().contiguous(), "V": cache[b][:, :d_v].contiguous()}
        s = ev.op("mul", ev.op("matmul", ev.load("Q"), ev.load("Kt")), ev.const(scale))
        sh = ev.op("sub", s, ev.op("unsqueeze", ev.op("max_reduce", s, axis=1), axis=1))
        e = ev.op("exp", sh)
        p = ev.op("div", e, ev.op("unsqueeze", ev.op("sum", e, axis=1), axis=1))
        outs.append(stored(ev.op("matmul", p, ev.load("V")), env, [heads, d_v]))
    cases["mla"] = {"kind": "mla", "batch": batch, "heads": heads, "seq": seq, "d_qk": d_qk,
                    "d_v": d_v, "seed": 1243, "scale": scale, "expected": bits(torch.stack(outs))}
    # Multi-step stores with a BF16 intermediate and a register intermediate
    # (storage rounding only at non-register steps).
    x, _ = wl.rownorm_inputs(6, 64, 1244)
    for register in (False, True):
        root = {"op": "stores", "shape": [6, 64], "steps": [
            {"expression": ev.op("sigmoid", ev.load("X")), "register": register, "dtype": "bf16",
             "shape": [6, 64], "output": {"value": "t", "shape": [6, 64], "strides": [64, 1],
                                          "offset": 0}},
            {"expression": ev.op("mul", ev.load("t"), ev.load("X")), "register": False,
             "dtype": "bf16", "shape": [6, 64],
             "output": {"value": "y", "shape": [6, 64], "strides": [64, 1], "offset": 0}}]}
        out = ref(root, {"X": x}).to(torch.bfloat16)
        cases["silu_two_step_%s" % ("register" if register else "global")] = {
            "kind": "two_step", "register": register, "seed": 1244, "expected": bits(out)}
    torch.save(cases, Path(__file__).with_name("reference_eval.pt"))
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
