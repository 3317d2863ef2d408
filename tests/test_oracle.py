"""The CPU oracle must reproduce, bit for bit, what the reference's own evaluator produced
for the committed golden cases (tests/golden/make_golden.py)."""
import torch

from oracle import evaluator as ev
from oracle import workloads as wl


def bits(t):
    return t.contiguous().view(torch.int16)


def test_gemm_cases_match_reference_evaluator(golden):
    for name, case in golden.items():
        if case["kind"] != "gemm":
            continue
        a, w, bias = wl.gemm_inputs(case["m"], case["n"], case["k"], case["seed"],
                                    case["distribution"])
        if case["bias_mode"] == "matrix":
            bias = wl._normal((case["m"], case["n"]), 0.5, wl._gen(case["seed"] + 100))
        out = wl.gemm_oracle(a, w, bias, case["activation"], case["bias_mode"])
        assert torch.equal(bits(out), case["expected"]), name


def test_gated_matches_reference_evaluator(golden):
    case = golden["gated"]
    a, wg, wu, _ = wl.mlp_inputs(case["m"], case["d_model"], case["d_ff"], case["seed"])
    assert torch.equal(bits(wl.gated_oracle(a, wu, wg)), case["expected"])


def test_row_kernels_match_reference_evaluator(golden):
    for name in ("rmsnorm_eps_gain", "rmsnorm_plain"):
        case = golden[name]
        x, g = wl.rownorm_inputs(case["rows"], case["cols"], case["seed"])
        if name == "rmsnorm_plain":
            x[0].zero_()
        out = wl.rmsnorm_oracle(x, g if case["gain"] else None, case["eps"])
        assert torch.equal(bits(out), case["expected"]), name
    # the eps-free form keeps 0/0 -> NaN for an all-zero row
    assert torch.isnan(out[0].float()).all()
    case = golden["softmax"]
    x, _ = wl.rownorm_inputs(case["rows"], case["cols"], case["seed"])
    assert torch.equal(bits(wl.softmax_oracle(x)), case["expected"])


def test_mla_matches_reference_evaluator(golden):
    case = golden["mla"]
    q, cache = wl.mla_inputs(case["batch"], case["heads"], case["seq"], case["d_qk"], case["seed"])
    out = wl.mla_oracle(q, cache, case["scale"], case["d_v"])
    assert torch.equal(bits(out), case["expected"])


def test_storage_rounding_only_at_non_register_steps(golden):
    x, _ = wl.rownorm_inputs(6, 64, 1244)
    results = {}
    for register in (False, True):
        root = {"op": "stores", "shape": [6, 64], "steps": [
            {"expression": ev.op("sigmoid", ev.load("X")), "register": register, "dtype": "bf16",
             "shape": [6, 64],
             "output": {"value": "t", "shape": [6, 64], "strides": [64, 1], "offset": 0}},
            {"expression": ev.op("mul", ev.load("t"), ev.load("X")), "register": False,
             "dtype": "bf16", "shape": [6, 64],
             "output": {"value": "y", "shape": [6, 64], "strides": [64, 1], "offset": 0}}]}
        out = ev.evaluate(root, {"X": x}).to(torch.bfloat16)
        key = "silu_two_step_%s" % ("register" if register else "global")
        assert torch.equal(bits(out), golden[key]["expected"]), key
        results[register] = out
    assert not torch.equal(results[False], results[True])  # the BF16 intermediate is visible


def test_dyadic_pattern_is_exact_in_fp32():
    """reference.cu:17-19 pattern: FP32 accumulation in any order equals float64."""
    a, b = wl.dyadic_gemm_inputs(128, 128, 256)
    exact = (a.double() @ b.double())
    assert torch.equal((a.float() @ b.float()).double(), exact)
    assert a.float().abs().max() <= 1.0 and b.float().abs().max() <= 1.125


def test_relu_keeps_nan_and_signed_zero():
    """python/tests/test_tensor_ops.py:161-186 special values."""
    values = torch.tensor([-float("inf"), -2.0, -1e-8, -0.0, 0.0, 1e-8, 2.0, float("inf"),
                           float("nan")])
    out = ev.evaluate(ev.op("relu", ev.load("x")), {"x": values})
    assert torch.equal(torch.isnan(out), torch.isnan(values))
    assert out[1] == 0 and out[6] == 2.0 and out[7] == float("inf")
