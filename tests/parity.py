"""Shared comparison helpers for the parity tests (tolerances are stated here once)."""
import torch

# Floating-point bar of the path: BF16 results within rel-L2 <= 1e-2 of the FP32-accumulated
# oracle, and max-abs <= 2e-2 where outputs are O(1).  Against the oracle *rounded to BF16*
# results are expected within one BF16 ulp (the reference's own bound,
# python/tests/test_tensor_ops.py:105-119).
REL_L2 = 1e-2
MAX_ABS = 2e-2


def ordered(t):
    raw = t.contiguous().view(torch.int16).to(torch.int32)
    return torch.where(raw < 0, -32768 - raw, raw)


def ulp_distance(actual, expected):
    return (ordered(actual) - ordered(expected)).abs()


def assert_special_values_equal(actual, expected):
    a, e = actual.float(), expected.float()
    assert torch.equal(torch.isnan(a), torch.isnan(e))
    assert torch.equal(torch.isposinf(a), torch.isposinf(e))
    assert torch.equal(torch.isneginf(a), torch.isneginf(e))


def assert_close_bf16(actual, expected, max_ulp=1, max_abs=None, rel_l2=REL_L2,
                      ulp_outlier_fraction=0.0, abs_floor_scale=1e-3):
    """actual/expected: BF16 tensors on the CPU.

    An element passes when it is within ``max_ulp`` BF16 ulps of the oracle, or within
    ``abs_floor_scale`` x rms(expected) absolutely: outputs that cancel to nearly zero carry the
    FP32-versus-float64 accumulation difference of much larger partial sums, which no ulp count
    of the tiny result can bound."""
    assert actual.shape == expected.shape and actual.dtype == expected.dtype == torch.bfloat16
    assert_special_values_equal(actual, expected)
    finite = torch.isfinite(expected.float())
    a, e = actual.float()[finite], expected.float()[finite]
    if e.numel() == 0:
        return
    err = (a - e).norm() / e.norm().clamp_min(1e-30)
    assert err <= rel_l2, f"rel-L2 {err.item():.3e} > {rel_l2}"
    if max_abs is not None:
        worst = (a - e).abs().max().item()
        assert worst <= max_abs, f"max-abs {worst:.3e} > {max_abs}"
    if max_ulp is None:
        return
    distance = ulp_distance(actual, expected)[finite]
    floor = abs_floor_scale * e.square().mean().sqrt().item()
    over = ((distance > max_ulp) & ((a - e).abs() > floor)).float().mean().item()
    assert over <= ulp_outlier_fraction, (
        f"{over:.3e} of elements beyond {max_ulp} ulp (max {distance.max().item()})")
