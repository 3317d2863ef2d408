"""RMSNorm and row softmax through the C ABI versus the CPU oracle (B200 only)."""
import pytest
import torch

from oracle import workloads as wl
from parity import assert_close_bf16

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def kernels():
    from trinity_lowering import kernels as k
    k.library()
    return k


@pytest.mark.parametrize("name", ["rmsnorm_eps_gain", "rmsnorm_plain"])
def test_rmsnorm_golden(kernels, golden, name):
    case = golden[name]
    x, g = wl.rownorm_inputs(case["rows"], case["cols"], case["seed"])
    if name == "rmsnorm_plain":
        x[0].zero_()
    out = kernels.rmsnorm(x.to(DEV), g.to(DEV) if case["gain"] else None, case["eps"]).cpu()
    assert_close_bf16(out, case["expected"].view(torch.bfloat16), max_ulp=1)


def test_softmax_golden(kernels, golden):
    case = golden["softmax"]
    x, _ = wl.rownorm_inputs(case["rows"], case["cols"], case["seed"])
    out = kernels.softmax(x.to(DEV)).cpu()
    assert_close_bf16(out, case["expected"].view(torch.bfloat16), max_ulp=1)


@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 136), (16, 4096), (257, 4096), (33, 2048),
                                       (7, 8192), (5, 1000), (64, 256)])
def test_rmsnorm_shapes(kernels, rows, cols):
    x, g = wl.rownorm_inputs(rows, cols, 99 + rows)
    out = kernels.rmsnorm(x.to(DEV), g.to(DEV), 1e-6).cpu()
    assert_close_bf16(out, wl.rmsnorm_oracle(x, g, 1e-6), max_ulp=1, max_abs=4e-2)


@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 136), (16, 4096), (257, 4096), (33, 2048),
                                       (7, 8192), (5, 1000), (64, 256)])
def test_softmax_shapes(kernels, rows, cols):
    x, _ = wl.rownorm_inputs(rows, cols, 199 + rows)
    out = kernels.softmax((x * 3).to(DEV)).cpu()
    expected = wl.softmax_oracle(x * 3)
    assert_close_bf16(out, expected, max_ulp=1, max_abs=2e-2)
    assert torch.allclose(out.float().sum(1), torch.ones(rows), atol=2e-2)


def test_full_size_properties(kernels):
    """[32768, 4096] rows: oracle on a strided sample; scale invariance and unit row sums."""
    x, g = wl.rownorm_inputs(32768, 4096, 1236)
    xd, gd = x.to(DEV), g.to(DEV)
    y = kernels.rmsnorm(xd, gd, 1e-6)
    s = kernels.softmax(xd)
    rows = torch.arange(0, 32768, 1021)
    assert_close_bf16(y[rows.to(DEV)].cpu(), wl.rmsnorm_oracle(x[rows], g, 1e-6), max_ulp=1,
                      max_abs=4e-2)
    assert_close_bf16(s[rows.to(DEV)].cpu(), wl.softmax_oracle(x[rows]), max_ulp=1, max_abs=2e-2)
    # RMSNorm is invariant to a power-of-two rescale of the row (exact in BF16/FP32, eps=0)
    y1 = kernels.rmsnorm(xd, None, 0.0)
    y2 = kernels.rmsnorm(xd * 4, None, 0.0)
    assert torch.equal(y1, y2)
    sums = s.float().sum(1)
    assert (sums - 1).abs().max().item() < 2e-2
    # softmax is invariant to adding a constant that is exact in BF16 for this range? not in
    # general -- instead check idempotence of the argmax and monotonicity on one row
    assert torch.equal(s.float().argmax(1), xd.float().argmax(1))


def test_rejects_unsupported(kernels):
    x = torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError):
        kernels.rmsnorm(x)
    with pytest.raises(kernels.KernelError):
        kernels.softmax(torch.zeros(2, 16384, dtype=torch.bfloat16, device=DEV))
