"""GEMM + fused epilogue through the C ABI versus the CPU oracle (B200 only)."""
import pytest
import torch

from oracle import workloads as wl
from parity import assert_close_bf16

pytestmark = pytest.mark.gpu

kernels = None


@pytest.fixture(scope="module", autouse=True)
def _library():
    global kernels
    from trinity_lowering import kernels as k
    k.library()
    kernels = k
    yield
    assert k.device_status() == 0


def run_gemm(a, w, bias=None, **kw):
    dev = torch.device("cuda:0")
    out = kernels.gemm(a.to(dev), w.to(dev), bias=None if bias is None else bias.to(dev), **kw)
    torch.cuda.synchronize()
    return out.cpu()


# The reference's exact-arithmetic cases (hopper/tests.rs:179-225 shapes: K widths 64..256,
# a clipped M tile) plus multi-tile and ragged shapes.
@pytest.mark.parametrize("m,n,k", [
    (128, 128, 64), (128, 128, 128), (128, 128, 192), (128, 128, 256), (1, 128, 64),
    (133, 128, 192), (256, 256, 192), (384, 520, 328), (1000, 264, 72),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_dyadic_inputs_are_bit_exact(m, n, k, out_dtype):
    a, b = wl.dyadic_gemm_inputs(m, n, k)
    exact = (a.double() @ b.double()).float().to(out_dtype)
    for _ in range(3):  # repeated launches must not leak pipeline state
        out = run_gemm(a, b, out_dtype=out_dtype)
        assert torch.equal(out, exact)


@pytest.mark.parametrize("m,n,k", [(2309, 2312, 328), (4096, 2560, 64), (2432, 4104, 200)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_dyadic_inputs_on_cta_pairs(m, n, k, out_dtype):
    """Shapes with at least as many 256 x 256 tiles as SM pairs run on two-CTA clusters (one MMA
    over both CTAs' shared memory); an odd count of 128-row tiles leaves the last pair with one
    empty half, ragged edges clip.  Exact operands: any correct kernel matches bit for bit."""
    a, b = wl.dyadic_gemm_inputs(m, n, k)
    exact = (a.double() @ b.double()).float().to(out_dtype)
    for _ in range(2):
        out = run_gemm(a, b, out_dtype=out_dtype)
        assert torch.equal(out, exact)


def test_gated_form_on_cta_pairs():
    """In the gated form each CTA of the pair stages 64 up-weight and the matching 64 gate-weight
    columns of the tile."""
    a, wg, wu, _ = wl.mlp_inputs(2000, 256, 1304, 31)
    dev = torch.device("cuda:0")
    out = kernels.gemm(a.to(dev), wu.to(dev), b2=wg.to(dev), activation=kernels.ACT_SILU_GATE)
    torch.cuda.synchronize()
    assert_close_bf16(out.cpu(), wl.gated_oracle(a, wu, wg), max_ulp=1)


def test_output_outside_the_matrix_is_untouched():
    """Sentinel fill (reference.cu:16,39): only [m,n] of a wider allocation may change."""
    dev = torch.device("cuda:0")
    a, b = wl.dyadic_gemm_inputs(200, 136, 128)
    backing = torch.full((256, 192), -123.0, dtype=torch.bfloat16, device=dev)
    out = backing[:200, :136]
    kernels.gemm(a.to(dev), b.to(dev), out=out)
    torch.cuda.synchronize()
    host = backing.cpu()
    assert torch.equal(host[:200, :136], (a.double() @ b.double()).float().bfloat16())
    assert (host[200:] == -123.0).all() and (host[:, 136:] == -123.0).all()


@pytest.mark.parametrize("name", ["gemm_bias", "gemm_bias_relu", "gemm_matrix_bias", "gemm_silu"])
def test_golden_cases(golden, name):
    case = golden[name]
    a, w, bias = wl.gemm_inputs(case["m"], case["n"], case["k"], case["seed"], case["distribution"])
    mode = {"col": kernels.BIAS_COL_VECTOR, "matrix": kernels.BIAS_MATRIX}[case["bias_mode"]]
    if case["bias_mode"] == "matrix":
        bias = wl._normal((case["m"], case["n"]), 0.5, wl._gen(case["seed"] + 100))
    act = {None: kernels.ACT_NONE, "relu": kernels.ACT_RELU, "silu": kernels.ACT_SILU}[
        case["activation"]]
    out = run_gemm(a, w, bias, bias_mode=mode, activation=act)
    expected = case["expected"].view(torch.bfloat16)
    assert_close_bf16(out, expected, max_ulp=1)


def test_gated_golden_case(golden):
    case = golden["gated"]
    a, wg, wu, _ = wl.mlp_inputs(case["m"], case["d_model"], case["d_ff"], case["seed"])
    dev = torch.device("cuda:0")
    out = kernels.gemm(a.to(dev), wu.to(dev), b2=wg.to(dev), activation=kernels.ACT_SILU_GATE)
    torch.cuda.synchronize()
    assert_close_bf16(out.cpu(), case["expected"].view(torch.bfloat16), max_ulp=1)


def test_streamed_config_1024_uniform():
    """A[1024,1024] @ B[1024,1024] + bias[1024], U(-1,1): |y| reaches ~50, so the bound on the
    raw difference is the reference's atol=0.125, rtol=0.02 (python/tests/test_gpu.py:55)."""
    a, w, bias = wl.gemm_inputs(1024, 1024, 1024, 1234, "uniform")
    out = run_gemm(a, w, bias, bias_mode=kernels.BIAS_COL_VECTOR)
    expected = wl.gemm_oracle(a, w, bias)
    assert_close_bf16(out, expected, max_ulp=1)
    torch.testing.assert_close(out.float(), expected.float(), atol=0.125, rtol=0.02)


@pytest.mark.parametrize("m,n,k", [(16, 8192, 1024), (1, 4096, 2048), (100, 1000, 4096)])
def test_decode_time_shapes(m, n, k):
    """A few output rows against a large weight: the kernel streams the weight (one partly
    filled row tile, many column tiles; up to 32 rows through the form that splits K)."""
    a, w, bias = wl.gemm_inputs(m, n, k, 77, "normal")
    out = run_gemm(a, w, bias, bias_mode=kernels.BIAS_COL_VECTOR)
    assert_close_bf16(out, wl.gemm_oracle(a, w, bias), max_ulp=1, max_abs=2e-2)
    out32 = run_gemm(a, w, None, out_dtype=torch.float32)
    exact = (a.double() @ w.double()).float()
    assert (out32 - exact).norm() / exact.norm() < 1e-5


@pytest.mark.parametrize("m,n,k", [
    (16, 256, 512),      # one tile, two parts of four K blocks
    (1, 2048, 1024),     # 16 K blocks: four parts of four
    (16, 4096, 8192),    # eight parts (16 rows are handed over)
    (17, 8192, 4096),    # 17..32 rows: four parts at most, 32 rows handed over
    (32, 8200, 1000),    # ragged columns and a ragged last K block
    (9, 1032, 4104),     # five tiles, the last 8 columns wide; K blocks not a multiple of the parts
    (33, 4096, 2048),    # 33..64 rows: two warps of each CTA hand rows over, two parts
    (64, 8192, 1024),
    (50, 1000, 4096),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_few_rows_split_over_k_bit_exact(m, n, k, out_dtype):
    """Up to 64 output rows with fewer 256-column tiles than half the SMs: the CTAs of a cluster
    share a tile, each sums a part of K, and the first adds the parts in a fixed order.  Exact
    operands, so the sum must not depend on how K was cut, and repeated launches must agree."""
    a, b = wl.dyadic_gemm_inputs(m, n, k)
    exact = (a.double() @ b.double()).float().to(out_dtype)
    for _ in range(3):
        out = run_gemm(a, b, out_dtype=out_dtype)
        assert torch.equal(out, exact)


def test_few_rows_split_over_k_epilogue_and_determinism():
    """Bias, activation and row-vector bias run after the parts are added; two launches give the
    same bits (the order of the additions is fixed, not the order of arrival)."""
    a, w, bias = wl.gemm_inputs(16, 8192, 8192, 79, "normal")
    first = run_gemm(a, w, bias, bias_mode=kernels.BIAS_COL_VECTOR, activation=kernels.ACT_RELU)
    assert_close_bf16(first, wl.gemm_oracle(a, w, bias, "relu"), max_ulp=1, max_abs=2e-2)
    for _ in range(3):
        assert torch.equal(run_gemm(a, w, bias, bias_mode=kernels.BIAS_COL_VECTOR, activation=kernels.ACT_RELU), first)
    rows = wl._normal((16,), 0.5, wl._gen(80))
    out32 = run_gemm(a, w, rows, bias_mode=kernels.BIAS_ROW_VECTOR, out_dtype=torch.float32)
    exact = (a.double() @ w.double() + rows.double()[:, None]).float()
    assert (out32 - exact).norm() / exact.norm() < 1e-5


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_few_rows_split_over_k_ragged_columns_and_matrix_bias(out_dtype):
    """A column count that is no multiple of eight (the last eight-column store falls back to
    single elements), operands and output as views of wider allocations, a matrix side operand
    and SiLU, in the form that splits K."""
    dev = torch.device("cuda:0")
    m, n, k, pitch = 5, 1001, 2048, 1008
    a, w, _ = wl.gemm_inputs(m, pitch, k, 81, "normal")
    side = wl._normal((m, pitch), 0.5, wl._gen(82))
    backing = torch.full((8, pitch), -7.0, dtype=out_dtype, device=dev)
    kernels.gemm(a.to(dev), w.to(dev)[:, :n], bias=side.to(dev)[:, :n], bias_mode=kernels.BIAS_MATRIX,
                 activation=kernels.ACT_SILU, out=backing[:m, :n])
    torch.cuda.synchronize()
    host = backing.cpu()
    x = a.double() @ w.double()[:, :n] + side.double()[:, :n]
    expected = x * torch.sigmoid(x)
    if out_dtype == torch.float32:
        torch.testing.assert_close(host[:m, :n], expected.float(), rtol=1e-4, atol=1e-4)
    else:
        assert_close_bf16(host[:m, :n], expected.float().bfloat16(), max_ulp=1, max_abs=2e-2)
    assert (host[m:] == -7.0).all() and (host[:, n:] == -7.0).all()


@pytest.mark.parametrize("m,n,k", [(16, 3584, 8192), (24, 1000, 2048), (1, 128, 512)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_few_rows_gated_form_split_over_k(m, n, k, out_dtype):
    """The gated form with few rows and few tiles (a tensor-parallel shard of a SwiGLU projection
    at decode time): each CTA of the cluster sums its part of K for the up and the gate
    accumulator, the first CTA adds the parts and gates."""
    a, wg, wu, _ = wl.mlp_inputs(m, k, n, 83)
    dev = torch.device("cuda:0")
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    for _ in range(2):
        kernels.gemm(a.to(dev), wu.to(dev), b2=wg.to(dev), activation=kernels.ACT_SILU_GATE, out=out)
    torch.cuda.synchronize()
    if out_dtype == torch.float32:
        gate = a.double() @ wg.double()
        expected = (a.double() @ wu.double()) * (gate * torch.sigmoid(gate))
        torch.testing.assert_close(out.cpu(), expected.float(), rtol=1e-4, atol=1e-5)
    else:
        assert_close_bf16(out.cpu(), wl.gated_oracle(a, wu, wg), max_ulp=1)


def test_few_rows_output_outside_the_matrix_is_untouched():
    dev = torch.device("cuda:0")
    a, b = wl.dyadic_gemm_inputs(20, 1000, 2048)
    backing = torch.full((64, 1024), -123.0, dtype=torch.bfloat16, device=dev)
    kernels.gemm(a.to(dev), b.to(dev), out=backing[:20, :1000])
    torch.cuda.synchronize()
    host = backing.cpu()
    assert torch.equal(host[:20, :1000], (a.double() @ b.double()).float().bfloat16())
    assert (host[20:] == -123.0).all() and (host[:, 1000:] == -123.0).all()


@pytest.mark.parametrize("m,n,k", [(2048, 2304, 1024), (4096, 4096, 512)])
def test_bias_relu_many_tiles(m, n, k):
    a, w, bias = wl.gemm_inputs(m, n, k, 1235, "normal")
    out = run_gemm(a, w, bias, bias_mode=kernels.BIAS_COL_VECTOR, activation=kernels.ACT_RELU)
    rows = torch.arange(0, m, 37)
    expected = wl.gemm_oracle(a, w, bias, "relu", rows=rows)
    assert_close_bf16(out[rows], expected, max_ulp=1, max_abs=2e-2)
    # linearity in the bias where ReLU is inactive is checked through a second launch
    out2 = run_gemm(a, w, None)
    both = (out2.float() + bias.float()).clamp_min(0).bfloat16()
    assert_close_bf16(out, both, max_ulp=2, ulp_outlier_fraction=1e-3)


def test_row_vector_bias_and_fp32_output():
    a, w, _ = wl.gemm_inputs(300, 200, 136, 77, "normal")
    bias = wl._normal((300,), 0.5, wl._gen(78))
    out = run_gemm(a, w, bias, bias_mode=kernels.BIAS_ROW_VECTOR, out_dtype=torch.float32)
    expected = wl.gemm_oracle(a, w, bias, None, "row", out_dtype="fp32")
    torch.testing.assert_close(out, expected, rtol=1e-4, atol=1e-4)


def test_relu_special_values_in_epilogue():
    """x < 0 ? 0 : x keeps NaN, +inf and the sign of zero (pointwise/special.rs:3-6)."""
    dev = torch.device("cuda:0")
    a = torch.zeros(128, 64, dtype=torch.bfloat16)
    a[:, 0] = 1.0
    w = torch.zeros(64, 128, dtype=torch.bfloat16)
    special = torch.tensor([-float("inf"), -2.0, -0.0, 0.0, 2.0, float("inf"), float("nan"), 1e-8])
    bias = special.repeat(16).bfloat16()
    out = run_gemm(a, w, bias, bias_mode=kernels.BIAS_COL_VECTOR, activation=kernels.ACT_RELU)
    expected = torch.where(bias.float() < 0, torch.zeros(()), bias.float()).bfloat16()
    row = out[5]
    assert torch.equal(torch.isnan(row.float()), torch.isnan(expected.float()))
    ok = ~torch.isnan(expected.float())
    assert torch.equal(row[ok], expected[ok])


def test_invalid_arguments_are_rejected():
    dev = torch.device("cuda:0")
    a = torch.zeros(64, 60, dtype=torch.bfloat16, device=dev)  # K pitch not a multiple of 8
    b = torch.zeros(60, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(kernels.KernelError):
        kernels.gemm(a, b)
    with pytest.raises(ValueError):
        kernels.gemm(a.float(), b)


def test_batched_matches_the_single_launches():
    """One batched launch equals the per-entry launches bit for bit (same tiles, same order of
    accumulation), with a shared and a per-entry right operand, bias and activation."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(11)
    a = torch.randn(5, 200, 192, generator=g).bfloat16().to(dev)
    w = (torch.randn(5, 192, 264, generator=g) / 14).bfloat16().to(dev)
    bias = torch.randn(5, 264, generator=g).bfloat16().to(dev)
    out = kernels.gemm_batched(a, w, bias=bias, activation=kernels.ACT_RELU)
    for z in range(5):
        single = kernels.gemm(a[z], w[z], bias=bias[z], bias_mode=kernels.BIAS_COL_VECTOR, activation=kernels.ACT_RELU)
        assert torch.equal(out[z], single)
    shared = kernels.gemm_batched(a, w[0], out_dtype=torch.float32)
    for z in range(5):
        assert torch.equal(shared[z], kernels.gemm(a[z], w[0], out_dtype=torch.float32))
    torch.cuda.synchronize()


def test_per_head_projections_around_latent_attention():
    """The grouped products of the reference's batched-MLA fixtures: absorb
    q_nope[b,h,:128] @ W_DK[h] -> [b,h,512] and output t2[b,h,:512] @ W_DV[h] -> [b,h,128], the
    heads interleaved with the tokens in memory (batch stride below the row pitch), against
    float64 einsum rounded once."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(12)
    tokens, heads = 64, 128
    q_nope = torch.randn(tokens, heads, 128, generator=g).bfloat16()
    w_dk = (torch.randn(heads, 128, 512, generator=g) / 11.3).bfloat16()
    absorbed = torch.empty(tokens, heads, 512, dtype=torch.bfloat16, device=dev)
    kernels.gemm_batched(q_nope.to(dev).permute(1, 0, 2), w_dk.to(dev), out=absorbed.permute(1, 0, 2))
    expected = torch.einsum("thk,hkn->thn", q_nope.double(), w_dk.double()).float().bfloat16()
    assert_close_bf16(absorbed.cpu(), expected, max_ulp=1, max_abs=2e-2)
    t2 = torch.randn(tokens, heads, 512, generator=g).bfloat16()
    w_dv = (torch.randn(heads, 512, 128, generator=g) / 22.6).bfloat16()
    projected = torch.full((tokens, heads, 128), -123.0, dtype=torch.bfloat16, device=dev)
    kernels.gemm_batched(t2.to(dev).permute(1, 0, 2), w_dv.to(dev), out=projected.permute(1, 0, 2))
    expected = torch.einsum("thk,hkn->thn", t2.double(), w_dv.double()).float().bfloat16()
    assert_close_bf16(projected.cpu(), expected, max_ulp=1, max_abs=2e-2)
    # ragged: 37 tokens, 3 heads, rows clipped per head without touching the next head's rows
    small = torch.full((37, 3, 72), -123.0, dtype=torch.bfloat16, device=dev)
    x = torch.randn(37, 3, 40, generator=g).bfloat16()
    w = torch.randn(3, 40, 72, generator=g).bfloat16()
    kernels.gemm_batched(x.to(dev).permute(1, 0, 2), w.to(dev), out=small.permute(1, 0, 2))
    expected = torch.einsum("thk,hkn->thn", x.double(), w.double()).float().bfloat16()
    assert_close_bf16(small.cpu(), expected, max_ulp=1)
