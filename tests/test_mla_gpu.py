"""Batched MLA decode through the C ABI versus the CPU oracle (B200 only).

Tolerance: the path's stated floating-point bar, rel-L2 <= 1e-2 and max-abs <= 2e-2 against
the FP32 oracle rounded to BF16.  Probabilities are rounded to BF16 before the value product
(as in any fused attention), so a per-element ulp bound does not apply to outputs that are
weighted means close to zero."""
import math

import pytest
import torch

from oracle import workloads as wl
from parity import assert_close_bf16

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCALE = 1.0 / math.sqrt(192.0)


@pytest.fixture(scope="module")
def kernels():
    from trinity_lowering import kernels as k
    k.library()
    yield k
    assert k.device_status() == 0


def test_golden_case(kernels, golden):
    case = golden["mla"]
    q, cache = wl.mla_inputs(case["batch"], case["heads"], case["seq"], case["d_qk"], case["seed"])
    for splits in (1, 2, 3):
        out = kernels.mla_decode(q.to(DEV), cache.to(DEV), case["scale"], kv_splits=splits).cpu()
        assert_close_bf16(out, case["expected"].view(torch.bfloat16), max_ulp=None, max_abs=2e-2)


@pytest.mark.parametrize("batch,heads,seq,splits", [
    (1, 128, 32, 1), (2, 128, 64, 1), (1, 128, 4096, 1), (3, 128, 1000, 0), (2, 64, 257, 2),
    (1, 16, 2048, 4), (4, 128, 512, 3), (1, 128, 40, 2),
    (1, 1, 1, 0), (2, 128, 63, 1), (1, 7, 65, 2), (3, 128, 129, 0), (150, 8, 64, 0),
])
def test_against_oracle(kernels, batch, heads, seq, splits):
    q, cache = wl.mla_inputs(batch, heads, seq, 576, 1237 + seq)
    out = kernels.mla_decode(q.to(DEV), cache.to(DEV), SCALE, kv_splits=splits).cpu()
    expected = wl.mla_oracle(q, cache, SCALE, 512)
    assert_close_bf16(out, expected, max_ulp=None, max_abs=2e-2)


@pytest.mark.parametrize("batch,heads,seq", [
    (5, 128, 1000),     # clusters own parts of two sequences; ragged last chunk
    (9, 128, 1536),     # three-chunk pieces, most sequences cut twice
    (100, 32, 320),     # more sequences than SM pairs: several whole sequences per cluster
    (1, 128, 8192),     # one sequence over many clusters
])
@pytest.mark.parametrize("mode", [-1, 0])
def test_balanced_and_automatic_schedule(kernels, batch, heads, seq, mode):
    """kv_splits = -1: the (sequence, chunk) grid is cut into equal runs, one per cluster; a
    cluster then works through pieces of several sequences with one set of barriers.
    kv_splits = 0: the library chooses between that and equal splits."""
    q, cache = wl.mla_inputs(batch, heads, seq, 576, 99 + seq)
    out = kernels.mla_decode(q.to(DEV), cache.to(DEV), SCALE, kv_splits=mode).cpu()
    picks = sorted({0, batch // 2, batch - 1})
    expected = wl.mla_oracle(q, cache, SCALE, 512, batches=picks)
    assert_close_bf16(out[picks], expected, max_ulp=None, max_abs=2e-2)
    # every sequence, not only the picked ones, against the one-cluster-per-sequence path
    single = kernels.mla_decode(q.to(DEV), cache.to(DEV), SCALE, kv_splits=1).cpu()
    assert_close_bf16(out, single, max_ulp=None, max_abs=2e-2)


def test_negative_scale(kernels):
    """A negative scale is applied by flipping the query's sign on its way into tensor memory."""
    q, cache = wl.mla_inputs(2, 128, 256, 576, 777)
    out = kernels.mla_decode(q.to(DEV), cache.to(DEV), -SCALE, kv_splits=1).cpu()
    expected = wl.mla_oracle(q, cache, -SCALE, 512)
    assert_close_bf16(out, expected, max_ulp=None, max_abs=2e-2)


def test_rescale_path_with_growing_scores(kernels):
    """Scores that grow along the sequence force the accumulator rescale again and again."""
    q, cache = wl.mla_inputs(1, 128, 1024, 576, 4242)
    ramp = torch.linspace(0.2, 3.0, 1024).view(1, 1024, 1)
    cache = (cache.float() * ramp).bfloat16()
    q = (q.float() * 2).bfloat16()
    out = kernels.mla_decode(q.to(DEV), cache.to(DEV), SCALE, kv_splits=1).cpu()
    expected = wl.mla_oracle(q, cache, SCALE, 512)
    # outputs reach |y| ~ 10 here, where one BF16 ulp is 0.0625: bound the error by one ulp of
    # the largest output instead of the O(1)-output bound
    top = expected.float().abs().max().item()
    assert_close_bf16(out, expected, max_ulp=None, max_abs=2.0 ** (math.floor(math.log2(top)) - 7))


@pytest.mark.parametrize("gain", [16.0, 64.0])
def test_large_logits(kernels, gain):
    """Queries scaled by 16 and 64 and a cache whose positions carry different gains: scaled
    logits reach several hundred, the softmax is sharply peaked, and an error of the score
    exchange between the two CTAs that is relative to the partial scores' magnitude would show
    directly in the weights.  Checked at the path's stated bar without loosening it."""
    q, cache = wl.mla_inputs(2, 128, 1024, 576, 555)
    q = (q.float() * gain).bfloat16()
    # gains below one keep the outputs (values of the few positions the softmax picks) of order
    # one, where the max-abs bound of 2e-2 is meaningful for BF16 results
    position_gain = torch.linspace(0.2, 0.8, 1024).view(1, 1024, 1)
    cache = (cache.float() * position_gain).bfloat16()
    for splits in (1, 2):
        out = kernels.mla_decode(q.to(DEV), cache.to(DEV), SCALE, kv_splits=splits).cpu()
        expected = wl.mla_oracle(q, cache, SCALE, 512)
        assert_close_bf16(out, expected, max_ulp=None, max_abs=2e-2)


def test_heads_of_very_different_magnitude(kernels):
    """Rows of very different magnitude in one tile: the exchange between the two CTAs scales
    every head's partial scores by that head's own largest magnitude."""
    q, cache = wl.mla_inputs(1, 128, 512, 576, 556)
    head_gain = torch.cat([torch.full((64,), 1.0), torch.linspace(2.0, 12.0, 64)]).view(1, 128, 1)
    q = (q.float() * head_gain).bfloat16()
    out = kernels.mla_decode(q.to(DEV), cache.to(DEV), SCALE, kv_splits=1).cpu()
    assert_close_bf16(out, wl.mla_oracle(q, cache, SCALE, 512), max_ulp=None, max_abs=2e-2)


def test_full_size_properties(kernels):
    """batch 64 x 128 heads x 4096 positions: oracle on two batches, and the convexity
    property: with a cache whose value part is constant per batch, the output is that constant."""
    q, cache = wl.mla_inputs(64, 128, 4096, 576, 1237)
    qd, cd = q.to(DEV), cache.to(DEV)
    out = kernels.mla_decode(qd, cd, SCALE)
    picks = [0, 37]
    expected = wl.mla_oracle(q, cache, SCALE, 512, batches=picks)
    assert_close_bf16(out[picks].cpu(), expected, max_ulp=None, max_abs=2e-2)
    # split invariance: 1 split and 2 splits agree to rounding
    out2 = kernels.mla_decode(qd, cd, SCALE, kv_splits=2)
    assert_close_bf16(out2.cpu(), out.cpu(), max_ulp=None, max_abs=2e-2)
    const = torch.linspace(-1, 1, 512).bfloat16()
    cd[:, :, :512] = const.to(DEV)
    flat = kernels.mla_decode(qd, cd, SCALE).cpu()
    assert (flat.float() - const.float()).abs().max().item() <= 1.0 / 128


def test_decode_between_its_per_head_projections(kernels):
    """The whole latent-attention step of the reference's batched-MLA fixtures
    (tests/fixtures/batched_mla/batched_mla_postprocessed_stage14.txt:19-68, 208-241): absorb
    q_nope through W_DK per head straight into the query's latent columns, decode over the
    compressed cache, project the result through W_DV per head.  Three launches, BF16 between
    them; the oracle rounds at the same points."""
    g = torch.Generator().manual_seed(2024)
    batch, heads, seq = 4, 128, 640
    q_nope = torch.randn(batch, heads, 128, generator=g).bfloat16()
    q_rope = torch.randn(batch, heads, 64, generator=g).bfloat16()
    w_dk = (torch.randn(heads, 128, 512, generator=g) / math.sqrt(128)).bfloat16()
    w_dv = (torch.randn(heads, 512, 128, generator=g) / math.sqrt(512)).bfloat16()
    cache = torch.randn(batch, seq, 576, generator=g).bfloat16()
    q = torch.empty(batch, heads, 576, dtype=torch.bfloat16, device=DEV)
    q[:, :, 512:] = q_rope.to(DEV)
    kernels.gemm_batched(q_nope.to(DEV).permute(1, 0, 2), w_dk.to(DEV), out=q[:, :, :512].permute(1, 0, 2))
    latent = kernels.mla_decode(q, cache.to(DEV), SCALE)
    out = torch.empty(batch, heads, 128, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_batched(latent.permute(1, 0, 2), w_dv.to(DEV), out=out.permute(1, 0, 2))

    absorbed = torch.einsum("bhk,hkn->bhn", q_nope.double(), w_dk.double()).float().bfloat16()
    assert_close_bf16(q[:, :, :512].cpu(), absorbed, max_ulp=1, max_abs=2e-2)
    assert torch.equal(q[:, :, 512:].cpu(), q_rope)          # the rope columns are untouched
    expected_latent = wl.mla_oracle(torch.cat([absorbed, q_rope], dim=2), cache, SCALE, 512)
    expected = torch.einsum("bhk,hkn->bhn", expected_latent.double(), w_dv.double()).float().bfloat16()
    assert_close_bf16(out.cpu(), expected, max_ulp=None, max_abs=2e-2)


def test_rejects_unsupported_geometry(kernels):
    q = torch.zeros(1, 128, 512, dtype=torch.bfloat16, device=DEV)
    c = torch.zeros(1, 64, 512, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError):
        kernels.mla_decode(q, c, SCALE)
