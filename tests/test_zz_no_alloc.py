"""The allocation-free MLA decode entry point (B200 only).

Some callers of the kernel library cannot provide scratch memory: a streamed artifact's launch
function gets only the plan's buffers and may run under CUDA-Graph stream capture, so it can
neither pass a workspace nor allocate one.  ``trinity_sm100_mla_decode_bf16_noalloc`` serves them
from a fixed array inside the library.  It must give what the ordinary entry point gives, on
back-to-back calls that reuse the array, and refuse requests that do not fit.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import math

import pytest
import torch

from oracle import workloads as wl
from parity import assert_close_bf16

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCALE = 1.0 / math.sqrt(192.0)


def test_matches_the_ordinary_entry_point_on_two_calls_in_a_row():
    from trinity_lowering import kernels as k
    k.library()
    calls = [(3, 128, 1024, 4, 501), (2, 64, 640, 3, 502)]   # batch, heads, seq, splits, seed
    for batch, heads, seq, splits, seed in calls:
        q, cache = wl.mla_inputs(batch, heads, seq, 576, seed)
        qd, cd = q.to(DEV), cache.to(DEV)
        assert k.mla_scratch_bytes(batch, heads, 512, splits) > 0      # the scratch path is used
        out = torch.full((batch, heads, 512), float("nan"), dtype=torch.bfloat16, device=DEV)
        k.mla_decode_noalloc(qd, cd, SCALE, kv_splits=splits, out=out)
        expected = k.mla_decode(qd, cd, SCALE, kv_splits=splits)
        torch.cuda.synchronize()
        assert_close_bf16(out.cpu(), expected.cpu(), max_ulp=None, max_abs=2e-2)
        assert_close_bf16(out.cpu(), wl.mla_oracle(q, cache, SCALE, 512), max_ulp=None,
                          max_abs=2e-2)
    assert k.device_status() == 0


def test_refuses_what_does_not_fit_the_built_in_array():
    from trinity_lowering import kernels as k
    batch, heads, seq, splits = 64, 128, 4096, 4
    assert k.mla_scratch_bytes(batch, heads, 512, splits) > k.MLA_STATIC_SCRATCH_BYTES
    q = torch.zeros(batch, heads, 576, dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros(batch, seq, 576, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(k.KernelError, match="scratch bytes"):
        k.mla_decode_noalloc(q, cache, SCALE, kv_splits=splits)
