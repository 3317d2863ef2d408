"""The give-up path of a bounded in-kernel wait, exercised without faulting the GPU (B200 only).

One rank of the two-rank peer-memory all-reduce is launched over local buffers while the other
rank's kernel never runs, so the flag it waits for is never written.  With the wait budget set to
about a millisecond the kernel gives up, records the wait's site in the device status word and
returns; the artifact-level status call reports the timeout; the context stays usable and the
flag pad's counters are back at zero."""
import pytest
import torch

import trinity_lowering as tl
from oracle import workloads as wl
from parity import assert_close_bf16
from trinity_lowering import plans

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    from trinity_lowering import kernels as k
    k.library()
    torch.cuda.synchronize()
    assert k.device_status() == 0
    a, w, bias = wl.gemm_inputs(256, 256, 128, 5, "normal")
    artifact = tl.compile(tl.emit(plans.gemm_bias(256, 256, 128)))
    module = tl.load(artifact, DEV)
    artifact.close()
    execution = module.prepare({"A": a.to(DEV), "W": w.to(DEV), "bias": bias.to(DEV)})
    mine = torch.ones(64, 64, dtype=torch.bfloat16, device=DEV)
    theirs = torch.ones(64, 64, dtype=torch.bfloat16, device=DEV)
    pads = [torch.zeros(k.allreduce_flag_words(), dtype=torch.int32, device=DEV) for _ in range(2)]
    try:
        k.set_wait_budget(2_000_000)   # about one millisecond
        k.allreduce([mine.data_ptr(), theirs.data_ptr()], [p.data_ptr() for p in pads], 64, 64, rank=0, epoch=1)
        torch.cuda.synchronize()       # returns: the kernel left its wait by itself
        # the artifact-level status call sees the recorded timeout
        execution.run()
        with pytest.raises(tl.RuntimeFailure) as failure:
            execution.wait(timeout=30)
        assert failure.value.code == -5   # TRINITY_SM100_E_TIMEOUT
        status = k.device_status(clear=True)
        assert status & 0x80000000 and (status & 0xFFFF) == 0x701, hex(status)
    finally:
        k.set_wait_budget(0)
    assert k.device_status() == 0
    # nothing was published, the data was not touched, and the counters are back at zero
    assert torch.equal(mine.cpu(), torch.ones(64, 64, dtype=torch.bfloat16))
    words = pads[0].cpu()
    assert words[24].item() == 0 and words[25].item() == 0 and words[8].item() == 0 and words[16].item() == 0
    # the same context launches and completes further work
    out = k.gemm(a.to(DEV), w.to(DEV), bias=bias.to(DEV), bias_mode=k.BIAS_COL_VECTOR)
    torch.cuda.synchronize()
    assert_close_bf16(out.cpu(), wl.gemm_oracle(a, w, bias), max_ulp=1)
    assert k.device_status() == 0
    with pytest.raises(k.KernelError):
        k.allreduce([mine.data_ptr(), theirs.data_ptr()], [p.data_ptr() for p in pads], 64, 64, rank=0, epoch=0)
    with pytest.raises(tl.RuntimeFailure):   # the execution whose completion failed closes and says so
        execution.close()
    assert execution._closed
    module.close()
