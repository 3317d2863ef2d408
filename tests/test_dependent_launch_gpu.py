"""Kernels are launched with programmatic stream serialization: a kernel's thread blocks may start
while the previous kernel of the stream is still running and wait, after their set-up, for its
results.  Chains of dependent kernels, launched directly and replayed from a CUDA graph with the
input rewritten before every replay, must see each other's fresh results (B200 only)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def kernels():
    from trinity_lowering import kernels as k
    k.library()
    yield k
    torch.cuda.synchronize()
    assert k.device_status() == 0


def chain(k, x, gain, w, y, z, s):
    k.rmsnorm(x, gain, 1e-6, out=y)
    k.gemm(y, w, out=z)
    k.softmax(z, out=s)


def expected(x, gain, w):
    xf = x.float()
    y = (xf / torch.sqrt((xf * xf).mean(dim=1, keepdim=True) + 1e-6) * gain.float()).bfloat16()
    z = (y.float() @ w.float()).bfloat16()
    return z.float(), torch.softmax(z.float(), dim=1)


@pytest.mark.parametrize("rows", [16, 300])
@pytest.mark.parametrize("replayed", [False, True])
def test_chained_kernels_see_fresh_results(kernels, rows, replayed):
    """RMSNorm -> GEMM -> softmax over intermediates in global memory (16 rows: the GEMM form
    that splits K over a cluster; 300 rows: ordinary tiles).  Forty rounds with new inputs."""
    k = kernels
    cols, n = 2048, 2048
    g = torch.Generator(device=DEV)
    g.manual_seed(5)
    gain = (1.0 + 0.1 * torch.randn(cols, generator=g, device=DEV)).bfloat16()
    w = (torch.randn(cols, n, generator=g, device=DEV) / 45.0).bfloat16()
    x = torch.empty(rows, cols, dtype=torch.bfloat16, device=DEV)
    y = torch.empty_like(x)
    z = torch.empty(rows, n, dtype=torch.bfloat16, device=DEV)
    s = torch.empty_like(z)
    stream = torch.cuda.Stream(device=DEV)
    with torch.cuda.stream(stream):
        x.copy_(torch.randn(rows, cols, generator=g, device=DEV))
        chain(k, x, gain, w, y, z, s)
        stream.synchronize()
        graph = None
        if replayed:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                chain(k, x, gain, w, y, z, s)
        for round_ in range(40):
            fresh = torch.randn(rows, cols, generator=g, device=DEV) * (1.0 + round_ % 3)
            x.copy_(fresh)
            if replayed:
                graph.replay()
            else:
                chain(k, x, gain, w, y, z, s)
            got_z, got = z.float().clone(), s.float().clone()
            want_z, want = expected(x, gain, w)
            stream.synchronize()
            # the products are of order one; a stale input or intermediate (the previous round's)
            # would differ by as much, a BF16 rounding flip in y moves them by about 1e-2
            assert (got_z - want_z).abs().max().item() < 6e-2, round_
            assert ((got - want).abs() <= 0.08 * want + 1e-6).all(), round_
