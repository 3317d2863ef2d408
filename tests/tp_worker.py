"""One GPU rank of the tensor-parallel MLP test (launched by tests/test_tp_mlp_gpu.py)."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
for entry in (ROOT, ROOT / "trinity-be_b200", ROOT / "tests"):
    sys.path.insert(0, str(entry))

import torch  # noqa: E402

from oracle import workloads as wl  # noqa: E402
from parity import assert_close_bf16  # noqa: E402
from trinity_lowering import kernels as k  # noqa: E402
from trinity_lowering.tp_mlp import TensorParallelMLP  # noqa: E402
from trinity_lowering.world import World  # noqa: E402


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    world = World.from_torchrun(timeout=60.0)
    dev = world.device
    m, d_model, d_ff = 512, 1024, 2048
    x, wg, wu, wd = wl.mlp_inputs(m, d_model, d_ff, 1238)
    shards = [t.to(dev) for t in TensorParallelMLP.shard_weights(wg, wu, wd, world.rank, world.size)]
    variants = [TensorParallelMLP(world, m, d_model, d_ff, *shards, fused=True),
                TensorParallelMLP(world, m, d_model, d_ff, *shards, fused=False)]
    xd = x.to(dev)
    expected = None
    for step in range(6):  # repeated steps reuse the flags with a growing epoch
        mlp = variants[step % 2]
        out = mlp.forward(xd)
        torch.cuda.synchronize()
        assert k.device_status() == 0
        if expected is None:
            # oracle of the sharded computation: BF16 partial outputs summed in FP32, rounded once
            partials = []
            for r in range(world.size):
                g, u, d = TensorParallelMLP.shard_weights(wg, wu, wd, r, world.size)
                partials.append(wl.mlp_oracle(x, g, u, d).float())
            expected = sum(partials).bfloat16()
        # two chained GEMMs with a BF16 hidden activation: the path's stated bar (rel-L2 <= 1e-2,
        # max-abs <= 2e-2); a one-ulp flip in H moves small outputs by more than one ulp
        assert_close_bf16(out.cpu(), expected, max_ulp=None, max_abs=2e-2)
        if step == 1:   # fused and unfused add the same BF16 partials in the same order
            assert torch.equal(variants[0].output, variants[1].output)
        world.barrier()
    # plain all-reduce of a ragged matrix against an FP32 sum
    buffer = world.allocate((301, 264), torch.bfloat16)
    torch.manual_seed(100 + world.rank)
    buffer.tensor.copy_(torch.randn(301, 264, device=dev))
    local = buffer.tensor.clone()
    gathered = [torch.empty_like(local) for _ in range(world.size)]
    torch.distributed.all_gather(gathered, local)
    world.barrier()
    world.all_reduce(buffer)
    torch.cuda.synchronize()
    total = torch.zeros(301, 264, device=dev)
    for g in gathered:
        total += g.float()
    assert torch.equal(buffer.tensor, total.bfloat16()), "all-reduce differs from the FP32 sum in rank order"
    assert k.device_status() == 0
    world.barrier()
    print(f"rank {world.rank} ok", flush=True)
    world.close()
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
