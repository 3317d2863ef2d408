"""One GPU rank of the persistent all-gather test (launched by tests/test_gather_gpu.py under
torchrun).  The scenario of the reference's distributed worker
(python/tests/distributed_worker.py:14-60 there): a rank-major all-gather plan along axis 0 and
1, compiled to a persistent artifact, loaded with the world, run ten times, then captured in a
CUDA Graph and replayed twenty times; the result must equal the concatenation bit for bit."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
for entry in (ROOT, ROOT / "trinity-be_b200", ROOT / "tests"):
    sys.path.insert(0, str(entry))

import torch  # noqa: E402

import trinity_lowering as tl  # noqa: E402
from trinity_lowering import kernels as k  # noqa: E402
from trinity_lowering import plans  # noqa: E402


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    world = tl.World.from_torchrun(timeout=60)
    with torch.inference_mode():
        for axis in (0, 1):
            artifact = tl.compile(tl.emit(plans.gather(axis=axis, world_size=world.size)))
            module = tl.load(artifact, world.device, world)
            io = module.allocate_io()
            x = io.inputs["X"]

            def pattern(rank):
                return (torch.arange(x.numel(), device=world.device).reshape(x.shape) % 64 + rank * 64).bfloat16()
            x.copy_(pattern(world.rank))
            world.record_stream(x)
            execution = module.prepare(io.inputs, out=io.output)
            expected = torch.cat([pattern(r) for r in range(world.size)], dim=axis)
            for _ in range(10):
                execution.run()
            execution.wait(30)
            assert torch.equal(execution.output, expected), f"axis {axis}: gathered result differs"
            # new shard contents are picked up by the next run (the buffers' addresses are static)
            x.copy_(pattern(world.rank) + 1)
            world.barrier()
            execution.run()
            execution.wait(30)
            assert torch.equal(execution.output, torch.cat([pattern(r) + 1 for r in range(world.size)], dim=axis))
            x.copy_(pattern(world.rank))
            world.barrier()

            stream = torch.cuda.Stream(device=world.device)
            stream.wait_stream(torch.cuda.current_stream(world.device))
            graph = tl.Graph.capture(lambda: execution.run().clone(), executions=[execution], stream=stream)
            with torch.cuda.stream(stream):
                for _ in range(20):
                    graph.replay()
            graph.wait(30)
            assert torch.equal(graph.output, expected), f"axis {axis}: replayed result differs"
            assert k.device_status() == 0
            graph.close()
            execution.close()
            module.close()
            artifact.close()
            del x, io
            world.barrier()
    print(f"rank {world.rank} ok", flush=True)
    world.close()
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
