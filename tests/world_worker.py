"""Worker for tests/test_world_cpu.py: one CPU rank of a two-rank Gloo world.
Scenarios exercise the control plane only (agreement, failure propagation, heartbeat)."""
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "trinity-be_b200"))

import torch.distributed as dist  # noqa: E402

from trinity_lowering.errors import DistributedFailure  # noqa: E402
from trinity_lowering.world import World  # noqa: E402


def main():
    scenario = sys.argv[1]
    world = World.from_torchrun(timeout=float(os.environ.get("WORLD_TIMEOUT", "20")))
    rank = world.rank
    if scenario == "agree":
        assert world._stage("step", lambda: rank * 10, signature=[1, 2]) == rank * 10
        assert world._exchange("values", rank) == [0, 1]
        world.barrier()
        print(f"rank {rank} ok")
    elif scenario == "signature_mismatch":
        try:
            world._stage("step", lambda: None, signature=["a"] if rank == 0 else ["b"])
        except DistributedFailure as e:
            assert "disagree" in str(e)
            print(f"rank {rank} saw disagreement")
        else:
            raise SystemExit("expected DistributedFailure")
    elif scenario == "one_rank_fails":
        def step():
            if rank == 1:
                raise ValueError("injected failure on rank 1")
            return 7
        try:
            world._stage("step", step)
        except DistributedFailure as e:
            assert "rank 1" in str(e) and "injected failure" in str(e)
            print(f"rank {rank} saw the failure")
        else:
            raise SystemExit("expected DistributedFailure")
        try:  # the world is terminal afterwards
            world._stage("next", lambda: None)
        except DistributedFailure:
            print(f"rank {rank} world is terminal")
        else:
            raise SystemExit("a failed world must stay failed")
    elif scenario == "peer_stops":
        # rank 1 leaves between steps; rank 0 notices through the heartbeat
        world.barrier()
        if rank == 1:
            world.close()
            time.sleep(4.0)
            print("rank 1 left")
            os._exit(0)
        deadline = time.time() + 15
        while time.time() < deadline:
            try:
                world.check_peers()
            except DistributedFailure as e:
                assert "rank 1" in str(e)
                print("rank 0 noticed the silent peer")
                os._exit(0)
            time.sleep(0.2)
        raise SystemExit("heartbeat loss was not noticed")
    world.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
