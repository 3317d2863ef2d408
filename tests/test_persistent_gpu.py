"""Persistent (multi-GPU) artifacts on two B200s: the all-gather plan and the row-parallel GEMM +
all-reduce plan through emit, compile, load with a world, run and CUDA-Graph replay (skipped with
fewer GPUs).  Ranks run as child processes; NVLS is off in NCCL and the kernels use plain peer
loads and stores."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def two_ranks(worker, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / worker)]
    result = subprocess.run(command, capture_output=True, text=True, timeout=600, env=env)
    assert result.returncode == 0, result.stdout[-4000:] + result.stderr[-4000:]
    assert "rank 0 ok" in result.stdout and "rank 1 ok" in result.stdout


needs_two_gpus = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                    reason="needs at least two GPUs")


@needs_two_gpus
def test_all_gather_plan_two_ranks():
    two_ranks("gather_worker.py", 29641)


@needs_two_gpus
def test_row_parallel_gemm_all_reduce_plan_two_ranks():
    two_ranks("row_parallel_worker.py", 29642)
