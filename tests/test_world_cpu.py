"""Two-rank Gloo tests of the World control plane on CPU: staged agreement, failure
propagation to every rank, terminal state, heartbeat loss.  Failures are injected on the host
(an exception, a mismatching signature, a rank that leaves between steps); no GPU is involved."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def run(scenario, port, timeout="20"):
    env = dict(os.environ, WORLD_TIMEOUT=timeout)
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
               "--master-addr", "127.0.0.1", "--master-port", str(port),
               str(ROOT / "tests" / "world_worker.py"), scenario]
    return subprocess.run(command, capture_output=True, text=True, timeout=180, env=env)


def test_ranks_agree_and_exchange():
    result = run("agree", 29611)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "rank 0 ok" in result.stdout and "rank 1 ok" in result.stdout


def test_signature_mismatch_fails_every_rank():
    result = run("signature_mismatch", 29612)
    assert result.returncode == 0, result.stdout + result.stderr
    assert result.stdout.count("saw disagreement") == 2


def test_failure_on_one_rank_reaches_all_and_is_terminal():
    result = run("one_rank_fails", 29613)
    assert result.returncode == 0, result.stdout + result.stderr
    assert result.stdout.count("saw the failure") == 2
    assert result.stdout.count("world is terminal") == 2


def test_silent_peer_is_noticed_through_the_heartbeat():
    result = run("peer_stops", 29614, timeout="2")
    assert "rank 0 noticed the silent peer" in result.stdout, result.stdout + result.stderr
