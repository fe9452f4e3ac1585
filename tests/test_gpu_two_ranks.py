"""The sharded path on two real GPUs, when the machine has them: constants replicated by the library's NCCL
broadcast, rows computed per rank, the output assembled by the library's all-gather - against the unsharded run."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def test_two_ranks_replicate_constants_and_gather_the_output():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                           "127.0.0.1", "--master-port", "29541", str(ROOT / "tests" / "workers" / "two_rank_gather.py")],
                          capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    for rank in (0, 1):
        assert f"rank {rank} own_rows_equal=True gathered_equal=True" in proc.stdout, proc.stdout[-2000:]
