"""KV-head-parallel decode on 2 (and, when present, 4 and 8) GPUs of one node over NCCL."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_decode_matches_unsharded(built_lib, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", "29517",
           str(ROOT / "tests" / "multi_gpu_worker.py")]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "multi_gpu_worker ok" in run.stdout


def test_absent_rank_times_out_instead_of_hanging(built_lib):
    """Host-made failure: one rank skips a gather step; the other's bounded wait reports it."""
    import os
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29518",
           str(ROOT / "tests" / "multi_gpu_worker.py"), "--timeout-case"]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "multi_gpu_worker ok" in run.stdout
