"""Pose sharding over two GPUs with NCCL (skipped on boxes with a single GPU; the host logic is
covered on CPU ranks with gloo in test_host_logic.py)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_rank_sharded_projection_and_backprojection(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = Path(__file__).resolve().parent / "multi_gpu_check.py"
    # small slabs (4 planes of the box-32 accumulator each): the final stage of the sharded
    # back-projection then really runs slab group by slab group, with the fold and the reduce of a
    # finished group on the second stream
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", B200PROJ_SLAB_MIN_MB="0", B200PROJ_SLAB_MB="0.03")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29537", str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "MULTI-OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
