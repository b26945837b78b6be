"""Multi-GPU paths on real GPUs (skipped with fewer than two): N-sharded linear with the all-gather folded into the GEMM epilogue (peer stores into symmetric
memory) against the NCCL all-gather form and the unsharded product, expert-parallel routed layer against the single-GPU layer. Ranks are child processes
(one per GPU, NCCL); nothing here waits on another rank inside a kernel except the bounded barrier of the symmetric-memory handle."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_cases():
    env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE) + os.pathsep + os.environ.get("PYTHONPATH", ""), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(HERE, "multi_rank_cases.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "MULTI_RANK_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
