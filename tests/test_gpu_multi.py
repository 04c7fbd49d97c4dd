"""2-GPU test of the column-split GEMM + exchange through the library's communicator, and of requests partitioned
over the ranks (skipped on a single-GPU box)."""
import os
import subprocess
import sys

import pytest

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


def test_colsplit_gemm_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533",
                        os.path.join(entry.ROOT, "tests", "multi_gpu_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
