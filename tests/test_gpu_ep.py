"""Expert-parallel decode on 2 GPUs equals the single-GPU engine token for token.  Needs two
devices: on a one-GPU box the test is skipped (the host-side partition logic is covered on CPU
by tests/test_ep_host.py)."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows_per_rank", [4, 12])
def test_expert_parallel_tokens_match_single_gpu(rows_per_rank):
    """4 rows per rank: the one-to-eight-row kernels on the gathered rows; 12: the many-row router and expert kernels."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", EP_ROWS_PER_RANK=str(rows_per_rank))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "ep_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0 and "EP_CHECK_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
