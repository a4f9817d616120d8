"""Tensor parallelism of the 27B engine on 2 (and 4) GPUs of one node: one process per GPU under torchrun,
the all-reduce inside the megakernel over peer mailboxes.  Skipped where the machine has one GPU."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(n, fmt, M, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="4")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "tp_worker.py"), fmt, str(M)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("n,fmt,M", [(2, "mxfp4", 2), (2, "bf16", 5), (4, "mxfp4", 1)])
def test_ranks_agree_with_the_oracle_and_with_each_other(n, fmt, M):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    p = _run(n, fmt, M, 29600 + n + M)
    out = p.stdout + p.stderr
    assert p.returncode == 0, out[-3000:]
    for r in range(n):
        assert f"TP_OK {r}" in out, out[-3000:]
