"""Row-parallel SharQ linear with the in-switch (multimem) all-reduce on two or more GPUs.
Skips on a single-GPU box.  The ranks run as child processes (tests/tp_gpu_worker.py)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def test_row_parallel_multimem_allreduce():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "tp_gpu_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240, cwd=ROOT)
    assert "TP_GPU_WORKER_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
