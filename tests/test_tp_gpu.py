"""Row-parallel SharQ linear with the in-switch (multimem) all-reduce on two or more GPUs.
Skips on a single-GPU box.  The ranks run as child processes (tests/tp_gpu_worker.py)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _run_ranks(worker: str, port: int, marker: str):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / worker)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert marker in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


def test_row_parallel_multimem_allreduce():
    _run_ranks("tp_gpu_worker.py", 29533, "TP_GPU_WORKER_OK")


def test_layer_transition_equals_single_gpu_prepare():
    """reduce-scatter + residual add + RMSNorm prepare + all-gather of the packed activation in
    one kernel per GPU: byte-identical to the single-GPU RMSNorm prepare of the gathered rows."""
    _run_ranks("tp_sp_worker.py", 29534, "TP_SP_WORKER_OK")
