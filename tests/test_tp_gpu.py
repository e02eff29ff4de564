"""Row-parallel contraction with the sum over ranks formed inside the kernel, on 2 (or more) GPUs of
one box: one process per GPU, started through torch.distributed.run.  Skipped on a single-GPU box;
the one-rank case is covered in test_gpu_parity.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_in_kernel_sum_over_ranks():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 4 if n >= 4 else 2
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_in_kernel_sum_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", "29531", worker],
                          capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and "TP_IN_KERNEL_SUM OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-4000:]
