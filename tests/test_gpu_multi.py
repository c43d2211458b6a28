"""Column-parallel layer on 2+ GPUs: fused push gather and NCCL baseline against
the oracle.  Needs two visible GPUs; on a one-GPU box it is skipped (the CPU
suite covers the host logic with gloo ranks, test_sharding_cpu.py)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus(q4b):
    return q4b.library().q4b_device_count()


@pytest.mark.parametrize("which", ["small", "27b"])
def test_column_parallel_matches_oracle(q4b, which):
    count = _gpus(q4b)
    if count < 2:
        pytest.skip("needs at least two GPUs")
    ranks = 2 if count < 4 else 4
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
               "--master-addr", "127.0.0.1", "--master-port", "29611",
               os.path.join(ROOT, "tests", "multi_gpu_worker.py"), which]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    result = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert "multi-gpu parity ok" in result.stdout
