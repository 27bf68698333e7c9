"""Expert-parallel layer on real GPUs (2 ranks over NCCL): every rank's output
must match the single-GPU layer on the same seeded inputs - routing exactly,
outputs bit for bit where both take the same kernels (rel-L2 <= 1e-3 otherwise)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
    pytest.skip("needs two CUDA devices", allow_module_level=True)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_gpu_expert_parallel_matches_single_gpu():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29711",
           os.path.join(ROOT, "tests", "ep_gpu_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    lines = [l for l in res.stdout.splitlines() if l.startswith("EP_RESULT")]
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert len(lines) == 1 and "ok=True" in lines[0], (lines, res.stderr[-2000:])
