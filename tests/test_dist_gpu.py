"""GPU (needs two B200s in the box; skipped with fewer): real NCCL through libgt_b200.so.
All-reduce, gradient averaging of a tiny GPT-2 with and without the backward overlap,
init_sync, and the strict signature check failing on every rank together
(mirrors gradtuity/tests/test_dist.py:216-537).  NVLS is off in these runs."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "dist_gpu_worker.py")


def gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


needs2 = pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs in one box")


def _launch(mode, timeout=300):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("GRADTUITY_DEVICE", None)
    cmd = [sys.executable, "-m", "gradtuity_b200.launch", "--nproc", "2", "--master-addr", "127.0.0.1", WORKER, mode]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


@needs2
@pytest.mark.parametrize("mode", ["allreduce", "sync_grads", "init_sync", "init_sync_strict_fail"])
def test_two_gpu(mode):
    r = _launch(mode)
    assert r.returncode == 0, (r.stdout[-1500:] + "\n" + r.stderr[-3000:])
