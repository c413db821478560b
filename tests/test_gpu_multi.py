"""Multi-rank parity: launches tests/multi_worker.py with one process per GPU (needs >= 2 GPUs on the node; skipped
otherwise), and the bounded-wait check of tests/timeout_worker.py (two ranks; runs on one GPU too)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_collectives_and_tp_ffn(world):
    if _ngpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29600 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert p.stdout.count("multi-GPU checks passed") == world


@pytest.mark.parametrize("same_device", [True, False])
def test_peer_wait_runs_out_and_reports(same_device):
    """A Recv whose peer never runs: the wait gives up after 50 ms, wait() raises GpuError with status 3, destroy is
    clean and the next executor on that GPU passes a parity case."""
    if not same_device and _ngpus() < 2:
        pytest.skip("needs 2 GPUs")
    if _ngpus() < 1:
        pytest.skip("needs a GPU")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ARKB_SAME_DEVICE="1" if same_device else "0")
    port = 29650 + int(same_device)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "timeout_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert p.stdout.count("bounded-wait checks passed") == 2


@pytest.mark.parametrize("world", [2, 8])
def test_nvls_all_reduce(world):
    """The large all_reduce through the NVSwitch (multimem.ld_reduce / multimem.st over a multicast-bound arena),
    against the oracle; falls back, and says so, where the GPUs offer no multicast."""
    if _ngpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ)
    port = 29670 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "nvls_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert p.stdout.count("nvls checks passed") == world
