"""Multi-rank paths: world_size-2 gloo ranks on CPU (always), and one rank per GPU over NCCL when >= 2 GPUs are visible."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, backend, port):
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "dist_worker.py"), backend]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)


def test_sharding_and_gather_order_with_gloo_ranks(built_lib):
    r = _torchrun(2, "gloo", 29611)
    assert r.returncode == 0 and "GLOO-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.gpu
def test_dotmpi_over_nccl(built_lib):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    r = _torchrun(min(n, 4), "nccl", 29612)
    assert r.returncode == 0 and "NCCL-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
