"""Multi-GPU parity of the fused NVLink kernels against the CPU oracle (needs >= 2 GPUs)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_strategies_on_all_local_gpus_match_the_oracle():
    n = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29731", os.path.join(ROOT, "tests", "mgpu", "worker_parity.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    out = r.stdout + r.stderr
    rep = [l for l in out.splitlines() if l.startswith("MGPU_REPORT ")]
    assert r.returncode == 0 and "MGPU_OK" in out, out[-4000:]
    report = json.loads(rep[0][len("MGPU_REPORT "):])
    assert all(v["ok"] for v in report.values()), report
