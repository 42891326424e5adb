"""TP+EP engine on 2 GPUs against the single-GPU engine, both collective backends (needs >= 2 GPUs)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_rank_selftest():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29511", "-m", "qwb200.parallel.selftest"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0 and "SELFTEST OK" in r.stdout
