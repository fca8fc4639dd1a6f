"""Row-split tensor parallelism on real GPUs (needs at least two): a small Llama split over 2 GPUs gives
the single-GPU logits within 1e-5 of their largest magnitude and the same greedy tokens on every rank."""
import os
import subprocess
import sys

import pytest

import b200

pytestmark = pytest.mark.gpu


def test_tp2_matches_one_gpu():
    m = b200.load()
    if m.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29641", os.path.join(here, "tp_rank_main.py")], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ok=True" in r.stdout
