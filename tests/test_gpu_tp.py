"""Row-split tensor parallelism on real GPUs (needs at least two): a small Llama split over 2 GPUs gives
the single-GPU logits to within the activation-quantization noise (the partial sums of a K-split are added in
another order, and a last-bit difference can flip a Q8 rounding in the next layer; the per-op 1e-5 bound of the
split itself is checked on the CPU in test_tp_sharding.py) and the same token on every rank."""
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
