"""Row-split tensor parallelism on real GPUs (needs at least two): a small Llama split over 2 GPUs (and over 4 where
there are 4) gives, bit for bit, the logits of the CPU restatement of the same cut, the same greedy tokens, and
the same token on every rank.  The same comparison with the ranks played as threads on one GPU is in
test_gpu_tp_one_gpu.py; here the partial sums really cross NVLink."""
import os
import subprocess
import sys

import pytest

import b200

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_tp_matches_the_cpu_cut(world, exchange):
    m = b200.load()
    if m.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TP_LL="1" if exchange == "peer" else "0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29641 + world), os.path.join(here, "tp_rank_main.py")], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ok=True" in r.stdout
    print(r.stdout[-400:])
