"""Tensor-parallel parity (70B sharding over the GPUs of one box): runs tests/tp_worker.py on 2 ranks whenever the box
has at least 2 GPUs.  The worker's output is part of the assertion message either way, and a passing run prints it, so
that a log of the run shows what was compared."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tensor_parallel_two_ranks(capsys):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    # NVLS off: the ranks only use plain peer stores (and NCCL's ring for the all-gather baseline); a rank that died with
    # memory bound to an NVLink multicast object would fault the others
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29517", os.path.join(ROOT, "tests", "tp_worker.py")], capture_output=True, text=True, timeout=900, env=env)
    out = r.stdout[-4000:] + r.stderr[-4000:]
    assert r.returncode == 0, out
    assert "tp parity ok on 2 ranks" in r.stdout, out
    with capsys.disabled():
        print("\n[tp_worker] " + "\n[tp_worker] ".join(line for line in r.stdout.splitlines() if "tp parity" in line))
