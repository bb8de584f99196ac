"""Tensor parallel over 2 GPUs (NCCL): a sharded tiny model must reproduce the CPU oracle's full-model
logits within the single-GPU tolerance, and all ranks must agree bit for bit.  Skipped on boxes with
one GPU; the host-side sharding rules are covered on CPU in test_host_tp.py."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_rank_model_matches_oracle():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = 29500 + os.getpid() % 2000
    # GGB_TP_ONE_SHOT: take the peer-memory all-reduce also at 2 ranks (by default it starts at 4, where it wins)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", GGB_TP_ONE_SHOT="1")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "tp_worker.py"), str(r), "2", str(port)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(2)]
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=420)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "TP_WORKER_OK" in out, f"rank {r}:\n{out[-3000:]}"
