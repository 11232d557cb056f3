"""Multi-GPU parity of the fused forward: experts sharded over 2 (and 4) GPUs of one box, rows
exchanged by in-kernel peer stores through CUDA-IPC mapped symmetric blocks.  Skipped when the
box shows a single GPU."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, case, tokens=None, timeout=600):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "multi_worker.py"), "--case", case]
    if tokens:
        cmd += ["--tokens", str(tokens)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    lines = [l for l in p.stdout.splitlines() if l.startswith("MULTI_RESULT ")]
    assert p.returncode == 0 and lines, p.stdout[-3000:] + p.stderr[-3000:]
    return json.loads(lines[-1][len("MULTI_RESULT "):])


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("case", ["bf16_gated_k2", "bf16_two_mtiles", "bf16_vanilla_gelu_k8", "bf16_drop"])
def test_two_gpus_match_the_oracle(case):
    _need(2)
    for r in _run(2, case):
        assert r["ok"], r


def test_two_gpus_scout_shape_trimmed():
    _need(2)
    for r in _run(2, "scout", tokens=256):
        assert r["ok"], r


def test_four_gpus_match_the_oracle():
    _need(4)
    for r in _run(4, "bf16_vanilla_gelu_k8"):
        assert r["ok"], r
