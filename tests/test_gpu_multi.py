"""Multi-GPU parity of the fused forward: experts sharded over 2, 4 and 8 GPUs of one box, rows
exchanged by in-kernel peer stores through CUDA-IPC mapped symmetric blocks.  A case is skipped
when the box shows fewer GPUs than it needs."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, case, tokens=None, timeout=600, env=None):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "multi_worker.py"), "--case", case]
    if tokens:
        cmd += ["--tokens", str(tokens)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env={**os.environ, **(env or {})})
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


def test_two_gpus_fp32_planes_cross_the_link():
    """FP32 layers push every row to the owner as three BF16 planes made by the sender."""
    _need(2)
    for r in _run(2, "fp32_gated_k2"):
        assert r["ok"], r


def test_two_gpus_cta_pair_form():
    """The cta_group::2 form of the GEMM loop with peer stores (no multicast load anywhere)."""
    _need(2)
    for r in _run(2, "bf16_two_mtiles", env={"FMOE_PAIR": "1"}):
        assert r["ok"], r


def test_four_gpus_match_the_oracle():
    _need(4)
    for r in _run(4, "bf16_vanilla_gelu_k8"):
        assert r["ok"], r


@pytest.mark.parametrize("case,tokens", [("bf16_vanilla_gelu_k8", None), ("scout", 256)])
def test_eight_gpus_match_the_oracle(case, tokens):
    """The full box: 8 source ranks per landing area, counts exchanged among 8, rows returned to 8."""
    _need(8)
    for r in _run(8, case, tokens=tokens, timeout=900):
        assert r["ok"], r
