"""The per-description kernel specialisation (flashmoe_b200.jit.specialised_library): cache key,
the lock / atomic-publish protocol of the reference's JIT (flashmoe/jit.py:188-296) with two
processes racing for one artefact, and what a specialised library exports.  Needs nvcc, no GPU."""
import ctypes as C
import multiprocessing as mp
import os
import shutil

import pytest

import flashmoe_b200 as flashmoe
from flashmoe_b200 import jit

needs_nvcc = pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                                reason="nvcc not found")


def _args(**kw):
    d = dict(data_type=flashmoe.DataType.BF16, tokens_per_rank=96, token_dim=256, ffn_size=384, num_experts=8,
             top_k=2, gpu_arch=1000, mlp_type=flashmoe.MLPType.GATED, act_type=flashmoe.ActivationType.SILU,
             stream_ptr=0, device_id=0)
    d.update(kw)
    return flashmoe.InitArgs(**d)


def test_key_follows_what_the_kernel_is_specialised_on():
    base = jit.spec_key(_args(), False)
    assert base == jit.spec_key(_args(), False)
    # tokens, experts and capacity stay run-time arguments: same library
    assert base == jit.spec_key(_args(tokens_per_rank=4096, num_experts=64, expert_peer_capacity=7), False)
    others = [jit.spec_key(_args(token_dim=512), False), jit.spec_key(_args(ffn_size=512), False),
              jit.spec_key(_args(top_k=1), False), jit.spec_key(_args(mlp_type=flashmoe.MLPType.VANILLA), False),
              jit.spec_key(_args(act_type=flashmoe.ActivationType.GELU), False),
              jit.spec_key(_args(data_type=flashmoe.DataType.FP16), False), jit.spec_key(_args(), True)]
    assert len({base, *others}) == len(others) + 1


def test_nothing_is_built_unless_asked(tmp_path, monkeypatch):
    monkeypatch.setenv("FLASHMOE_CACHE_DIR", str(tmp_path))
    monkeypatch.delenv("FMOE_JIT", raising=False)
    assert jit.specialised_library(_args()) is None
    assert list(tmp_path.iterdir()) == []


def _build(cache, q):
    os.environ["FLASHMOE_CACHE_DIR"] = cache
    q.put(str(jit.specialised_library(_args(token_dim=320), build=True)))


@needs_nvcc
def test_two_processes_race_for_one_artefact(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_build, args=(str(tmp_path), q)) for _ in range(2)]
    for p in procs:
        p.start()
    paths = {q.get(timeout=300) for _ in procs}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert len(paths) == 1
    left = sorted(f.name for f in tmp_path.iterdir())
    assert left == [os.path.basename(paths.pop())], left      # no lock file, no temporary left behind
    lib = C.CDLL(str(tmp_path / left[0]))
    info = (C.c_int32 * 8)()
    assert lib.fmoe_spec_info(info) == 0
    assert list(info)[:7] == [320, 384, 2, 1, 1, 0, 0]
    assert hasattr(lib, "fmoe_spec_prepare") and hasattr(lib, "fmoe_spec_launch")


@needs_nvcc
def test_benchmark_shapes_have_their_specialised_kernels_after_build():
    """`__graft_entry__.build()` leaves a library for every benchmark description in the in-tree
    cache, keyed by the CURRENT sources: a stale cache (sources edited, build not re-run) would
    silently put the benchmark on the generic kernel."""
    import __graft_entry__ as entry
    from flashmoe_b200.workloads import CONFIGS
    entry.build_specialised()
    for w in CONFIGS.values():
        a = flashmoe.InitArgs(w.data_type, w.tokens_per_rank, w.token_dim, w.ffn_size, w.num_experts, w.top_k,
                              1000, w.mlp_type, w.act_type, 0, 0)
        assert jit.specialised_library(a, build=False) is not None, w.name
