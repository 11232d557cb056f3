"""Model-description types of the layer's public API, and the in-tree native build.

The names, constructor arguments, defaults and enum values mirror the reference's
flashmoe/jit.py:7-151 so that a script written against `flashmoe` runs against this package
unchanged (`import flashmoe_b200 as flashmoe`).

The reference compiles one shared object per model description at `initialize` time
(flashmoe/jit.py:153-296).  Here the ahead-of-time library (`_get_compiled`) already runs every
description with the shapes as run-time arguments; on top of it `specialised_library` builds,
per description, a small library holding the persistent kernel with H, I, top-k, the MLP type,
the activation, the element type and the tile form as compile-time constants, under the
reference's cache protocol: a key hashed from the description and the kernel sources, a lock file
created with O_EXCL so that one process of a job builds while the others wait for the artefact,
and an atomic rename to publish it.  `initialize` loads a specialised library when the cache holds
one (or builds it when FMOE_JIT=1) and falls back to the generic kernel otherwise; both give the
same bits.
"""
from __future__ import annotations

import hashlib
import math
import os
import shutil
import socket
import subprocess
import threading
import time
from enum import IntEnum
from pathlib import Path
from typing import List, Optional


class Topology(IntEnum):
    NVLINK_ONLY = 0
    MIXED = 1


class MLPType(IntEnum):
    GATED = 0
    VANILLA = 1


class DataType(IntEnum):
    BF16 = 0
    FP16 = 1
    FP32 = 2
    FP64 = 3


class ActivationType(IntEnum):
    IDENTITY = 0
    SILU = 1
    GELU = 2
    RELU = 3


class ContextHandle:
    """Pairs the native module with the opaque context it created (jit.py:7-20)."""
    __slots__ = ("_mod", "_ctx")

    def __init__(self, mod, ctx):
        self._mod, self._ctx = mod, ctx

    @property
    def context(self):
        return self._ctx

    @property
    def mod(self):
        return self._mod


class ForwardArgs:
    """Device addresses (ints) of the contiguous buffers one forward reads and writes.

    tokens [S, H]; expert_counts [E] int32; local_expert_up / local_expert_up_v stored
    [nLx, I, H]; local_expert_down stored [nLx, H, I]; biases [nLx, I], [nLx, I], [nLx, H];
    moe_out [S, H].  `local_expert_up` is the activated branch, `_v` the linear one.
    A gated MLP must supply both `_v` buffers (jit.py:72-73); for a plain MLP they stay None
    and are handed to the library as null.  A null bias address means a zero bias
    (an addition of this package; the reference always reads its biases).
    """

    def __init__(self, mt: MLPType, tokens: int, expert_counts: int, local_expert_up: int,
                 local_bias_up: int, local_expert_down: int, local_bias_down: int, moe_out: int,
                 stream_ptr: int, *, swish_alpha: float = 1.0, swish_beta: float = 1.0,
                 local_expert_up_v: Optional[int] = None, local_bias_up_v: Optional[int] = None):
        if mt == MLPType.GATED:
            assert local_expert_up_v is not None, "a gated MLP needs local_expert_up_v"
            assert local_bias_up_v is not None, "a gated MLP needs local_bias_up_v"
        self.tokens = tokens
        self.expert_counts = expert_counts
        self.local_expert_up = local_expert_up
        self.local_expert_up_v = local_expert_up_v
        self.local_bias_up = local_bias_up
        self.local_bias_up_v = local_bias_up_v
        self.local_expert_down = local_expert_down
        self.local_bias_down = local_bias_down
        self.moe_out = moe_out
        self.swish_alpha = swish_alpha
        self.swish_beta = swish_beta
        self.stream_ptr = stream_ptr


class InitArgs:
    """Description of the layer and of this rank's place in the expert-parallel group.

    `gpu_arch` is the compute capability times 100 (1000 for sm_100), as in the reference
    (quickstart.py:50).  `expert_peer_capacity` defaults to ceil(S / E) * k (jit.py:148-151):
    the most tokens one rank may send to one expert; later ones are dropped.  Pass
    `expert_peer_capacity=tokens_per_rank` to drop nothing.  `initialize` fills the fields
    left at None (ep_world, ep_rank, my_pe, num_local_experts, expert_map, rank_map, topo).
    """
    topo: Topology = Topology.MIXED

    def __init__(self, data_type: DataType, tokens_per_rank: int, token_dim: int, ffn_size: int,
                 num_experts: int, top_k: int, gpu_arch: int, mlp_type: MLPType,
                 act_type: ActivationType, stream_ptr: int, device_id: int, *,
                 ep_world: Optional[int] = None, num_local_experts: Optional[int] = None,
                 ep_rank: Optional[int] = None, my_pe: Optional[int] = None,
                 expert_map: Optional[List[int]] = None, rank_map: Optional[List[int]] = None,
                 expert_peer_capacity: Optional[int] = None) -> None:
        assert gpu_arch >= 700
        self.data_type = data_type
        self.tokens_per_rank = tokens_per_rank
        self.token_dim = token_dim
        self.ffn_size = ffn_size
        self.num_experts = num_experts
        self.top_k = top_k
        self.gpu_arch = gpu_arch
        self.mlp_type = mlp_type
        self.act_type = act_type
        self.stream_ptr = stream_ptr
        self.device_id = device_id
        self.ep_world = ep_world
        self.num_local_experts = num_local_experts
        self.ep_rank = ep_rank
        self.my_pe = my_pe
        self.expert_map = expert_map
        self.rank_map = rank_map
        if expert_peer_capacity is None:
            expert_peer_capacity = math.ceil(float(tokens_per_rank) / num_experts) * top_k
        self.expert_peer_capacity = expert_peer_capacity


def _get_compiled(arg: Optional[InitArgs] = None, src=None, mod_prefix: str = "", mod_name: str = ""):
    """Return the loaded native library (the reference's per-model JIT collapses to this).

    Raises if the library has not been built: there is no fallback implementation.
    """
    from . import _native
    return _native.lib()


# ---- per-description specialisation of the persistent kernel ------------------------------------

SPEC_SOURCES = ("csrc/moe_kernel.cu", "csrc/common.cuh", "csrc/ptx.cuh", "csrc/router_math.cuh",
                "../include/flashmoe_b200.h")
SPEC_FLAGS = ("-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared")


def spec_cache_dir() -> Path:
    """FLASHMOE_CACHE_DIR as in the reference (jit.py:199); the default is inside the package so
    that libraries built ahead of time travel with it."""
    return Path(os.environ.get("FLASHMOE_CACHE_DIR", str(Path(__file__).resolve().parent / "lib" / "spec")))


def _source_fingerprint() -> str:
    root = Path(__file__).resolve().parent
    h = hashlib.sha256(b"flashmoe-b200-spec-v1")
    for rel in SPEC_SOURCES:
        path = (root / rel).resolve()
        h.update(rel.encode())
        h.update(path.read_bytes())
    return h.hexdigest()[:16]


def spec_defines(arg: "InitArgs", pair: bool) -> List[str]:
    return [f"-DFMOE_SPEC=1", f"-DFMOE_SPEC_H={arg.token_dim}", f"-DFMOE_SPEC_I={arg.ffn_size}",
            f"-DFMOE_SPEC_K={arg.top_k}", f"-DFMOE_SPEC_GATED={1 if arg.mlp_type == MLPType.GATED else 0}",
            f"-DFMOE_SPEC_ACT={int(arg.act_type)}", f"-DFMOE_SPEC_DT={int(arg.data_type)}",
            f"-DFMOE_SPEC_PAIR={1 if pair else 0}"]


def spec_key(arg: "InitArgs", pair: bool) -> str:
    text = "|".join(spec_defines(arg, pair) + list(SPEC_FLAGS) + [_source_fingerprint()])
    return hashlib.sha256(text.encode()).hexdigest()[:16]


def specialised_library(arg: "InitArgs", pair: bool = False, build: Optional[bool] = None,
                        timeout_s: float = 600.0) -> Optional[Path]:
    """Path of the kernel library specialised for `arg`, or None.

    Cached under spec_cache_dir()/fmoe_spec_<key>.so.  A missing library is built when `build` is
    true (default: the FMOE_JIT environment variable is "1"): the first process to create the lock
    file compiles into a private temporary name and publishes it with an atomic rename; every other
    process polls for the final name (flashmoe/jit.py:223-296 does the same around cmake)."""
    cache = spec_cache_dir()
    so_path = cache / f"fmoe_spec_{spec_key(arg, pair)}.so"
    if so_path.exists():
        return so_path
    if build is None:
        build = os.environ.get("FMOE_JIT", "0") == "1"
    if not build:
        return None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return None
    cache.mkdir(parents=True, exist_ok=True)
    lock_path = so_path.with_suffix(".lock")
    uniq = f"{socket.gethostname()}_pid{os.getpid()}_tid{threading.get_ident()}"
    try:
        fd = os.open(lock_path, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
        with os.fdopen(fd, "w") as f:
            f.write(f"{uniq}\ntime={time.time()}\n")
    except FileExistsError:
        start = time.time()                      # somebody else is the builder: wait for the artefact
        while not so_path.exists():
            if time.time() - start > timeout_s:
                raise TimeoutError(f"timed out waiting for {so_path} while another process was building it")
            time.sleep(0.1)
        return so_path
    try:
        if so_path.exists():                     # finished just before we took the lock
            return so_path
        src = Path(__file__).resolve().parent / "csrc" / "moe_kernel.cu"
        tmp = cache / f".{so_path.stem}.{uniq}.tmp.so"
        cmd = [nvcc, *SPEC_FLAGS, *spec_defines(arg, pair), "-o", str(tmp), str(src)]
        proc = subprocess.run(cmd, cwd=src.parent, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed building a specialised kernel:\n" + proc.stdout + proc.stderr)
        tmp.replace(so_path)                     # atomic publish
    finally:
        try:
            lock_path.unlink()
        except FileNotFoundError:
            pass
    return so_path
