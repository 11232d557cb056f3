"""Communication bootstrap: who am I, who are my peers, and a way to swap a few bytes.

Same role and function names as the reference's flashmoe/cb.py:19-72, with NVSHMEM's UID
hand-shake replaced by what this package needs: `torch.distributed` (NCCL or gloo, already
initialised by the launcher) to all-gather CUDA IPC handles once at `initialize`.  With no
process group the world is this one process.  No collective runs on the data path.
"""
from __future__ import annotations

import os
from typing import List

IS_INITIALIZED = False
_rank = 0
_world = 1


def has_package(name: str) -> bool:
    import importlib.util
    return importlib.util.find_spec(name) is not None


def get_local_rank() -> int:
    """GPU ordinal of this process: LOCAL_RANK under torchrun, else 0 (cb.py:8-17)."""
    v = os.environ.get("LOCAL_RANK")
    return int(v) if v is not None else 0


def _dist():
    import torch.distributed as dist
    return dist if (dist.is_available() and dist.is_initialized()) else None


def initialize() -> None:
    global IS_INITIALIZED, _rank, _world
    d = _dist()
    if d is not None:
        _rank, _world = d.get_rank(), d.get_world_size()
    else:
        _rank, _world = 0, 1
    IS_INITIALIZED = True


def get_rank() -> int:
    assert IS_INITIALIZED
    return _rank


def get_world_size() -> int:
    assert IS_INITIALIZED
    return _world


def all_on_one_node() -> bool:
    """True when every rank is on this host (the reference asks NVSHMEM's shared team,
    flashmoe/__init__.py:37-43)."""
    d = _dist()
    if d is None:
        return True
    import socket
    names: List[str] = [None] * d.get_world_size()
    d.all_gather_object(names, socket.gethostname())
    return len(set(names)) == 1


def all_gather_bytes(payload: bytes) -> List[bytes]:
    d = _dist()
    if d is None:
        return [payload]
    out: List[bytes] = [None] * d.get_world_size()
    d.all_gather_object(out, payload)
    return out


def exchange_by_rank_map(payload: bytes, ep_rank: int, rank_map) -> List[bytes]:
    """Every process hands in `payload` and its expert-parallel rank; returns the payloads of this
    process's EP group ordered by EP rank.  `rank_map[p]` is the global rank (position in the
    default process group) of EP rank p, as in the reference (bootstrap.cuh:140,
    epRankToGlobalRank): the map may be a permutation of the world, and an EP group may be a
    subset of it (every process of the world still takes part in the gather).  Raises ValueError
    when the map does not describe this process or when the peers disagree with it."""
    mine = get_rank()
    ep_world = len(rank_map)
    if not 0 <= ep_rank < ep_world or rank_map[ep_rank] != mine:
        raise ValueError(f"rank_map[{ep_rank}] = {rank_map[ep_rank] if 0 <= ep_rank < ep_world else '?'} "
                         f"but this process is global rank {mine}")
    if len(set(rank_map)) != ep_world or min(rank_map) < 0 or max(rank_map) >= get_world_size():
        raise ValueError("rank_map must name ep_world distinct global ranks of this job")
    tagged = all_gather_bytes(ep_rank.to_bytes(4, "little") + payload)
    out = []
    for p in range(ep_world):
        blob = tagged[rank_map[p]]
        theirs = int.from_bytes(blob[:4], "little")
        if theirs != p:
            raise ValueError(f"rank_map says global rank {rank_map[p]} is EP rank {p}, "
                             f"but that process says it is EP rank {theirs}")
        out.append(blob[4:])
    return out


def sync_all(stream_ptr: int) -> None:
    """Drain `stream_ptr`, then barrier across ranks (cb.py:67-72: nvshmem sync_all)."""
    assert IS_INITIALIZED
    import torch
    if torch.cuda.is_available():
        torch.cuda.ExternalStream(stream_ptr).synchronize() if stream_ptr else torch.cuda.synchronize()
    d = _dist()
    if d is not None:
        d.barrier()
