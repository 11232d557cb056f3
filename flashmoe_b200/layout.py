"""Host-side mirror of the index arithmetic the persistent kernel performs after the count
exchange: where a rank's rows land at an expert's owner, how M tiles are laid over the
landing area, and the order in which tiles are handed out.  Used by tests (to check the
kernel's intermediate buffers and to replay the exchange between CPU ranks) and by the
benchmark (to count algorithmic work from the routing counts).  Plain integers; no device code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

TILE_M = 128


def _round_up(v: int, a: int) -> int:
    return -(-v // a) * a


@dataclass
class RankLayout:
    sent: List[List[int]]      # [W][E] rows rank s sends to expert e (clamped to EC)
    dst_row0: List[int]        # [E] landing row at e's owner where THIS rank's rows start
    lx_base: List[int]         # [nLx] first landing row of local expert lx (multiple of 128)
    lx_rows: List[int]         # [nLx] rows of local expert lx over all sources
    mtile0: List[int]          # [nLx+1] prefix of M tiles
    tasks: List[tuple]         # (kind, lx, group, n) in ticket order; kind 0 = GEMM0, 1 = GEMM1;
                               # a group is two consecutive M tiles, one per CTA of a pair


def build(counts: Sequence[Sequence[int]], rank: int, expert_map: Sequence[int], ec: int,
          tiles_n0: int, tiles_n1: int, grid: int = 148, pair: bool = True) -> RankLayout:
    """counts[s][e] = tokens of rank s that chose expert e (unclamped, as the router writes them)."""
    W, E = len(counts), len(expert_map)
    nlx = E // W
    sent = [[min(max(int(c), 0), ec) for c in row] for row in counts]
    local = [[e for e in range(E) if expert_map[e] == r] for r in range(W)]
    dst_row0 = [0] * E
    lx_base, lx_rows = [0] * nlx, [0] * nlx
    for r in range(W):
        base = 0
        for lx, e in enumerate(local[r]):
            tot = sum(sent[s][e] for s in range(W))
            dst_row0[e] = base + sum(sent[s][e] for s in range(rank))
            if r == rank:
                lx_base[lx], lx_rows[lx] = base, tot
            base += _round_up(tot, TILE_M)
    mtile0 = [0]
    for lx in range(nlx):
        mtile0.append(mtile0[-1] + -(-lx_rows[lx] // TILE_M))
    # GEMM1 of expert i trails GEMM0 of expert i by `lag` experts: the smallest lag whose GEMM0
    # tiles cover two tickets per CTA
    lag = 1
    while lag < nlx and mtile0[lag] * tiles_n0 < 2 * grid:
        lag += 1
    gsz = 2 if pair else 1     # M tiles per ticket: a CTA pair takes two, a lone CTA one
    tasks = []
    for i in range(nlx + lag):
        if i < nlx:
            groups = (mtile0[i + 1] - mtile0[i] + gsz - 1) // gsz
            tasks += [(0, i, g, n) for n in range(tiles_n0) for g in range(groups)]
        if i >= lag:
            j = i - lag
            groups = (mtile0[j + 1] - mtile0[j] + gsz - 1) // gsz
            tasks += [(1, j, g, n) for n in range(tiles_n1) for g in range(groups)]
    return RankLayout(sent, dst_row0, lx_base, lx_rows, mtile0, tasks)


def landing_rows(nlx: int, world: int, ec: int, tokens_per_rank: int, top_k: int) -> int:
    """Capacity of the landing area (rows): the smaller of 'every expert full' and 'every token
    of every rank lands here', each expert rounded up to whole tiles."""
    cap_a = nlx * _round_up(world * ec, TILE_M)
    cap_b = _round_up(world * tokens_per_rank * top_k, TILE_M) + nlx * TILE_M
    return min(cap_a, cap_b)
