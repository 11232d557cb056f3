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


# ---- the kernel's own formulas, step by step ---------------------------------------------------
# `build` above lists the tasks by walking the order; the kernel cannot afford a walk and works
# with closed forms instead (segment sizes, a prefix scan, a binary search per ticket).  The
# functions below restate those forms one to one (moe_forward_body in csrc/moe_kernel.cu: the
# task-order block of warp 0, `decode`, the send order, `chunk_range` and `lookup`), so that tests
# can hold them to the walk over many random count tables.

KIND_GEMM0, KIND_GEMM1, KIND_STOP = 0, 1, 2


@dataclass
class Segments:
    first: List[int]     # [2 nLx + 1] first ticket of every segment; last entry = number of tickets
    kind: List[int]      # [2 nLx]
    lx: List[int]        # [2 nLx]
    whole: List[int]     # [2 nLx] leading tickets of the segment that are whole tiles (the rest are K parts)
    lag: int


def task_segments(mtile0: Sequence[int], tiles_n0: int, tiles_n1: int, grid: int, pair: bool,
                  split_parts: int = 1, split_tiles: int = 0) -> Segments:
    """Segment table of the task order: G0(0..lag-1), G0(lag), G1(0), G0(lag+1), G1(1), ...  The last
    `split_tiles` GEMM1 tiles of the order are cut along K into `split_parts` tickets each (never in
    the CTA-pair form)."""
    nlx = len(mtile0) - 1
    gsz = 2 if pair else 1
    lag = nlx
    for t in range(1, nlx):
        if mtile0[t] * tiles_n0 >= 2 * grid:
            lag = t
            break
    size, kind, lxs, whole = [0] * (2 * nlx), [0] * (2 * nlx), [0] * (2 * nlx), [0] * (2 * nlx)
    for i in range(nlx):
        groups = (mtile0[i + 1] - mtile0[i] + gsz - 1) // gsz
        i0 = i + max(0, i - lag)
        s1 = i + lag
        i1 = min(s1, nlx) + i + (1 if s1 < nlx else 0)
        size[i0] = whole[i0] = groups * tiles_n0
        kind[i0], lxs[i0] = KIND_GEMM0, i
        tiles = groups * tiles_n1
        after = (mtile0[nlx] - mtile0[i + 1]) * tiles_n1
        cut = 0 if (pair or split_parts <= 1) else max(0, min(tiles, split_tiles - after))
        size[i1] = (tiles - cut) + cut * split_parts
        whole[i1] = tiles - cut
        kind[i1], lxs[i1] = KIND_GEMM1, i
    first, run = [], 0
    for s in size:
        first.append(run)
        run += s
    first.append(run)
    return Segments(first, kind, lxs, whole, lag)


@dataclass
class Ticket:
    kind: int
    lx: int = 0
    m_in_expert: int = 0     # M tile inside the expert (the leader's, in the CTA-pair form)
    n: int = 0
    part: int = 0
    nparts: int = 1
    split_idx: int = 0


def decode_ticket(ticket: int, seg: Segments, mtile0: Sequence[int], tiles_n1: int, pair: bool,
                  split_parts: int = 1) -> Ticket:
    nlx = len(mtile0) - 1
    gsz = 2 if pair else 1
    if ticket >= seg.first[-1]:
        return Ticket(KIND_STOP)
    lo, hi = 0, 2 * nlx
    while hi - lo > 1:      # the largest segment whose first ticket is <= ticket
        mid = (lo + hi) >> 1
        if seg.first[mid] <= ticket:
            lo = mid
        else:
            hi = mid
    lx = seg.lx[lo]
    idx = ticket - seg.first[lo]
    groups = (mtile0[lx + 1] - mtile0[lx] + gsz - 1) // gsz
    t = Ticket(seg.kind[lo], lx)
    if idx >= seg.whole[lo]:
        j = idx - seg.whole[lo]
        idx = seg.whole[lo] + j // split_parts
        t.part = j - (idx - seg.whole[lo]) * split_parts
        t.nparts = split_parts
        after = (mtile0[nlx] - mtile0[lx + 1]) * tiles_n1
        t.split_idx = after + (groups * tiles_n1 - 1 - idx)
    t.n = idx // groups
    t.m_in_expert = gsz * (idx - t.n * groups)
    return t


@dataclass
class SendPlan:
    order: List[int]        # [E] position in the send order -> expert
    pref: List[int]         # [E + 1] rows sent before position i
    class0_experts: int     # positions below this hold experts of the first half of their owner's list


def send_order(own_counts: Sequence[int], lidx: Sequence[int], nlx: int, ec: int) -> SendPlan:
    """Experts in the first half of their owner's local list first (ascending id), the others after
    them (ascending id); prefix sums of this rank's clamped counts in that order."""
    E = len(own_counts)
    first = [e for e in range(E) if 2 * lidx[e] < nlx]
    order = first + [e for e in range(E) if not 2 * lidx[e] < nlx]
    pref = [0]
    for e in order:
        pref.append(pref[-1] + min(max(int(own_counts[e]), 0), ec))
    return SendPlan(order, pref, len(first))


def dispatch_chunks(plan: SendPlan, cta: int, grid: int, dispatch_warps: int = 6) -> List[tuple]:
    """The chunk queue of one CTA: (first row, rows) in send-order row numbers, class 0 chunks first."""
    r0 = plan.pref[plan.class0_experts]
    r1 = plan.pref[-1] - r0
    a0, n0 = r0 * cta // grid, r0 * (cta + 1) // grid - r0 * cta // grid
    a1, n1 = r0 + r1 * cta // grid, (r0 + r1 * (cta + 1) // grid) - (r0 + r1 * cta // grid)
    rows = min(16, max(1, (n0 + n1 + dispatch_warps - 1) // dispatch_warps))
    chunks0 = (n0 + rows - 1) // rows
    total = chunks0 + (n1 + rows - 1) // rows
    out = []
    for ch in range(total):
        if ch < chunks0:
            first = a0 + ch * rows
            out.append((first, min(rows, a0 + n0 - first)))
        else:
            first = a1 + (ch - chunks0) * rows
            out.append((first, min(rows, a1 + n1 - first)))
    return out


def row_position(plan: SendPlan, row: int) -> int:
    """Position in the send order of the expert that routed row `row` belongs to: the largest position
    whose prefix is <= row (positions of experts that send nothing are skipped by construction)."""
    lo, hi = 0, len(plan.order)
    while hi - lo > 1:
        mid = (lo + hi) >> 1
        if plan.pref[mid] <= row:
            lo = mid
        else:
            hi = mid
    return lo
