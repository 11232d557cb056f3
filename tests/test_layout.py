"""The closed forms the persistent kernel uses after the count exchange (segment table + binary
search per ticket, K parts of the closing tiles, send order, per-CTA chunk queue), restated in
flashmoe_b200/layout.py, against a plain walk of the same order over many random count tables:
every tile is handed out exactly once, a task only depends on smaller tickets, every routed row is
sent by exactly one chunk.  CPU only."""
import zlib

import numpy as np
import pytest

from flashmoe_b200 import layout


def random_counts(rng, W, E, ec, style):
    if style == "zeros":
        c = np.zeros((W, E), dtype=np.int64)
        c[rng.integers(W), rng.integers(E)] = rng.integers(1, 4)
    elif style == "sparse":
        c = rng.integers(0, 3 * ec // 2 + 1, size=(W, E)) * (rng.random((W, E)) < 0.25)
    elif style == "full":
        c = np.full((W, E), ec, dtype=np.int64)
    else:
        c = rng.integers(0, 2 * ec + 1, size=(W, E))
    return c.astype(int).tolist()


CASES = [  # W, nLx, ec, tiles_n0, tiles_n1, grid, split_parts, split_tiles
    (1, 16, 64, 64, 20, 148, 2, 148),
    (2, 8, 300, 64, 20, 148, 2, 148),
    (8, 2, 130, 64, 20, 148, 2, 148),
    (4, 32, 40, 6, 8, 148, 2, 148),
    (1, 1, 700, 3, 2, 148, 2, 148),
    (2, 3, 129, 2, 1, 4, 4, 4),
    (1, 5, 257, 1, 3, 2, 2, 1),
    (8, 4, 64, 12, 16, 148, 1, 0),
    (1, 8, 500, 4, 2, 16, 8, 160),
]


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("style", ["dense", "sparse", "zeros", "full"])
def test_ticket_decode_hands_out_every_tile_once_in_the_walk_s_order(case, pair, style):
    W, nlx, ec, tn0, tn1, grid, parts, split_tiles = case
    E = W * nlx
    rng = np.random.default_rng(zlib.crc32(repr((case, pair, style)).encode()))
    emap = [e // nlx for e in range(E)]
    for rank in {0, W - 1}:
        counts = random_counts(rng, W, E, ec, style)
        lay = layout.build(counts, rank, emap, ec, tn0, tn1, grid=grid, pair=pair)
        seg = layout.task_segments(lay.mtile0, tn0, tn1, grid, pair, parts, split_tiles)
        total = seg.first[-1]
        gsz = 2 if pair else 1
        assert layout.decode_ticket(total, seg, lay.mtile0, tn1, pair, parts).kind == layout.KIND_STOP
        decoded = [layout.decode_ticket(t, seg, lay.mtile0, tn1, pair, parts) for t in range(total)]
        # collapse the K parts of a tile: what is left is the walk, tile by tile
        tiles, seen_parts = [], {}
        for t in decoded:
            key = (t.kind, t.lx, t.m_in_expert // gsz, t.n)
            if t.nparts > 1:
                assert t.kind == layout.KIND_GEMM1 and not pair and t.nparts == parts
                seen_parts.setdefault(key, []).append((t.part, t.split_idx))
                if t.part > 0:
                    assert tiles[-1] == key       # parts of one tile are consecutive tickets
                    continue
            tiles.append(key)
        assert tiles == lay.tasks
        assert len(set(tiles)) == len(tiles)
        # the cut tiles are exactly the last GEMM1 tiles of the order, each in `parts` parts, with
        # distinct scratch slots below split_tiles, numbered from the end of the order
        g1 = [k for k in tiles if k[0] == layout.KIND_GEMM1]
        want_cut = 0 if (pair or parts <= 1) else min(split_tiles, len(g1))
        assert list(seen_parts) == g1[len(g1) - want_cut:]
        for i, key in enumerate(seen_parts):
            assert [p for p, _ in seen_parts[key]] == list(range(parts))
            assert {s for _, s in seen_parts[key]} == {want_cut - 1 - i}
        # a task only waits on smaller tickets: GEMM1 of an M tile after every GEMM0 tile of it
        done = set()
        for t in decoded:
            for q in range(gsz):
                m = t.m_in_expert + q
                if m >= lay.mtile0[t.lx + 1] - lay.mtile0[t.lx]:
                    continue
                if t.kind == layout.KIND_GEMM0:
                    done.add((t.lx, m, t.n))
                else:
                    assert all((t.lx, m, n0) in done for n0 in range(tn0))
        # every M tile of every local expert got all its GEMM0 and GEMM1 column tiles
        for lx in range(nlx):
            for m in range(lay.mtile0[lx + 1] - lay.mtile0[lx]):
                assert all((lx, m, n0) in done for n0 in range(tn0))
                assert all((layout.KIND_GEMM1, lx, m // gsz, n1) in set(g1) for n1 in range(tn1))


@pytest.mark.parametrize("nk", [4, 8, 13, 64, 128])
@pytest.mark.parametrize("parts", [2, 3, 4, 8])
def test_k_parts_cover_the_k_blocks_once(nk, parts):
    edges = [(nk * p // parts, nk * (p + 1) // parts) for p in range(parts)]
    assert edges[0][0] == 0 and edges[-1][1] == nk
    assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
    if nk >= 4 * parts:          # what the host requires before it cuts at all
        assert all(b - a >= 4 for a, b in edges)


@pytest.mark.parametrize("W,nlx,ec", [(1, 16, 64), (2, 8, 1024), (8, 2, 1024), (4, 32, 7), (8, 16, 300), (1, 1, 5)])
@pytest.mark.parametrize("style", ["dense", "sparse", "zeros", "full"])
@pytest.mark.parametrize("grid", [148, 2, 1])
def test_every_routed_row_is_sent_by_exactly_one_chunk(W, nlx, ec, style, grid):
    E = W * nlx
    rng = np.random.default_rng(zlib.crc32(repr((W, nlx, ec, style, grid)).encode()))
    # experts dealt to the ranks round-robin here (the blocked map is covered above)
    lidx = [e // W for e in range(E)]
    own = random_counts(rng, 1, E, ec, style)[0]
    plan = layout.send_order(own, lidx, nlx, ec)
    assert sorted(plan.order) == list(range(E))
    c0 = plan.class0_experts
    assert all(2 * lidx[e] < nlx for e in plan.order[:c0]) and not any(2 * lidx[e] < nlx for e in plan.order[c0:])
    assert plan.order[:c0] == sorted(plan.order[:c0]) and plan.order[c0:] == sorted(plan.order[c0:])
    sent = [min(max(own[e], 0), ec) for e in plan.order]
    assert plan.pref == [sum(sent[:i]) for i in range(E + 1)]
    total, r0 = plan.pref[-1], plan.pref[c0]
    covered = np.zeros(total, dtype=np.int64)
    for cta in range(grid):
        chunks = layout.dispatch_chunks(plan, cta, grid)
        in_class1 = False
        for first, rows in chunks:
            assert 1 <= rows <= 16
            covered[first:first + rows] += 1
            if first >= r0:
                in_class1 = True
            else:
                assert not in_class1 and first + rows <= r0     # class 0 chunks come first and stay in class 0
        # the queue holds exactly this CTA's slice of both classes
        assert sum(r for _, r in chunks) == (r0 * (cta + 1) // grid - r0 * cta // grid) + \
            ((total - r0) * (cta + 1) // grid - (total - r0) * cta // grid)
    assert (covered == 1).all()
    # the binary search finds the expert a row belongs to, skipping experts that send nothing
    for row in ([0, total - 1] + rng.integers(0, max(total, 1), size=64).tolist() if total else []):
        pos = layout.row_position(plan, row)
        assert plan.pref[pos] <= row < plan.pref[pos + 1]
