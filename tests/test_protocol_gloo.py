"""World-size-2 replay of the exchange protocol on CPU ranks (gloo): each rank routes its own
tokens, the ranks all-gather their per-expert counts, every rank derives the landing layout with
the same arithmetic the kernel uses (flashmoe_b200.layout), rows travel to the expert's owner,
the owner runs the expert MLP, rows travel back indexed by (token, choice), and the owner of the
token combines.  The result must equal the single-rank oracle on that rank's tokens."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

from cases import GOLDEN_CASES  # noqa: E402
from flashmoe_b200 import cb, layout  # noqa: E402
from flashmoe_b200.workloads import make_tokens, make_weights  # noqa: E402


def _rank_main(rank, world, port, name, q):
    from helpers import oracle_layer, oracle_route, oracle_weights
    from oracle import moe_oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cb.initialize()
        assert (cb.get_rank(), cb.get_world_size()) == (rank, world)
        assert cb.all_on_one_node()
        blobs = cb.all_gather_bytes(bytes([rank]) * 64)
        assert [b[0] for b in blobs] == list(range(world))

        w = GOLDEN_CASES[name]
        lw = make_weights(w)
        wts = oracle_weights(lw)
        x = make_tokens(w, rank)
        E, k, ec = w.num_experts, w.top_k, w.expert_peer_capacity
        nlx = E // world
        emap = [e // nlx for e in range(E)]
        r = oracle_route(w, x=x, lw=lw)
        counts = [None] * world
        dist.all_gather_object(counts, r.counts.tolist())
        lay = layout.build(counts, rank, emap, ec, tiles_n0=3, tiles_n1=2)
        cap = layout.landing_rows(nlx, world, ec, w.tokens_per_rank, k)
        assert lay.lx_base[-1] + -(-lay.lx_rows[-1] // 128) * 128 <= cap
        # every GEMM1 task comes after all GEMM0 tasks of its M tile (deadlock freedom of the order)
        seen = set()
        for kind, lx, grp, n in lay.tasks:
            if kind == 0:
                seen.add((lx, grp, n))
            else:
                assert all((lx, grp, n0) in seen for n0 in range(3))

        # dispatch: (dst rank) -> list of (landing row, meta, row)
        outbox = [[] for _ in range(world)]
        for e in range(E):
            for j in range(lay.sent[rank][e]):
                t = int(r.table_tok[e, j])
                c = int(np.nonzero(r.topk_idx[t] == e)[0][0])
                outbox[emap[e]].append((lay.dst_row0[e] + j, (rank << 26) | (t * k + c), x[t].clone()))
        gathered = [None] * world
        dist.all_gather_object(gathered, outbox)
        landing, meta = {}, {}
        for src in range(world):
            for row, m, v in gathered[src][rank]:
                assert row not in landing, "two rows landed on the same slot"
                landing[row], meta[row] = v, m
        # experts on the packed rows
        back = [[] for _ in range(world)]
        for lx in range(nlx):
            e = rank * nlx + lx
            rows = list(range(lay.lx_base[lx], lay.lx_base[lx] + lay.lx_rows[lx]))
            assert all(rw in landing for rw in rows)
            if not rows:
                continue
            xe = torch.stack([landing[rw] for rw in rows])
            _, o = O.expert_mlp(xe, wts, e, int(w.mlp_type), int(w.act_type))
            for i, rw in enumerate(rows):
                back[meta[rw] >> 26].append((meta[rw] & ((1 << 26) - 1), o[i].clone()))
        returned = [None] * world
        dist.all_gather_object(returned, back)
        ret = {}
        for src in range(world):
            for row, v in returned[src][rank]:
                ret[row] = v
        S, H = x.shape
        out = torch.zeros(S, H, dtype=x.dtype)
        for t in range(S):
            acc = torch.zeros(H)
            for c in range(k):
                if r.topk_slot[t, c] < ec:
                    v = ret[t * k + c].float()
                    acc = v if k == 1 else acc + v * float(r.topk_w[t, c])
            out[t] = acc.to(x.dtype)
        ref, _ = oracle_layer(w, x=x, lw=lw)
        err = float((out.double() - ref.double()).abs().max() / ref.double().abs().max())
        q.put((rank, err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["bf16_gated_k2", "bf16_drop"])
def test_two_rank_exchange_matches_single_rank_oracle(name):
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, name, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in res:
        assert err < 1e-6, (rank, err)


def _failing_peer(rank, world, port, q):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    stage = "set-up"
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
        cb.initialize()
        dist.barrier()       # both ranks are up: what follows is the exchange itself
        stage = "exchange"
        if rank == 1:
            os._exit(0)      # leaves before the handle exchange, with nothing in flight
        cb.all_gather_bytes(b"x" * 64)
        q.put("no error")
    except Exception as exc:  # the survivor learns of it on the host, before any launch
        if rank == 0:
            q.put(("error: " if stage == "exchange" else "set-up failed: ") + type(exc).__name__)
    q.close()
    q.join_thread()          # the queue's feeder thread has written the message before the hard exit
    os._exit(0)


def test_a_rank_that_leaves_before_the_handle_exchange_is_noticed_on_the_host():
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_failing_peer, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    msg = q.get(timeout=60)
    for p in procs:
        p.join(timeout=30)
    assert msg.startswith("error"), msg


def _rank_map_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cb.initialize()
        res = {}
        # (1) a permuted map over the whole world: EP rank p lives in process world - 1 - p
        perm = [world - 1 - p for p in range(world)]
        got = cb.exchange_by_rank_map(bytes([rank]) * 8, world - 1 - rank, perm)
        res["permuted"] = [b[0] for b in got] == perm
        # (2) EP groups smaller than the world: {0, 1} and {2, 3}, the second one listed backwards
        groups = [[0, 1], [3, 2]]
        mine = groups[0] if rank in groups[0] else groups[1]
        got = cb.exchange_by_rank_map(bytes([100 + rank]) * 8, mine.index(rank), mine)
        res["subset"] = [b[0] for b in got] == [100 + g for g in mine]
        # (3) a map that does not describe this process is refused before anything is exchanged
        try:
            cb.exchange_by_rank_map(b"x", 0, [(rank + 1) % world])
            res["refused"] = False
        except ValueError:
            res["refused"] = True
        # (4) peers that disagree with the map: everyone claims EP rank 0 of a 2-rank group
        try:
            cb.exchange_by_rank_map(b"x", 0, [rank, (rank + 1) % world])
            res["disagree"] = False
        except ValueError:
            res["disagree"] = True
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_peer_handles_follow_rank_map():
    """The handle exchange of `initialize` resolves peers through rank_map (the reference's
    epRankToGlobalRank): a permuted map and EP groups smaller than the world give every rank its
    own group's payloads in EP-rank order; inconsistent maps raise on the host."""
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_map_main, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, r in res:
        assert all(r.values()), (rank, r)


def test_layout_matches_hand_computed_example():
    counts = [[3, 0, 130, 1], [2, 5, 0, 200]]
    lay = layout.build(counts, 1, [0, 0, 1, 1], ec=128, tiles_n0=2, tiles_n1=1, grid=1)
    assert lay.sent == [[3, 0, 128, 1], [2, 5, 0, 128]]
    # owner 0: expert 0 has 5 rows at base 0, expert 1 has 5 rows at base 128;
    # owner 1: expert 2 has 128 rows at base 0, expert 3 has 129 rows at base 128
    assert lay.dst_row0 == [3, 128, 128, 129]
    assert lay.lx_base == [0, 128] and lay.lx_rows == [128, 129]
    assert lay.mtile0 == [0, 1, 3]
    kinds = [(t[0], t[1]) for t in lay.tasks]
    # expert 0: one M tile, expert 1: two M tiles = one group (a CTA pair takes both)
    assert kinds == [(0, 0)] * 2 + [(0, 1)] * 2 + [(1, 0)] * 1 + [(1, 1)] * 1
    # a wider grid makes GEMM1 trail by more experts: all GEMM0 tiles first here
    wide = layout.build(counts, 1, [0, 0, 1, 1], ec=128, tiles_n0=2, tiles_n1=1, grid=148)
    assert [(t[0], t[1]) for t in wide.tasks] == kinds
    lone = layout.build(counts, 1, [0, 0, 1, 1], ec=128, tiles_n0=2, tiles_n1=1, grid=1, pair=False)
    assert [(t[0], t[1]) for t in lone.tasks] == [(0, 0)] * 2 + [(0, 1)] * 4 + [(1, 0)] * 1 + [(1, 1)] * 2
