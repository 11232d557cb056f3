"""CPU checks of the oracle itself: against the committed golden fixtures, against an
independent float64 evaluation, and against the structural invariants the reference's own
tests assert (csrc/tests/common.cuh:290-301: every token appears exactly k times, at most once
per expert, counts sum to S*k)."""
import numpy as np
import pytest
import torch

from cases import GOLDEN_CASES, ROUTER_CASES
from helpers import from_bits, golden, max_rel_err, oracle_layer, oracle_route, oracle_weights
from flashmoe_b200.workloads import TORCH_DTYPE, make_tokens, make_weights
from oracle import moe_oracle as O


def test_det_exp_is_accurate_and_monotone_enough():
    x = -np.linspace(0, 60, 200001).astype(np.float32)
    got = O.det_exp(x).astype(np.float64)
    want = np.exp(x.astype(np.float64))
    rel = np.abs(got - want) / want
    # the fp32 product x*log2(e) carries |x| * 2^-24 of absolute error into the exponent
    assert np.max(rel) < 1e-5
    assert np.max(rel[x > -1.0]) < 4e-7
    assert O.det_exp(np.float32(0.0)) == np.float32(1.0)


def test_router_logits_close_to_float64():
    w = ROUTER_CASES["r_bf16_e128_k8"]
    lw, x = make_weights(w), make_tokens(w)
    got = O.router_logits(x.float().numpy(), lw.router.float().numpy())
    want = x.double().numpy() @ lw.router.double().numpy().T
    assert np.max(np.abs(got - want)) < 1e-4


@pytest.mark.parametrize("name", list(ROUTER_CASES) + list(GOLDEN_CASES))
def test_router_matches_golden_bit_for_bit(name):
    w = ROUTER_CASES.get(name) or GOLDEN_CASES[name]
    lw = make_weights(w)
    wr = lw.router
    if name == "r_bf16_ties":
        wr = wr.clone()
        wr[1::2] = wr[0::2]
    r = oracle_route(w, router_w=wr, lw=lw)
    g = golden(name)
    assert np.array_equal(r.probs.view(np.uint32), g["probs_bits"])
    assert np.array_equal(r.topk_idx, g["topk_idx"])
    assert np.array_equal(r.topk_w.view(np.uint32), g["topk_w_bits"])
    assert np.array_equal(r.topk_slot, g["topk_slot"])
    assert np.array_equal(r.counts, g["counts"])
    assert np.array_equal(r.table_tok, g["table_tok"])


@pytest.mark.parametrize("name", list(ROUTER_CASES))
def test_routing_invariants(name):
    w = ROUTER_CASES[name]
    r = oracle_route(w)
    S, k, E = w.tokens_per_rank, w.top_k, w.num_experts
    assert int(r.counts.sum()) == S * k
    for t in range(S):
        assert len(set(r.topk_idx[t].tolist())) == k
    assert np.allclose(r.probs.sum(axis=1), 1.0, atol=1e-5)
    assert np.allclose(r.topk_w.sum(axis=1), 1.0, atol=1e-5)
    # selection order is by descending probability
    p_sel = np.take_along_axis(r.probs, r.topk_idx, axis=1)
    assert (np.diff(p_sel, axis=1) <= 0).all()
    # slots are handed out in ascending token order
    for e in range(E):
        n = min(int(r.counts[e]), w.expert_peer_capacity)
        assert (np.diff(r.table_tok[e, :n].astype(np.int64)) > 0).all()


def test_exact_ties_go_to_the_lower_expert():
    logits = np.zeros((3, 8), np.float32)
    logits[1, [2, 5]] = 1.0
    logits[2, 7] = 2.0
    r = O.route_from_logits(logits, 2, 8)
    assert r.topk_idx.tolist() == [[0, 1], [2, 5], [7, 0]]


@pytest.mark.parametrize("name", list(GOLDEN_CASES))
def test_layer_matches_golden_and_float64(name):
    w = GOLDEN_CASES[name]
    lw, x = make_weights(w), make_tokens(w)
    out, r = oracle_layer(w, x=x, lw=lw)
    gold = from_bits(golden(name)["out_bits"], TORCH_DTYPE[w.data_type]).reshape(out.shape)
    # CPU GEMM blocking may differ between hosts: one Element ulp of slack, not bit equality
    assert max_rel_err(out, gold) <= 1e-2
    dense = O.dense_f64(x, r, oracle_weights(lw), w.top_k, w.expert_peer_capacity, int(w.mlp_type),
                        int(w.act_type))
    assert max_rel_err(out, dense) <= 2e-2
    if w.top_k > 1:
        lit, _ = oracle_layer(w, x=x, lw=lw, combine="element")
        assert max_rel_err(lit, dense) <= 3e-2


def test_dropped_tokens_follow_the_capacity_rule():
    w = GOLDEN_CASES["bf16_drop"]
    out, r = oracle_layer(w)
    ec = w.expert_peer_capacity
    assert (r.counts > ec).any()
    fully_dropped = (r.topk_slot >= ec).all(axis=1)
    assert fully_dropped.any()
    assert (out[torch.from_numpy(fully_dropped)] == 0).all()
