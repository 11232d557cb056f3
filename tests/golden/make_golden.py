"""Generates tests/golden/*.npz from the CPU oracle:  python tests/golden/make_golden.py

Inputs are NOT stored: every case is regenerated from its seed by flashmoe_b200.workloads.
Stored per case: the router's integer results and the raw bits of its probabilities, and
the layer output as raw Element bits.  The reference ships no golden vectors of its own and
cannot run without a GPU, so these pin the oracle against drift, not against the reference.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from cases import GOLDEN_CASES, ROUTER_CASES  # noqa: E402
from flashmoe_b200.workloads import make_tokens, make_weights  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.float32:
        return t.numpy().view(np.uint32)
    return t.view(torch.int16).numpy().view(np.uint16)


def ties_tokens(w):
    """Tokens whose logits tie exactly: expert weight rows duplicated pairwise."""
    x = make_tokens(w)
    lw = make_weights(w)
    r = lw.router.clone()
    r[1::2] = r[0::2]
    return x, r


def router_case(w):
    lw = make_weights(w)
    x = make_tokens(w)
    wr = lw.router
    if w.name == "r_bf16_ties":
        x, wr = ties_tokens(w)
    bias = None if lw.logit_bias is None else lw.logit_bias.numpy()
    r = O.route(x.float().numpy(), wr.float().numpy(), w.top_k, w.expert_peer_capacity, logit_bias=bias)
    return dict(probs_bits=r.probs.view(np.uint32), topk_idx=r.topk_idx, topk_w_bits=r.topk_w.view(np.uint32),
                topk_slot=r.topk_slot, counts=r.counts, table_tok=r.table_tok,
                table_w_bits=r.table_w.view(np.uint32))


def layer_case(w):
    lw = make_weights(w)
    x = make_tokens(w)
    wts = O.ExpertWeights(lw.up, lw.up_v, lw.down, lw.bias_up, lw.bias_up_v, lw.bias_down)
    bias = None if lw.logit_bias is None else lw.logit_bias.numpy()
    out, r = O.layer_forward(x, lw.router, wts, w.top_k, w.expert_peer_capacity, int(w.mlp_type),
                             int(w.act_type), logit_bias=bias)
    d = router_case(w)
    d["out_bits"] = bits(out)
    return d


if __name__ == "__main__":
    torch.set_num_threads(1)
    for name, w in ROUTER_CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **router_case(w))
        print("wrote", name)
    for name, w in GOLDEN_CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **layer_case(w))
        print("wrote", name)
