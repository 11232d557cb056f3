"""GPU parity of the router: every integer result and the raw bits of every probability must
equal the CPU oracle's and the committed golden fixtures."""
import numpy as np
import pytest
import torch

from cases import GOLDEN_CASES, ROUTER_CASES
from helpers import golden, oracle_route
from flashmoe_b200.workloads import CONFIGS, TORCH_DTYPE, make_tokens, make_weights

pytestmark = pytest.mark.gpu


def run_router(w, x, router_w, logit_bias):
    """Router alone through the C ABI (the MoE context only lends its routing table)."""
    from flashmoe_b200.layer import MoELayer
    from flashmoe_b200.workloads import LayerWeights
    from flashmoe_b200.jit import DataType
    E, H, I = w.num_experts, w.token_dim, w.ffn_size
    # The expert kernels are 16-bit only; a router-only run of an fp32 case borrows a bf16 context.
    wm = w if w.data_type != DataType.FP32 else w.scaled(data_type=DataType.BF16)
    z = lambda *s: torch.zeros(*s, dtype=TORCH_DTYPE[wm.data_type])
    lw = LayerWeights(router_w, z(E, I, H), z(E, I, H), z(E, H, I), z(E, I), z(E, I), z(E, H), logit_bias)
    layer = MoELayer(wm, lw, return_logits=True)
    try:
        import flashmoe_b200 as flashmoe
        if w.data_type == DataType.FP32:
            # fp32 router context, fp32 tokens and weights
            rh = flashmoe.router.initialize(_init_args(w, layer), return_logits=True)
            xt, wt = x.cuda(), router_w.cuda()
            ra = flashmoe.router.RouterForwardArgs(
                tokens=xt.data_ptr(), weights=wt.data_ptr(), expert_counts=layer.counts.data_ptr(),
                stream_ptr=layer.stream.cuda_stream, routing=layer.routing.data_ptr(),
                logit_bias=0 if layer.logit_bias is None else layer.logit_bias.data_ptr())
            torch.cuda.synchronize()
            flashmoe.router.forward(rh, layer.handle, ra)
            layer.stream.synchronize()
            flashmoe.router.finalize(rh, layer.stream.cuda_stream)
        else:
            layer.tokens.copy_(x)
            torch.cuda.synchronize()
            layer.route()
            layer.stream.synchronize()
        S, k = w.tokens_per_rank, w.top_k
        routes = layer.debug(4, torch.int32, (S, k, 4)).cpu().numpy()
        g = layer.geometry()
        table = _table(layer, E, g.round_ec)
        return dict(counts=layer.counts.cpu().numpy(), probs=layer.routing.cpu().numpy(),
                    expert=routes[:, :, 0], slot=routes[:, :, 1],
                    weight=routes[:, :, 2].copy().view(np.float32), table=table, round_ec=g.round_ec)
    finally:
        layer.close()


def _init_args(w, layer):
    import flashmoe_b200 as flashmoe
    return flashmoe.InitArgs(data_type=w.data_type, tokens_per_rank=w.tokens_per_rank, token_dim=w.token_dim,
                             ffn_size=w.ffn_size, num_experts=w.num_experts, top_k=w.top_k, gpu_arch=1000,
                             mlp_type=w.mlp_type, act_type=w.act_type, stream_ptr=layer.stream.cuda_stream,
                             device_id=0, expert_peer_capacity=w.expert_peer_capacity)


def _table(layer, E, round_ec):
    ptr = layer.handle.mod.get_tIdx(layer.handle.context)

    class _Raw:
        __cuda_array_interface__ = {"shape": (E * round_ec * 2,), "typestr": "<u4", "data": (ptr, False),
                                    "version": 2}
    torch.cuda.synchronize()
    return torch.as_tensor(_Raw(), device="cuda").clone().cpu().numpy().reshape(E, round_ec, 2)


def check_against(r, got, w):
    """r: oracle Routing; got: dict from run_router.  Bit-exact everywhere."""
    assert np.array_equal(got["counts"], r.counts)
    assert np.array_equal(got["expert"], r.topk_idx)
    assert np.array_equal(got["slot"], r.topk_slot)
    assert np.array_equal(got["weight"].view(np.uint32), r.topk_w.view(np.uint32))
    assert np.array_equal(got["probs"].view(np.uint32), r.probs.view(np.uint32))
    ec = w.expert_peer_capacity
    for e in range(w.num_experts):
        n = min(int(r.counts[e]), ec)
        assert np.array_equal(got["table"][e, :n, 0], r.table_tok[e, :n])
        assert np.array_equal(got["table"][e, :n, 1], r.table_w[e, :n].view(np.uint32))


@pytest.mark.parametrize("name", list(ROUTER_CASES) + list(GOLDEN_CASES))
def test_router_bit_exact_vs_oracle_and_golden(name):
    w = (ROUTER_CASES.get(name) or GOLDEN_CASES[name])
    lw = make_weights(w)
    x, wr = make_tokens(w), lw.router
    if name == "r_bf16_ties":
        wr = wr.clone()
        wr[1::2] = wr[0::2]
    r = oracle_route(w, x=x, router_w=wr, lw=lw)
    got = run_router(w, x, wr, lw.logit_bias)
    check_against(r, got, w)
    g = golden(name)
    assert np.array_equal(got["counts"], g["counts"])
    assert np.array_equal(got["expert"], g["topk_idx"])
    assert np.array_equal(got["probs"].view(np.uint32), g["probs_bits"])
    if name == "r_bf16_ties":
        # duplicated router rows tie exactly: the lower expert id of each pair must come first
        ex = got["expert"]
        pos = {int(e): j for j, e in enumerate(ex[0])}
        for e in ex[0]:
            if e % 2 == 1:
                assert (e - 1) in pos and pos[e - 1] < pos[int(e)]


@pytest.mark.parametrize("cfg,S", [("scout", 1024), ("qwen3", 1), ("qwen3", 16), ("qwen3", 1024),
                                   ("deepseek_v3", 512), ("cpu_ref_fp32", 128)])
def test_router_benchmark_shapes(cfg, S):
    """Full H and E of the benchmark configurations (token count trimmed where the oracle would
    take long); also checks the structural invariants the reference's tests assert
    (csrc/tests/common.cuh:290-301)."""
    w = CONFIGS[cfg].scaled(tokens_per_rank=S, ffn_size=64)
    lw = make_weights(w)
    x = make_tokens(w)
    r = oracle_route(w, x=x, lw=lw)
    got = run_router(w, x, lw.router, lw.logit_bias)
    check_against(r, got, w)
    assert int(got["counts"].sum()) == S * w.top_k
    for t in range(min(S, 64)):
        assert len(set(got["expert"][t].tolist())) == w.top_k
