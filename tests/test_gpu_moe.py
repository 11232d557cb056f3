"""GPU parity of the fused forward (dispatch + expert GEMMs + combine) at world size 1:
stage by stage against the CPU oracle, end to end against the oracle and the golden
fixtures, and through size-independent properties at benchmark shapes."""
import numpy as np
import pytest
import torch

from cases import GOLDEN_CASES
from helpers import REL_TOL, assert_close, from_bits, golden, max_rel_err, oracle_layer, oracle_weights
from flashmoe_b200.workloads import CONFIGS, TORCH_DTYPE, make_tokens, make_weights
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def make_layer(w, lw=None):
    from flashmoe_b200.layer import MoELayer
    return MoELayer(w, lw or make_weights(w))


@pytest.mark.parametrize("name", list(GOLDEN_CASES))
def test_forward_matches_oracle_and_golden(name):
    w = GOLDEN_CASES[name]
    lw, x = make_weights(w), make_tokens(w)
    ref, r = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        out = layer.forward(x).cpu()
        assert_close(out, ref, w.data_type, f"{name} vs oracle")
        gold = from_bits(golden(name)["out_bits"], TORCH_DTYPE[w.data_type]).reshape(ref.shape)
        assert_close(out, gold, w.data_type, f"{name} vs golden")
        # a second and third launch on the same context (epoch protocol, no host-side clearing)
        for _ in range(2):
            again = layer.forward(x).cpu()
            assert torch.equal(again, out)
    finally:
        layer.close()


def test_fp32_reference_configuration():
    """The benchmark description's first configuration: FP32, 128 tokens, H=1024, I=2048, E=8, k=2,
    gated SiLU, one rank; tolerance 1e-5 of the output's largest magnitude."""
    w = CONFIGS["cpu_ref_fp32"]
    lw, x = make_weights(w), make_tokens(w)
    ref, r = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        out = layer.forward(x).cpu()
        assert_close(out, ref, w.data_type, "cpu_ref_fp32 vs oracle")
        dense = O.dense_f64(x, r, oracle_weights(lw), w.top_k, w.expert_peer_capacity, int(w.mlp_type),
                            int(w.act_type))
        assert_close(out, dense, w.data_type, "cpu_ref_fp32 vs float64 evaluation")
    finally:
        layer.close()


@pytest.mark.parametrize("name", ["bf16_two_mtiles", "bf16_gated_k2", "fp32_gated_k2"])
def test_cta_pair_form_of_the_gemm_loop(name, monkeypatch):
    """FMOE_PAIR=1 selects the tcgen05.mma.cta_group::2 form (CTA pairs on 256-row tile groups);
    it must give the same answers as the default form."""
    monkeypatch.setenv("FMOE_PAIR", "1")
    w = GOLDEN_CASES[name]
    lw, x = make_weights(w), make_tokens(w)
    ref, _ = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        assert layer.geometry().cta_pairs == 1
        for _ in range(2):
            out = layer.forward(x).cpu()
            assert max_rel_err(out, ref) <= REL_TOL[int(w.data_type)]
    finally:
        layer.close()


@pytest.mark.parametrize("parts", ["1", "2", "4"])
@pytest.mark.parametrize("name", ["bf16_two_mtiles", "fp32_gated_k2"])
def test_closing_gemm1_tiles_cut_along_k(name, parts, monkeypatch):
    """The last GEMM1 tiles of the task order are cut along K into FMOE_SPLIT_PARTS tickets whose
    fp32 partial sums are added in part order (1 = never cut).  I = 512 gives eight K blocks, two
    per part at 4 parts; every tile of these small cases is a closing tile."""
    monkeypatch.setenv("FMOE_SPLIT_PARTS", parts)
    w = GOLDEN_CASES[name].scaled(token_dim=512, ffn_size=1024)
    lw, x = make_weights(w), make_tokens(w)
    ref, _ = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        assert layer.geometry().split_parts == int(parts)
        first = layer.forward(x).cpu()
        assert_close(first, ref, w.data_type, f"{name} split {parts}")
        assert torch.equal(layer.forward(x).cpu(), first)      # same bits on every launch
    finally:
        layer.close()


@pytest.mark.parametrize("name", ["bf16_gated_k2", "fp32_vanilla_gelu_k4"])
def test_specialised_kernel_gives_the_generic_kernel_s_bits(name, monkeypatch):
    """The kernel compiled for this layer's description (H, I, top-k, MLP type, activation and
    element type as constants; built by flashmoe_b200.jit, cached in the package) against the
    generic one that reads them from the launch parameters."""
    w = GOLDEN_CASES[name]
    lw, x = make_weights(w), make_tokens(w)
    ref, _ = oracle_layer(w, x=x, lw=lw)
    outs = {}
    for mode in ("off", "1"):
        monkeypatch.setenv("FMOE_JIT", mode)
        layer = make_layer(w, lw)
        try:
            assert layer.geometry().specialised == (0 if mode == "off" else 1)
            outs[mode] = layer.forward(x).cpu()
            assert_close(outs[mode], ref, w.data_type, f"{name} FMOE_JIT={mode}")
        finally:
            layer.close()
    assert torch.equal(outs["off"], outs["1"])


@pytest.mark.parametrize("name", ["bf16_gated_k2", "bf16_drop", "bf16_vanilla_gelu_k8", "fp32_gated_k2",
                                  "fp16_gated_relu", "bf16_two_mtiles"])
def test_router_inside_the_launch_gives_the_same_bits(name):
    """fmoe_forward_routed: ONE launch whose first phase is the router.  Counts, route records,
    probabilities and the layer's output must equal, bit for bit, what router.forward followed by
    forward gives; repeated launches and new tokens included."""
    w = GOLDEN_CASES[name]
    lw = make_weights(w)
    S, E, k = w.tokens_per_rank, w.num_experts, w.top_k
    from flashmoe_b200.layer import MoELayer
    layer = MoELayer(w, lw, return_logits=True)
    try:
        for step in range(3):
            x = make_tokens(w.scaled(seed=w.seed + step))
            layer.tokens.copy_(x)
            torch.cuda.synchronize()
            layer.step()
            layer.check()
            want = (layer.out.clone(), layer.counts.clone(), layer.routing.clone(),
                    layer.debug(4, torch.int32, (S, k, 4))[:, :, :3].clone())
            layer.out.zero_(); layer.counts.zero_(); layer.routing.zero_()
            before = _launches()
            layer.step_one_launch()
            layer.check()
            assert _launches() - before == 1
            got = (layer.out, layer.counts, layer.routing, layer.debug(4, torch.int32, (S, k, 4))[:, :, :3])
            assert torch.equal(got[1], want[1]), "counts"
            assert torch.equal(got[3], want[3]), "route records"
            assert torch.equal(got[2].view(torch.int32), want[2].view(torch.int32)), "probabilities"
            assert torch.equal(got[0].view(torch.uint8), want[0].view(torch.uint8)), "output"
        ref, _ = oracle_layer(w, x=x, lw=lw)
        assert_close(layer.out.cpu(), ref, w.data_type, f"{name} routed in the launch")
    finally:
        layer.close()


def test_router_inside_the_launch_at_decode_sizes():
    """Qwen3 shapes with 1 and 16 tokens: the case the one-launch form is for."""
    for S in (1, 16):
        w = CONFIGS["qwen3"].scaled(tokens_per_rank=S)
        lw, x = make_weights(w), make_tokens(w)
        ref, _ = oracle_layer(w, x=x, lw=lw)
        layer = make_layer(w, lw)
        try:
            layer.tokens.copy_(x)
            torch.cuda.synchronize()
            for _ in range(2):
                layer.step_one_launch()
                layer.check()
            assert_close(layer.out.cpu(), ref, w.data_type, f"qwen3 with {S} tokens, one launch")
        finally:
            layer.close()


@pytest.mark.parametrize("name", ["bf16_gated_k2", "fp32_gated_k2"])
def test_context_in_memory_the_caller_owns(name):
    """fmoe_ctx_create_in: the symmetric block and the workspace are the caller's (sized by the
    host-side query); creating the context and running forwards takes no device memory, the
    results are those of a context that allocated for itself, and destroying it leaves the
    caller's blocks alone."""
    import flashmoe_b200 as flashmoe
    from flashmoe_b200.layer import MoELayer
    w = GOLDEN_CASES[name]
    lw, x = make_weights(w), make_tokens(w)
    own = make_layer(w, lw)
    try:
        want = own.forward(x).cpu()
        need = flashmoe.get_workspace_bytes(own.args)
    finally:
        own.close()
    symm = torch.empty(need["symmetric"] + 1024, dtype=torch.uint8, device="cuda")
    work = torch.empty(need["workspace"] + 1024, dtype=torch.uint8, device="cuda")
    up = lambda t: (t.data_ptr() + 1023) // 1024 * 1024
    memory = (up(symm), need["symmetric"], up(work), need["workspace"])
    # creating (and destroying) a context inside the caller's blocks takes no device memory
    import ctypes as C
    from flashmoe_b200 import _native as N
    a = own.args
    ep = N.EpDesc(1, 0, 0, 0, w.num_experts, 0, (C.c_int32 * w.num_experts)(*([0] * w.num_experts)), (C.c_int32 * 1)(0))
    desc, raw = flashmoe._model_desc(a), C.c_void_p()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    assert N.lib().fmoe_ctx_create_in(C.byref(desc), C.byref(ep), None, C.c_void_p(memory[0]), memory[1],
                                      C.c_void_p(memory[2]), memory[3], C.byref(raw)) == 0, N.lib().fmoe_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert N.lib().fmoe_ctx_destroy(raw, None) == 0
    layer = MoELayer(w, lw, memory=memory)
    try:
        got = layer.forward(x).cpu()
        assert torch.equal(got, want)
        assert torch.equal(layer.forward(x).cpu(), want)
    finally:
        layer.close()
    # too little memory is refused with the sizes in the message
    with pytest.raises(flashmoe.FlashMoEError) as err:
        MoELayer(w, lw, memory=(memory[0], 4096, memory[2], memory[3]))
    assert str(need["symmetric"]) in str(err.value)
    del symm, work


def test_one_context_serves_several_layers():
    """Three layers of one model (same shapes, different weights) run through ONE context, in turn
    and repeatedly: every forward equals what a context of its own gives for that layer, bit for
    bit, and after the first visit a layer's forward builds no new TMA descriptors (the same
    number of launches, nothing allocated).  Sizes match the host-side query."""
    import flashmoe_b200 as flashmoe
    w = GOLDEN_CASES["bf16_gated_k2"]
    sets = [make_weights(w.scaled(seed=w.seed + 100 * i)) for i in range(3)]
    x = make_tokens(w)
    own = []
    for lw in sets:
        layer = make_layer(w, lw)
        try:
            own.append(layer.forward(x).cpu())
            ref, _ = oracle_layer(w, x=x, lw=lw)
            assert max_rel_err(own[-1], ref) <= REL_TOL[int(w.data_type)]
        finally:
            layer.close()
    assert not torch.equal(own[0], own[1])
    shared = make_layer(w, sets[0])
    try:
        g = shared.geometry()
        q = flashmoe.get_workspace_bytes(shared.args)
        assert q == {"symmetric": g.symm_bytes, "workspace": g.workspace_bytes}
        idx = [0, shared.add_layer(sets[1]), shared.add_layer(sets[2])]
        for _ in range(3):
            for i in (0, 1, 2, 1, 0):
                shared.select_layer(idx[i])
                assert torch.equal(shared.forward(x).cpu(), own[i]), i
    finally:
        shared.close()


def test_forwards_replay_from_a_cuda_graph():
    """The reference times its kernel by capturing many forwards in one CUDA graph and replaying
    it (quickstart.py:264-291).  Nothing on the host changes between launches here either: the
    epoch lives in device memory."""
    w = GOLDEN_CASES["bf16_gated_k2"]
    lw, x = make_weights(w), make_tokens(w)
    ref, _ = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        layer.forward(x)                      # warm-up outside the capture, routes the tokens
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=layer.stream):
            for _ in range(4):
                layer.step()             # router (2 launches) + fused forward
        layer.out.zero_()
        for _ in range(3):
            with torch.cuda.stream(layer.stream):
                g.replay()
        layer.stream.synchronize()
        layer.check()
        assert max_rel_err(layer.out.cpu(), ref) <= 2e-2
    finally:
        layer.close()


def test_stages_dispatch_gemm0_gemm1():
    """Checks the intermediate buffers: landed rows (exact), GEMM0 output and returned rows."""
    w = GOLDEN_CASES["bf16_gated_k2"]
    lw, x = make_weights(w), make_tokens(w)
    _, r = oracle_layer(w, x=x, lw=lw)
    wts = oracle_weights(lw)
    layer = make_layer(w, lw)
    try:
        layer.forward(x)
        g = layer.geometry()
        S, H, I, E, k = w.tokens_per_rank, w.token_dim, w.ffn_size, w.num_experts, w.top_k
        landing = layer.debug(0, torch.bfloat16, (g.landing_rows, H)).cpu()
        meta = layer.debug(1, torch.int32, (g.landing_rows,)).cpu().numpy().view(np.uint32)
        y = layer.debug(2, torch.bfloat16, (g.landing_rows, I)).cpu()
        ret = layer.debug(3, torch.bfloat16, (S * k, H)).cpu()
        base = 0
        for e in range(E):
            n = min(int(r.counts[e]), w.expert_peer_capacity)
            ids = torch.from_numpy(r.table_tok[e, :n].astype(np.int64))
            assert torch.equal(landing[base:base + n].view(torch.int16), x[ids].view(torch.int16)), f"expert {e}"
            ye, oe = O.expert_mlp(x[ids], wts, e, int(w.mlp_type), int(w.act_type))
            if n:
                assert max_rel_err(y[base:base + n], ye) <= 2e-2, f"gemm0 expert {e}"
                rows = meta[base:base + n] & ((1 << 26) - 1)
                assert np.array_equal(rows // k, r.table_tok[e, :n])
                assert max_rel_err(ret[torch.from_numpy(rows.astype(np.int64))], oe) <= 2e-2, f"gemm1 expert {e}"
            base += -(-n // 128) * 128
    finally:
        layer.close()


def test_new_tokens_each_step_and_empty_experts():
    """Different inputs on consecutive launches; a skewed router leaves several experts empty."""
    w = GOLDEN_CASES["bf16_drop"].scaled(capacity=None)
    lw = make_weights(w)
    layer = make_layer(w, lw)
    try:
        for step in range(3):
            x = make_tokens(w.scaled(seed=w.seed + step))
            ref, r = oracle_layer(w, x=x, lw=lw)
            out = layer.forward(x).cpu()
            assert_close(out, ref, w.data_type, f"step {step}")
        assert (r.counts == 0).any(), "the skewed router was meant to leave an expert empty"
    finally:
        layer.close()


def test_k1_dropped_rows_are_left_untouched():
    w = GOLDEN_CASES["bf16_gated_k1_bias"].scaled(capacity=3)
    lw, x = make_weights(w), make_tokens(w)
    ref, r = oracle_layer(w, x=x, lw=lw)
    dropped = r.topk_slot[:, 0] >= 3
    assert dropped.any()
    layer = make_layer(w, lw)
    try:
        layer.out.fill_(7.0)
        out = layer.forward(x).cpu()
        keep = torch.from_numpy(~dropped)
        assert max_rel_err(out[keep], ref[keep]) <= 2e-2
        assert (out[torch.from_numpy(dropped)].float() == 7.0).all()
    finally:
        layer.close()


@pytest.mark.parametrize("cfg,S", [("scout", 256), ("mixtral", 256), ("qwen3", 128), ("deepseek_v3", 64)])
def test_benchmark_shapes_trimmed_tokens(cfg, S):
    """Full H, I, E, k of the benchmark configurations with fewer tokens (the oracle runs every
    routed pair through fp32 CPU GEMMs)."""
    w = CONFIGS[cfg].scaled(tokens_per_rank=S)
    if cfg == "deepseek_v3":
        w = w.scaled(num_experts=64)       # 64 x 3 x 7168 x 2048 bf16 = 5.6 GB of weights on the host
    lw, x = make_weights(w), make_tokens(w)
    ref, r = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        out = layer.forward(x).cpu()
        assert_close(out, ref, w.data_type, f"{cfg} with {S} tokens")
    finally:
        layer.close()


@pytest.mark.parametrize("S", [1, 16])
def test_qwen3_decode_sizes(S):
    """The decode end of the Qwen3-30B-A3B sweep (1 and 16 tokens, E = 128, k = 8)."""
    w = CONFIGS["qwen3"].scaled(tokens_per_rank=S)
    lw, x = make_weights(w), make_tokens(w)
    ref, _ = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        for _ in range(2):
            out = layer.forward(x).cpu()
            assert_close(out, ref, w.data_type, f"qwen3 with {S} tokens")
    finally:
        layer.close()


@pytest.mark.parametrize("S", [16, 1024])
def test_qwen3_fp32_plain_gelu(S):
    """The FP32 leg of the Qwen3 sweep: plain (non-gated) MLP with GELU, all 128 experts' shapes, at
    16 and at 1024 tokens; tolerance 1e-5.  The second forward reuses the BF16 planes of the
    weights (nothing is split again) and must give the same bits."""
    w = CONFIGS["qwen3_fp32_gelu"].scaled(tokens_per_rank=S)
    lw, x = make_weights(w), make_tokens(w)
    ref, _ = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        out = layer.forward(x).cpu()
        assert_close(out, ref, w.data_type, f"qwen3 fp32 gelu with {S} tokens")
        before = _launches()
        assert torch.equal(layer.forward(x).cpu(), out)
        assert _launches() - before == 3, "weight planes were split again"
    finally:
        layer.close()


def _launches():
    from flashmoe_b200 import _native
    return _native.lib().fmoe_launch_count()


def _same_up_to_split_order(a, b):
    """A token's output depends on that token only.  Its bits may still differ between two batches:
    rows that fall into a GEMM1 tile of the closing wave have their K sum formed in parts (fp32, fixed
    order), the others in one pass, and a permutation moves rows between the two kinds of tile.  An
    expert's output row can therefore move by one unit in the last place of the 16-bit type, and a
    token's output by that much times its combine weight.  So: most elements identical, and every
    element within a few units in the last place of the larger of itself and a typical output."""
    assert (a == b).double().mean() >= 0.5
    diff = (a.double() - b.double()).abs()
    bound = 2.0 ** -6 * b.double().abs() + 2.0 ** -5 * float(b.double().pow(2).mean().sqrt())
    assert bool((diff <= bound).all()), float((diff / bound).max())


def _device_layer(w):
    """Layer with weights drawn on the GPU (full-size configurations: tens of GB would take minutes
    to draw on the host)."""
    import importlib.util
    import os
    from flashmoe_b200.layer import MoELayer
    spec = importlib.util.spec_from_file_location(
        "bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    lw = bench.device_weights(w, torch.device("cuda", 0), list(range(w.num_experts)))
    return MoELayer(w, lw, 0, local_experts=range(w.num_experts)), lw


@pytest.mark.parametrize("cfg,S", [("mixtral", 4096), ("deepseek_v3", 2048), ("qwen3", 8192)])
def test_full_size_properties(cfg, S):
    """Mixtral, DeepSeek-V3-shaped and Qwen3 (prefill end) at their full benchmark sizes, through
    properties that need no full-size oracle: finite output, determinism across launches, bit-exact
    equivariance under a permutation of the tokens, and a handful of tokens against the oracle
    (only the experts those tokens use are copied to the host)."""
    w = CONFIGS[cfg].scaled(tokens_per_rank=S)
    layer, lw = _device_layer(w)
    try:
        x = make_tokens(w)
        out = layer.forward(x).cpu()
        assert torch.isfinite(out.float()).all()
        again = layer.forward(x).cpu()
        assert torch.equal(out, again)
        perm = torch.randperm(S, generator=torch.Generator().manual_seed(9))
        outp = layer.forward(x[perm]).cpu()
        _same_up_to_split_order(outp, out[perm])
        # spot tokens: route them with the oracle, run their experts on the host
        sel = torch.arange(0, S, S // 6)[:6]
        bias = None if lw.logit_bias is None else lw.logit_bias.cpu().numpy()
        r = O.route(x[sel].float().numpy(), lw.router.cpu().float().numpy(), w.top_k, len(sel), logit_bias=bias)
        for i, t in enumerate(sel.tolist()):
            acc = torch.zeros(w.token_dim)
            for j in range(w.top_k):
                e = int(r.topk_idx[i, j])
                one = O.ExpertWeights(lw.up[e:e + 1].cpu(), None if lw.up_v is None else lw.up_v[e:e + 1].cpu(),
                                      lw.down[e:e + 1].cpu(), lw.bias_up[e:e + 1].cpu(),
                                      None if lw.bias_up_v is None else lw.bias_up_v[e:e + 1].cpu(),
                                      lw.bias_down[e:e + 1].cpu())
                _, o = O.expert_mlp(x[t:t + 1], one, 0, int(w.mlp_type), int(w.act_type))
                acc = o[0].float() if w.top_k == 1 else acc + o[0].float() * float(r.topk_w[i, j])
            ref_t = acc.to(out.dtype)
            assert max_rel_err(out[t], ref_t) <= 2e-2, (t, max_rel_err(out[t], ref_t))
    finally:
        layer.close()


def test_full_size_scout_properties():
    """Scout at its full benchmark size (S = 1024, H = 5120, I = 8192, E = 16, k = 1), checked
    through properties that need no full-size oracle: (1) determinism across launches, (2) a
    token's output depends only on that token: permuting the tokens permutes the outputs
    bit for bit, (3) spot rows against the oracle."""
    w = CONFIGS["scout"]
    lw, x = make_weights(w), make_tokens(w)
    layer = make_layer(w, lw)
    try:
        out = layer.forward(x).cpu()
        assert torch.isfinite(out.float()).all()
        again = layer.forward(x).cpu()
        assert torch.equal(out.view(torch.int16), again.view(torch.int16))
        perm = torch.randperm(w.tokens_per_rank, generator=torch.Generator().manual_seed(5))
        outp = layer.forward(x[perm]).cpu()
        _same_up_to_split_order(outp, out[perm])
        # spot check 32 tokens through the oracle (their routing needs only their own rows)
        sel = torch.arange(0, w.tokens_per_rank, 32)
        ws = w.scaled(tokens_per_rank=len(sel))
        ref, _ = O.layer_forward(x[sel], lw.router, oracle_weights(lw), w.top_k, len(sel),
                                 int(w.mlp_type), int(w.act_type))
        assert max_rel_err(out[sel], ref) <= 2e-2, max_rel_err(out[sel], ref)
    finally:
        layer.close()


def test_host_buffer_entry_point():
    w = GOLDEN_CASES["bf16_gated_k2"]
    lw, x = make_weights(w), make_tokens(w)
    ref, _ = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        xh = x.clone().pin_memory()
        oh = torch.zeros_like(xh).pin_memory()
        layer.forward_host(xh, oh)
        layer.check()
        assert max_rel_err(oh, ref) <= 2e-2
    finally:
        layer.close()


def test_a_wait_that_runs_out_is_reported_and_the_gpu_stays_usable(monkeypatch):
    """Failure detection without a fault: the count flags are withheld (nothing ever sets what the
    first wait polls), the wait gives up after its limit, the kernel leaves through its common
    exit and the host reads {code, phase} from the status record.  A fresh context then works."""
    import flashmoe_b200 as flashmoe
    w = GOLDEN_CASES["bf16_gated_k2"]
    lw, x = make_weights(w), make_tokens(w)
    monkeypatch.setenv("FMOE_WITHHOLD_FLAGS", "1")
    monkeypatch.setenv("FMOE_SPIN_LIMIT_MS", "20")
    layer = make_layer(w, lw)
    try:
        with pytest.raises(flashmoe.FlashMoEError) as err:
            layer.forward(x)
        assert err.value.code == 5 and "phase 1" in str(err.value)      # DEVICE_TIMEOUT in the count wait
        st = layer.handle.mod.last_status(layer.handle.context, layer.stream.cuda_stream)
        assert (st.code, st.phase, st.rank) == (5, 1, 0)
        # the context is poisoned from here on: nothing is launched on it any more
        before = _launches()
        with pytest.raises(flashmoe.FlashMoEError) as again:
            layer.step()
        assert again.value.code == 5 and _launches() == before
    finally:
        layer.close()
    monkeypatch.delenv("FMOE_WITHHOLD_FLAGS")
    monkeypatch.delenv("FMOE_SPIN_LIMIT_MS")
    ref, _ = oracle_layer(w, x=x, lw=lw)
    layer = make_layer(w, lw)
    try:
        assert max_rel_err(layer.forward(x).cpu(), ref) <= 2e-2
    finally:
        layer.close()


def test_pipelined_host_buffer_entry_point():
    """fmoe_forward_host_async: five steps with different tokens, copies overlapping kernels; every
    step's result must land in its own host buffer."""
    w = GOLDEN_CASES["bf16_gated_k2"]
    lw = make_weights(w)
    layer = make_layer(w, lw)
    try:
        xs = [make_tokens(w.scaled(seed=w.seed + i)).pin_memory() for i in range(5)]
        outs = [torch.zeros_like(x).pin_memory() for x in xs]
        for x, o in zip(xs, outs):
            layer.forward_host(x, o, wait=False)
        layer.host_wait()
        layer.check()
        for x, o in zip(xs, outs):
            ref, _ = oracle_layer(w, x=x, lw=lw)
            assert max_rel_err(o, ref) <= 2e-2
    finally:
        layer.close()


def test_argument_errors_are_reported_not_fatal():
    import flashmoe_b200 as flashmoe
    w = GOLDEN_CASES["bf16_gated_k2"]
    layer = make_layer(w)
    try:
        bad = flashmoe.ForwardArgs(mt=w.mlp_type, tokens=0, expert_counts=layer.counts.data_ptr(),
                                   local_expert_up=layer.up.data_ptr(), local_bias_up=0,
                                   local_expert_down=layer.down.data_ptr(), local_bias_down=0,
                                   moe_out=layer.out.data_ptr(), stream_ptr=layer.stream.cuda_stream,
                                   local_expert_up_v=layer.up_v.data_ptr(), local_bias_up_v=0)
        with pytest.raises(flashmoe.FlashMoEError):
            flashmoe.forward(layer.handle, bad)
        # the context is still usable
        out = layer.forward(make_tokens(w))
        assert torch.isfinite(out.float()).all()
    finally:
        layer.close()
