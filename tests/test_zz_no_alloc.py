"""The allocation-free router entry point (fmoe_router_forward_static) against the regular one.

Who needs it: a caller that may not allocate device memory when it asks for a routing decision
-- an inference engine whose own pool already owns the GPU and which treats a later cudaMalloc
as an error (it may fail and it synchronises the device), or a plug-in invoked between the
engine's launches.  The regular router keeps its scratch in a context it allocates; this one
keeps it in a fixed array inside the library.  Both must give the same bits.

This file sorts last on purpose, so that a run stopping at the first failure has already been
through every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from cases import GOLDEN_CASES
from flashmoe_b200 import _native as N
from flashmoe_b200.workloads import make_tokens, make_weights

pytestmark = pytest.mark.gpu


def _raw(ptr, nbytes):
    class _Raw:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
    return torch.as_tensor(_Raw(), device="cuda")


def test_static_router_matches_the_context_router_twice_in_a_row():
    from flashmoe_b200.layer import MoELayer
    import flashmoe_b200 as flashmoe
    w = GOLDEN_CASES["bf16_two_mtiles"]
    lw = make_weights(w)
    layer = MoELayer(w, lw, return_logits=True)
    lib = N.lib()
    try:
        S, E, k = w.tokens_per_rank, w.num_experts, w.top_k
        g = layer.geometry()
        table = torch.zeros(E * g.round_ec * 2, dtype=torch.int32, device="cuda")
        routes = torch.zeros(S * k * 4, dtype=torch.int32, device="cuda")
        counts = torch.zeros(E, dtype=torch.int32, device="cuda")
        probs = torch.zeros(S, E, dtype=torch.float32, device="cuda")
        desc = flashmoe._model_desc(layer.args)
        sp = layer.stream.cuda_stream
        for call in range(2):
            x = make_tokens(w.scaled(seed=w.seed + call))
            layer.tokens.copy_(x)
            torch.cuda.synchronize()
            # existing entry point (scratch in the router context it allocated)
            layer.route()
            layer.stream.synchronize()
            want_counts = layer.counts.clone()
            want_probs = layer.routing.clone()
            want_routes = layer.debug(4, torch.int32, (S * k * 4,))
            want_table = _raw(layer.handle.mod.get_tIdx(layer.handle.context), E * g.round_ec * 8).clone()
            # new entry point: caller-owned outputs, scratch inside the library, no context
            args = N.RouterArgsC(layer.tokens.data_ptr(), layer.router_w.data_ptr(), probs.data_ptr(),
                                 counts.data_ptr(),
                                 layer.logit_bias.data_ptr() if layer.logit_bias is not None else None)
            # the one property this entry point exists for: the device's free memory is the same
            # before and after (the first call only looks up the address of the library's array)
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
            rc = lib.fmoe_router_forward_static(C.byref(desc), 0, C.byref(args), C.c_void_p(table.data_ptr()),
                                                g.round_ec, C.c_void_p(routes.data_ptr()), C.c_void_p(sp))
            assert rc == 0, lib.fmoe_last_error().decode()
            layer.stream.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, f"call {call}: {free_before - free_after} bytes of device memory taken"
            # integer and bit-level equality (the tolerance of every router test in this suite)
            assert torch.equal(counts, want_counts), f"call {call}: counts"
            assert torch.equal(probs.view(torch.int32), want_probs.view(torch.int32)), f"call {call}: probs"
            assert torch.equal(routes, want_routes), f"call {call}: routes"
            got_table = table.view(torch.uint8)
            n_e = counts.cpu().numpy()
            gt = got_table.view(torch.int32).reshape(E, g.round_ec, 2).cpu().numpy()
            wt = want_table.view(torch.int32).reshape(E, g.round_ec, 2).cpu().numpy()
            for e in range(E):
                n = min(int(n_e[e]), w.expert_peer_capacity)
                assert np.array_equal(gt[e, :n], wt[e, :n]), f"call {call}: table row {e}"
    finally:
        layer.close()


def test_static_router_checks_alignment_and_leaves_the_current_device_alone():
    """An offset pointer is refused on the host (a misaligned store would fault the GPU), and the
    calling thread's current device is what it was, also when the call names another device."""
    lib = N.lib()
    desc = N.ModelDesc(64, 64, 64, 8, 2, 64, 0, 0, 1, 1000)
    buf = torch.zeros(4096, dtype=torch.int32, device="cuda")
    base = buf.data_ptr()
    ok = N.RouterArgsC(base, base, None, base, None)
    assert lib.fmoe_router_forward_static(C.byref(desc), 0, C.byref(ok), C.c_void_p(base + 4), 128,
                                          C.c_void_p(base), None) == 1
    assert b"token_table" in lib.fmoe_last_error()
    odd = N.RouterArgsC(base, base, None, base + 2, None)
    assert lib.fmoe_router_forward_static(C.byref(desc), 0, C.byref(odd), C.c_void_p(base), 128,
                                          C.c_void_p(base), None) == 1
    if torch.cuda.device_count() > 1:
        # tokens on device 1, the caller's thread on device 0
        with torch.cuda.device(1):
            far = torch.zeros(1 << 16, dtype=torch.int32, device="cuda")
        torch.cuda.set_device(0)
        p1 = far.data_ptr()
        a1 = N.RouterArgsC(p1, p1 + 8192, None, p1 + 16384, None)
        assert lib.fmoe_router_forward_static(C.byref(desc), 1, C.byref(a1), C.c_void_p(p1 + 32768), 128,
                                              C.c_void_p(p1 + 65536), None) == 0, lib.fmoe_last_error().decode()
        torch.cuda.synchronize(1)
        assert torch.cuda.current_device() == 0


def test_static_router_rejects_oversized_layers():
    import flashmoe_b200 as flashmoe
    lib = N.lib()
    desc = N.ModelDesc(32768, 64, 64, 8, 8, 32768, 0, 0, 1, 1000)   # 262144 pairs > 131072
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    args = N.RouterArgsC(dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), None)
    rc = lib.fmoe_router_forward_static(C.byref(desc), 0, C.byref(args), C.c_void_p(dummy.data_ptr()), 32768,
                                        C.c_void_p(dummy.data_ptr()), None)
    assert rc == 2
    assert b"131072" in lib.fmoe_last_error()
