"""flashmoe_b200: the MoE-layer forward of FlashMoE, rebuilt for B200 (sm_100a).

Drop-in for the reference's Python API (`import flashmoe_b200 as flashmoe`):
`initialize(InitArgs) -> ContextHandle`, `forward(handle, ForwardArgs)`,
`finalize(handle, stream_ptr)` (flashmoe/__init__.py:7-104), `router.*`, `cb.*`, and the
description types of flashmoe/jit.py.  Everything below the API is one native library behind
a C ABI (include/flashmoe_b200.h); this module only marshals arguments and, at `initialize`,
swaps CUDA IPC handles between the ranks of the expert-parallel group.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _native as N
from . import cb, reference, router
from .cb import get_local_rank
from .jit import (ActivationType, ContextHandle, DataType, ForwardArgs, InitArgs, MLPType,
                  Topology, _get_compiled, specialised_library)

__all__ = ["initialize", "forward", "finalize", "get_workspace_bytes", "router", "reference", "cb", "get_local_rank", "InitArgs",
           "ForwardArgs", "ContextHandle", "Topology", "MLPType", "ActivationType", "DataType",
           "FlashMoEError"]
FlashMoEError = N.FlashMoEError


def _model_desc(arg: InitArgs) -> N.ModelDesc:
    return N.ModelDesc(arg.tokens_per_rank, arg.token_dim, arg.ffn_size, arg.num_experts, arg.top_k,
                       arg.expert_peer_capacity, int(arg.data_type), int(arg.mlp_type),
                       int(arg.act_type), int(arg.gpu_arch))


class _MoEModule:
    """Stands where the reference's per-model JIT module stands: same four functions with the
    same keyword arguments (flashmoe/bindings.py:154-185)."""

    def __init__(self, lib, desc: N.ModelDesc, topo: int):
        self._lib, self._desc, self._topo = lib, desc, topo

    def initialize(self, num_experts, expert_peer_capacity, ep_world, my_pe, ep_rank, local_rank,
                   num_local_experts, expert_map, rank_map, stream_ptr, memory=None) -> int:
        if len(expert_map) != num_experts:
            raise ValueError("expert_map.size() != num_experts")
        if len(rank_map) != ep_world:
            raise ValueError("rank_map.size() != ep_world")
        emap = (C.c_int32 * num_experts)(*expert_map)
        rmap = (C.c_int32 * ep_world)(*rank_map)
        ep = N.EpDesc(ep_world, ep_rank, my_pe, local_rank, num_local_experts, int(self._topo), emap, rmap)
        ctx = C.c_void_p()
        if memory is None:
            N.check(self._lib.fmoe_ctx_create(C.byref(self._desc), C.byref(ep), C.c_void_p(stream_ptr),
                                              C.byref(ctx)), "initialize")
        else:   # (symmetric address, bytes, workspace address, bytes): the caller's device memory
            N.check(self._lib.fmoe_ctx_create_in(C.byref(self._desc), C.byref(ep), C.c_void_p(stream_ptr),
                                                 C.c_void_p(memory[0]), memory[1], C.c_void_p(memory[2]), memory[3],
                                                 C.byref(ctx)), "initialize")
        if ep_world > 1:
            handle = (C.c_ubyte * N.IPC_HANDLE_BYTES)()
            N.check(self._lib.fmoe_symm_export(ctx, handle), "initialize (export)")
            # peers are addressed by EP rank; rank_map says which process of the job each one is
            for peer, blob in enumerate(cb.exchange_by_rank_map(bytes(handle), ep_rank, list(rank_map))):
                if peer != ep_rank:
                    buf = (C.c_ubyte * N.IPC_HANDLE_BYTES).from_buffer_copy(blob)
                    N.check(self._lib.fmoe_symm_import(ctx, peer, buf), "initialize (import)")
        N.check(self._lib.fmoe_ctx_commit(ctx), "initialize (commit)")
        return ctx.value

    def load_specialised(self, raw_ctx, path) -> None:
        N.check(self._lib.fmoe_ctx_load_specialised(C.c_void_p(raw_ctx), str(path).encode()), "load_specialised")

    def forward(self, raw_ctx, tokens, expert_counts, local_expert_up, local_expert_up_v, local_bias_up,
                local_bias_up_v, local_expert_down, local_bias_down, moe_out, swish_alpha, swish_beta,
                stream_ptr) -> None:
        a = N.ForwardArgsC(tokens, expert_counts, local_expert_up, local_expert_up_v or None,
                           local_bias_up or None, local_bias_up_v or None, local_expert_down,
                           local_bias_down or None, moe_out, swish_alpha, swish_beta)
        N.check(self._lib.fmoe_forward(C.c_void_p(raw_ctx), C.byref(a), C.c_void_p(stream_ptr)), "forward")

    def forward_routed(self, raw_ctx, rargs: "router.RouterForwardArgs", fargs: ForwardArgs) -> None:
        ra = N.RouterArgsC(0, rargs.weights, rargs.routing or None, rargs.expert_counts, rargs.logit_bias or None)
        fa = N.ForwardArgsC(fargs.tokens, fargs.expert_counts, fargs.local_expert_up, fargs.local_expert_up_v or None,
                            fargs.local_bias_up or None, fargs.local_bias_up_v or None, fargs.local_expert_down,
                            fargs.local_bias_down or None, fargs.moe_out, fargs.swish_alpha, fargs.swish_beta)
        N.check(self._lib.fmoe_forward_routed(C.c_void_p(raw_ctx), C.byref(ra), C.byref(fa),
                                              C.c_void_p(fargs.stream_ptr)), "forward (routed)")

    def get_tIdx(self, raw_ctx) -> int:
        out = C.c_void_p()
        N.check(self._lib.fmoe_token_indices(C.c_void_p(raw_ctx), C.byref(out)), "get_tIdx")
        return out.value

    def finalize(self, raw_ctx, stream_ptr) -> None:
        N.check(self._lib.fmoe_ctx_destroy(C.c_void_p(raw_ctx), C.c_void_p(stream_ptr)), "finalize")

    # --- additions of this package -------------------------------------------------------
    def geometry(self, raw_ctx) -> N.Geometry:
        g = N.Geometry()
        N.check(self._lib.fmoe_get_geometry(C.c_void_p(raw_ctx), C.byref(g)), "geometry")
        return g

    def last_status(self, raw_ctx, stream_ptr) -> N.Status:
        s = N.Status()
        self._lib.fmoe_last_status(C.c_void_p(raw_ctx), C.c_void_p(stream_ptr), C.byref(s))
        return s

    def debug_buffer(self, raw_ctx, which: int):
        p, n = C.c_void_p(), C.c_size_t()
        N.check(self._lib.fmoe_debug_buffer(C.c_void_p(raw_ctx), which, C.byref(p), C.byref(n)), "debug_buffer")
        return p.value, n.value

    def forward_host_wait(self, raw_ctx, stream_ptr) -> None:
        N.check(self._lib.fmoe_forward_host_wait(C.c_void_p(raw_ctx), C.c_void_p(stream_ptr)), "forward_host_wait")

    def forward_host(self, raw_ctx, router_ctx, tokens_host, out_host, rargs: "router.RouterForwardArgs",
                     fargs: ForwardArgs, *, wait: bool = True) -> None:
        ra = N.RouterArgsC(0, rargs.weights, rargs.routing or None, rargs.expert_counts,
                           rargs.logit_bias or None)
        fa = N.ForwardArgsC(0, fargs.expert_counts, fargs.local_expert_up, fargs.local_expert_up_v or None,
                            fargs.local_bias_up or None, fargs.local_bias_up_v or None,
                            fargs.local_expert_down, fargs.local_bias_down or None, 0,
                            fargs.swish_alpha, fargs.swish_beta)
        fn = self._lib.fmoe_forward_host if wait else self._lib.fmoe_forward_host_async
        N.check(fn(C.c_void_p(raw_ctx), C.c_void_p(router_ctx), C.c_void_p(tokens_host), C.c_void_p(out_host),
                   C.byref(ra), C.byref(fa), C.c_void_p(fargs.stream_ptr)), "forward_host")


def initialize(arg: InitArgs, memory=None) -> ContextHandle:
    """Create this rank's context (flashmoe/__init__.py:7-77).

    `memory` = (symmetric address, bytes, workspace address, bytes) places the context in device
    memory the caller owns (sizes from `get_workspace_bytes`); by default the library allocates.
    With more than one rank the symmetric part must be a device allocation of its own, not a
    slice of a larger one (a tensor of torch's caching allocator usually is a slice): CUDA IPC
    maps whole allocations, and the export refuses anything else.

    With `ep_rank` unset the group is taken from the communication bootstrap and experts are
    blocked over the ranks (`expert_map[i] = i // num_local_experts`); the fields are written
    back into `arg`, as the reference does.
    """
    assert arg.ep_rank is None or (arg.rank_map is not None and arg.ep_world is not None
                                   and arg.expert_map is not None and arg.num_local_experts is not None
                                   and arg.my_pe is not None), \
        "if rank is set, then so should all dependent metadata"
    cb.initialize()
    if arg.ep_rank is None:
        arg.ep_rank = arg.my_pe = cb.get_rank()
        arg.ep_world = cb.get_world_size()
        assert arg.num_experts % arg.ep_world == 0
        arg.num_local_experts = arg.num_experts // arg.ep_world
        arg.expert_map = [i // arg.num_local_experts for i in range(arg.num_experts)]
        arg.rank_map = list(range(arg.ep_world))
    arg.topo = Topology.NVLINK_ONLY if cb.all_on_one_node() else Topology.MIXED
    lib = _get_compiled(arg)
    mod = _MoEModule(lib, _model_desc(arg), arg.topo)
    ctx = mod.initialize(num_experts=arg.num_experts, expert_peer_capacity=arg.expert_peer_capacity,
                         ep_world=arg.ep_world, my_pe=arg.my_pe, ep_rank=arg.ep_rank,
                         local_rank=arg.device_id, num_local_experts=arg.num_local_experts,
                         expert_map=arg.expert_map, rank_map=arg.rank_map, stream_ptr=arg.stream_ptr,
                         memory=memory)
    # the kernel specialised for this description, when the cache holds it (or FMOE_JIT=1 builds it);
    # FMOE_JIT=off keeps the generic kernel
    if os.environ.get("FMOE_JIT", "0") != "off":
        spec = specialised_library(arg, pair=bool(mod.geometry(ctx).cta_pairs))
        if spec is not None:
            mod.load_specialised(ctx, spec)
    cb.sync_all(arg.stream_ptr)
    return ContextHandle(mod, ctx)


def get_workspace_bytes(arg: InitArgs, ep_world: int = None, num_local_experts: int = None) -> dict:
    """What `initialize(arg)` would allocate on this rank, without allocating or touching a GPU
    (the reference's flashmoe::getWorkspaceBytes, bootstrap.cuh:377-410, is C++ only):
    {"symmetric": bytes of the block every peer maps, "workspace": bytes of the private part}."""
    world = ep_world if ep_world is not None else (arg.ep_world or 1)
    nlx = num_local_experts if num_local_experts is not None else (arg.num_local_experts or arg.num_experts // world)
    ep = N.EpDesc(world, 0, 0, 0, nlx, int(Topology.NVLINK_ONLY), None, None)
    desc = _model_desc(arg)
    symm, work = C.c_int64(), C.c_int64()
    N.check(N.lib().fmoe_workspace_bytes(C.byref(desc), C.byref(ep), C.byref(symm), C.byref(work)),
            "get_workspace_bytes")
    return {"symmetric": symm.value, "workspace": work.value}


def forward(handle: ContextHandle, args: ForwardArgs, router_args: "router.RouterForwardArgs" = None) -> None:
    """One launch of the fused dispatch + experts + combine kernel on `args.stream_ptr`.

    With `router_args` the same launch opens with the router (an addition of this package: no
    `router.forward` call is needed for that step; `router_args.tokens` is ignored)."""
    if router_args is not None:
        handle.mod.forward_routed(handle.context, router_args, args)
        return
    handle.mod.forward(handle.context, tokens=args.tokens, expert_counts=args.expert_counts,
                       local_expert_up=args.local_expert_up, local_expert_up_v=args.local_expert_up_v,
                       local_bias_up=args.local_bias_up, local_bias_up_v=args.local_bias_up_v,
                       local_expert_down=args.local_expert_down, local_bias_down=args.local_bias_down,
                       moe_out=args.moe_out, swish_alpha=args.swish_alpha, swish_beta=args.swish_beta,
                       stream_ptr=args.stream_ptr)


def finalize(handle: ContextHandle, stream_ptr: int) -> None:
    """Barrier, then free the context (flashmoe/__init__.py:94-104)."""
    cb.sync_all(stream_ptr)
    handle.mod.finalize(handle.context, stream_ptr)
