"""Router API: `initialize`, `RouterForwardArgs`, `forward`, `finalize`
(mirrors the reference's flashmoe/router.py:3-45)."""
from __future__ import annotations

import ctypes as C

from . import _native as N
from .jit import ContextHandle, InitArgs, _get_compiled


class _RouterModule:
    """Stands where the reference's JIT-built gate module stands (bindings.py:300-315)."""

    def __init__(self, lib, desc: N.ModelDesc, return_logits: bool):
        self._lib, self._desc, self._return_logits = lib, desc, return_logits

    def initialize(self, device_id: int, stream_ptr: int) -> int:
        ctx = C.c_void_p()
        N.check(self._lib.fmoe_router_create(C.byref(self._desc), device_id, int(self._return_logits),
                                             C.c_void_p(stream_ptr), C.byref(ctx)), "router.initialize")
        return ctx.value

    def forward(self, raw_ctx: int, tokens: int, weights: int, routing: int, expert_counts: int,
                token_indices: int, stream_ptr: int, *, moe_ctx: int, logit_bias: int = 0) -> None:
        args = N.RouterArgsC(tokens, weights, routing or None, expert_counts, logit_bias or None)
        N.check(self._lib.fmoe_router_forward(C.c_void_p(raw_ctx), C.c_void_p(moe_ctx), C.byref(args),
                                              C.c_void_p(stream_ptr)), "router.forward")

    def finalize(self, raw_ctx: int, stream_ptr: int) -> None:
        N.check(self._lib.fmoe_router_destroy(C.c_void_p(raw_ctx), C.c_void_p(stream_ptr)), "router.finalize")


def initialize(arg: InitArgs, return_logits: bool = False) -> ContextHandle:
    from . import _model_desc
    lib = _get_compiled(arg)
    mod = _RouterModule(lib, _model_desc(arg), return_logits)
    return ContextHandle(mod, mod.initialize(device_id=arg.device_id, stream_ptr=arg.stream_ptr))


class RouterForwardArgs:
    """Device addresses: tokens [S, H], weights stored [E, H], expert_counts [E] int32,
    routing [S, E] fp32 (only with return_logits).  `logit_bias` ([E] fp32, added to the logits
    before the softmax) is an addition of this package; 0 = none."""

    def __init__(self, tokens: int, weights: int, expert_counts: int, stream_ptr: int, *,
                 routing: int = 0, logit_bias: int = 0):
        self.tokens = tokens
        self.weights = weights
        self.routing = routing
        self.expert_counts = expert_counts
        self.stream_ptr = stream_ptr
        self.logit_bias = logit_bias


def forward(router_handle: ContextHandle, flash_handle: ContextHandle, arg: RouterForwardArgs) -> None:
    """Fills `expert_counts` and the routing table inside `flash_handle` (router.py:37-44)."""
    router_handle.mod.forward(router_handle.context,
                              tokens=arg.tokens, weights=arg.weights, routing=arg.routing,
                              expert_counts=arg.expert_counts, stream_ptr=arg.stream_ptr,
                              token_indices=flash_handle.mod.get_tIdx(flash_handle.context),
                              moe_ctx=flash_handle.context, logit_bias=arg.logit_bias)


def finalize(handle: ContextHandle, stream_ptr: int) -> None:
    handle.mod.finalize(handle.context, stream_ptr)
