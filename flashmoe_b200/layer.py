"""`MoELayer`: the call sequence of the reference's quickstart (quickstart.py:56-163) as one
object -- device-resident weights, a router context and an MoE context, `forward(tokens)`.

PyTorch is used for what it is good at here: owning device memory and streams.  All compute
goes through the package's public API (`initialize`, `router.forward`, `forward`).
"""
from __future__ import annotations

from typing import Optional

import torch

import flashmoe_b200 as flashmoe
from .workloads import TORCH_DTYPE, LayerWeights, Workload


class MoELayer:
    def __init__(self, w: Workload, weights: LayerWeights, device_id: int = 0, *,
                 stream: Optional[torch.cuda.Stream] = None, return_logits: bool = False,
                 local_experts: Optional[range] = None, memory=None):
        """`weights` holds either all E experts (this rank's slice is taken from it) or, when
        `local_experts` is given, exactly that slice."""
        self.w = w
        self.dev = torch.device("cuda", device_id)
        torch.cuda.set_device(self.dev)
        self.stream = stream or torch.cuda.Stream(device=self.dev)
        sp = self.stream.cuda_stream
        self.args = flashmoe.InitArgs(
            data_type=w.data_type, tokens_per_rank=w.tokens_per_rank, token_dim=w.token_dim,
            ffn_size=w.ffn_size, num_experts=w.num_experts, top_k=w.top_k, gpu_arch=1000,
            mlp_type=w.mlp_type, act_type=w.act_type, stream_ptr=sp, device_id=device_id,
            expert_peer_capacity=w.expert_peer_capacity)
        self.handle = flashmoe.initialize(self.args, memory=memory)
        self.router_handle = flashmoe.router.initialize(self.args, return_logits=return_logits)
        a = self.args
        if local_experts is None:
            mine = [e for e in range(w.num_experts) if a.expert_map[e] == a.ep_rank]
            take = lambda t: None if t is None else t[mine].contiguous().to(self.dev)
        else:
            take = lambda t: None if t is None else t.contiguous().to(self.dev)
        dt = TORCH_DTYPE[w.data_type]
        self.router_w = weights.router.to(self.dev)
        self.up, self.up_v, self.down = take(weights.up), take(weights.up_v), take(weights.down)
        nz = lambda t: t is not None and bool((t != 0).any())
        self.b_up = take(weights.bias_up) if nz(weights.bias_up) else None
        self.b_up_v = take(weights.bias_up_v) if nz(weights.bias_up_v) else None
        self.b_down = take(weights.bias_down) if nz(weights.bias_down) else None
        self.logit_bias = None if weights.logit_bias is None else weights.logit_bias.to(self.dev)
        S, H, E = w.tokens_per_rank, w.token_dim, w.num_experts
        self.counts = torch.zeros(E, dtype=torch.int32, device=self.dev)
        self.routing = torch.zeros(S, E, dtype=torch.float32, device=self.dev) if return_logits else None
        self.tokens = torch.zeros(S, H, dtype=dt, device=self.dev)
        self.out = torch.zeros(S, H, dtype=dt, device=self.dev)
        ptr = lambda t: 0 if t is None else t.data_ptr()
        self.fargs = flashmoe.ForwardArgs(
            mt=w.mlp_type, tokens=self.tokens.data_ptr(), expert_counts=self.counts.data_ptr(),
            local_expert_up=self.up.data_ptr(), local_bias_up=ptr(self.b_up),
            local_expert_down=self.down.data_ptr(), local_bias_down=ptr(self.b_down),
            moe_out=self.out.data_ptr(), stream_ptr=sp,
            local_expert_up_v=ptr(self.up_v) if self.up_v is not None else None,
            local_bias_up_v=ptr(self.b_up_v) if self.up_v is not None else None)
        self.rargs = flashmoe.router.RouterForwardArgs(
            tokens=self.tokens.data_ptr(), weights=self.router_w.data_ptr(),
            expert_counts=self.counts.data_ptr(), stream_ptr=sp, routing=ptr(self.routing),
            logit_bias=ptr(self.logit_bias))
        torch.cuda.synchronize(self.dev)

        self._layers = [dict(router_w=self.router_w, up=self.up, up_v=self.up_v, down=self.down,
                             b_up=self.b_up, b_up_v=self.b_up_v, b_down=self.b_down,
                             logit_bias=self.logit_bias)]
        self._take = take

    # several layers of one model through ONE context: a forward only reads the weights it is
    # handed, and the context keeps the TMA descriptors of every weight set it has seen
    def add_layer(self, weights: LayerWeights) -> int:
        """Device copies of another layer's weights (same shapes); returns its index."""
        take = self._take
        nz = lambda t: t is not None and bool((t != 0).any())
        self._layers.append(dict(
            router_w=weights.router.to(self.dev), up=take(weights.up), up_v=take(weights.up_v),
            down=take(weights.down), b_up=take(weights.bias_up) if nz(weights.bias_up) else None,
            b_up_v=take(weights.bias_up_v) if nz(weights.bias_up_v) else None,
            b_down=take(weights.bias_down) if nz(weights.bias_down) else None,
            logit_bias=None if weights.logit_bias is None else weights.logit_bias.to(self.dev)))
        torch.cuda.synchronize(self.dev)
        return len(self._layers) - 1

    def select_layer(self, index: int) -> None:
        """The next `route` / `experts` / `forward` calls use layer `index`'s weights."""
        L = self._layers[index]
        ptr = lambda t: 0 if t is None else t.data_ptr()
        f, r = self.fargs, self.rargs
        f.local_expert_up, f.local_expert_down = L["up"].data_ptr(), L["down"].data_ptr()
        f.local_bias_up, f.local_bias_down = ptr(L["b_up"]), ptr(L["b_down"])
        if L["up_v"] is not None:
            f.local_expert_up_v, f.local_bias_up_v = L["up_v"].data_ptr(), ptr(L["b_up_v"])
        r.weights, r.logit_bias = L["router_w"].data_ptr(), ptr(L["logit_bias"])

    # the three calls of the hot path, on self.stream
    def route(self) -> None:
        flashmoe.router.forward(self.router_handle, self.handle, self.rargs)

    def experts(self) -> None:
        flashmoe.forward(self.handle, self.fargs)

    def step(self) -> None:
        self.route()
        self.experts()

    def step_one_launch(self) -> None:
        """Router and experts as ONE launch (the router runs as the kernel's first phase)."""
        flashmoe.forward(self.handle, self.fargs, router_args=self.rargs)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [S, H] (any device) -> moe_out [S, H] on this layer's device (a fresh copy)."""
        with torch.cuda.stream(self.stream):
            self.tokens.copy_(tokens, non_blocking=True)
        self.step()
        self.check()
        return self.out.clone()

    def forward_host(self, tokens_host: torch.Tensor, out_host: torch.Tensor, wait: bool = True) -> None:
        """Host buffers in, host buffers out, through the C ABI's fmoe_forward_host (wait=True) or
        its pipelined form fmoe_forward_host_async (wait=False; call host_wait() at the end)."""
        self.handle.mod.forward_host(self.handle.context, self.router_handle.context,
                                     tokens_host.data_ptr(), out_host.data_ptr(), self.rargs, self.fargs,
                                     wait=wait)

    def host_wait(self) -> None:
        self.handle.mod.forward_host_wait(self.handle.context, self.stream.cuda_stream)

    def check(self) -> None:
        st = self.handle.mod.last_status(self.handle.context, self.stream.cuda_stream)
        if st.code != 0:
            raise flashmoe.FlashMoEError(
                st.code, "forward", f"device-side wait ran out: phase {st.phase}, rank {st.rank}, "
                f"cta {st.cta}, detail {st.detail}, epoch {st.epoch}")

    def debug(self, which: int, dtype: torch.dtype, shape) -> torch.Tensor:
        """Copy of an internal buffer (see fmoe_debug_buffer) as a tensor of `dtype`/`shape`."""
        p, n = self.handle.mod.debug_buffer(self.handle.context, which)

        class _Raw:
            __cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (p, False), "version": 2}

        torch.cuda.synchronize(self.dev)
        raw = torch.as_tensor(_Raw(), device=self.dev)
        count = 1
        for d in shape:
            count *= d
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        assert nbytes <= n
        return raw[:nbytes].view(dtype).reshape(shape).clone()

    def phases(self) -> dict:
        """Per-phase times of the LAST forward from the kernel's per-CTA %globaltimer stamps, in
        microseconds: median over CTAs for each phase, the whole kernel (first start to last end),
        and the share of the kernel a median CTA spent in communication it could not overlap:
        the count exchange, the wait of its first task for dispatched rows (tables built -> first
        operand tiles landed) and the wait, after its own last task, for returned rows.  The
        dispatch itself ("dispatch": all counts in -> this CTA's dispatch warps done) runs beside
        the GEMM loop."""
        g = self.geometry()
        t = self.debug(5, torch.int64, (g.grid, 16)).cpu().double()
        d = (t[:, 1:8] - t[:, 0:7]) / 1e3
        med = d.median(dim=0).values
        first = t[:, 8] > 0                      # CTAs that issued MMAs at all
        first_mma = float(((t[first, 8] - t[first, 2]) / 1e3).median()) if bool(first.any()) else 0.0
        # the dispatch warps start as soon as the landing rows are known, while warp 0 still builds
        # the task order: their time is counted from the moment all counts were in
        out = {"count_exchange": float(med[0]), "tables": float(med[1]),
               "dispatch": float(((t[:, 3] - t[:, 1]) / 1e3).median()),
               "first_rows_wait": first_mma,
               "gemm_tickets": float(((t[:, 4] - t[:, 2]) / 1e3).median()),
               "drain_last_task": float(med[4]),
               "wait_returns": float(med[5]), "combine": float(med[6]),
               "kernel": float((t[:, 7].max() - t[:, 0].min()) / 1e3)}
        out["exposed_comm_frac"] = (out["count_exchange"] + out["first_rows_wait"] + out["wait_returns"]) / \
            max(out["kernel"], 1e-9)
        # the last task of a median CTA: accumulator ready -> rows stored -> owners told
        ep = t[:, 9] > 0
        if bool(ep.any()):
            out["last_epilogue"] = [float(((t[ep, 10] - t[ep, 9]) / 1e3).median()),
                                    float(((t[ep, 11] - t[ep, 10]) / 1e3).median())]
        # when the CTAs drew their stop ticket and finished their last task, from the first CTA's
        # start: 10th, 50th, 90th percentile and the last one (the spread is the closing wave)
        t0 = t[:, 0].min()
        for name, col in (("stop_drawn_at", 4), ("last_task_done_at", 5)):
            v = ((t[:, col] - t0) / 1e3).sort().values
            n = len(v)
            out[name] = [float(v[n // 10]), float(v[n // 2]), float(v[(9 * n) // 10]), float(v[-1])]
        return out

    def geometry(self):
        return self.handle.mod.geometry(self.handle.context)

    def close(self) -> None:
        sp = self.stream.cuda_stream
        flashmoe.router.finalize(self.router_handle, sp)
        flashmoe.finalize(self.handle, sp)
