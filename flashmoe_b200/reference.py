"""`flashmoe.reference`: the checker a caller runs BESIDE the fused forward, as the reference's
quickstart does (quickstart.py:70,137-160): `initialize`, `RefForwardArgs`, `forward`, same names
and arguments as flashmoe/reference.py:3-80.

It is NOT on the product path and nothing in `forward` / `router.forward` uses it.  Like the
reference's own checker (flashmoe/bindings.py:560-626) it is a slow, unfused, independent
pipeline: for every expert in ascending order gather its rows from the routing table, GEMM0 with
the gate epilogue, GEMM1, then the combine in Element arithmetic (bindings.py:464-501), with the
rounding points of the tile epilogue (bindings.py:346-422).  The dense products go through torch
(cuBLAS, fp32 accumulation from the Element inputs), one expert's weights at a time, on the
caller's stream.  It reads the routing table and `expert_counts` the fused path's router wrote
(the reference's checker never re-derives the routing either, quickstart.py:155).
"""
from __future__ import annotations

import math

from .jit import ActivationType, ContextHandle, DataType, ForwardArgs, InitArgs, MLPType


class RefForwardArgs:
    """Device addresses (flashmoe/reference.py:28-61): ALL experts' weights -- expert_up /
    expert_up_v [E, I, H], expert_down [E, H, I], biases [E, I], [E, I], [E, H] (0 = no bias) --
    and three work buffers of at least roundEC rows: ref_input [*, H], ref_interim0 [*, I],
    ref_interim1 [*, H]; ref_out [S, H]."""

    def __init__(self, expert_up: int, expert_down: int, bias_up: int, bias_down: int, ref_input: int,
                 ref_interim0: int, ref_interim1: int, ref_out: int, *, expert_up_v: int,
                 bias_up_v: int):
        self.ref_input = ref_input
        self.ref_interim0 = ref_interim0
        self.ref_interim1 = ref_interim1
        self.ref_out = ref_out
        self.expert_up_v = expert_up_v
        self.bias_up = bias_up
        self.bias_down = bias_down
        self.bias_up_v = bias_up_v
        self.expert_up = expert_up
        self.expert_down = expert_down


class _Raw:
    """A device address as something torch can wrap without copying."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": None}


class _ReferenceModule:
    """Stands where the reference's JIT-built checker module stands (bindings.py:628-648)."""

    def __init__(self, arg: InitArgs):
        self.S, self.H, self.I, self.E = arg.tokens_per_rank, arg.token_dim, arg.ffn_size, arg.num_experts
        self.k, self.EC = arg.top_k, arg.expert_peer_capacity
        self.round_ec = -(-self.EC // 128) * 128          # row stride of the routing table
        self.dt, self.gated, self.act = DataType(arg.data_type), arg.mlp_type == MLPType.GATED, arg.act_type
        self.device_id = None

    def initialize(self, device_id: int) -> None:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("flashmoe.reference needs a CUDA device (it has no CPU path)")
        self.device_id = device_id

    def _wrap(self, ptr: int, shape, kind: str):
        import torch
        dev = torch.device("cuda", self.device_id)
        if kind == "i32":
            return torch.as_tensor(_Raw(ptr, shape, "<i4"), device=dev)
        if self.dt == DataType.FP32:
            return torch.as_tensor(_Raw(ptr, shape, "<f4"), device=dev)
        if self.dt == DataType.FP16:
            return torch.as_tensor(_Raw(ptr, shape, "<f2"), device=dev)
        return torch.as_tensor(_Raw(ptr, shape, "<i2"), device=dev).view(torch.bfloat16)

    def _activate(self, x):
        import torch
        if self.act == ActivationType.SILU:
            return x * torch.sigmoid(x)
        if self.act == ActivationType.GELU:
            return 0.5 * x * (1.0 + torch.erf(x * (1.0 / math.sqrt(2.0))))
        if self.act == ActivationType.RELU:
            return torch.relu(x)
        return x

    def forward(self, token_ids: int, tokens: int, ref_input: int, expert_up: int, expert_up_v: int,
                expert_down: int, bias_up: int, bias_up_v: int, bias_down: int, ref_interim0: int,
                ref_interim1: int, expert_counts: int, ref_out: int, swish_alpha: float = 1.0,
                swish_beta: float = 1.0, stream_ptr: int = 0) -> None:
        import torch
        if self.device_id is None:
            raise RuntimeError("reference.initialize was not called")
        S, H, I, E, k, EC, R = self.S, self.H, self.I, self.E, self.k, self.EC, self.round_ec
        eb = 4 if self.dt == DataType.FP32 else 2
        tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False      # fp32 layers: full-precision products
        stream = torch.cuda.ExternalStream(stream_ptr, device=torch.device("cuda", self.device_id)) \
            if stream_ptr else torch.cuda.current_stream(self.device_id)
        try:
            with torch.cuda.stream(stream):
                x_all = self._wrap(tokens, (S, H), "el")
                out = self._wrap(ref_out, (S, H), "el")
                out.zero_()                                 # bindings.py:594
                counts = self._wrap(expert_counts, (E,), "i32").cpu()   # synchronises, as bindings.py:596-597
                table = self._wrap(token_ids, (E, R, 2), "i32")        # {u32 token, f32 weight}
                el = out.dtype
                for e in range(E):
                    cnt = min(int(counts[e]), EC)
                    if cnt <= 0:
                        continue
                    tok = table[e, :cnt, 0].long()
                    prob = table[e, :cnt, 1].contiguous().view(torch.float32)
                    x = x_all[tok]
                    self._wrap(ref_input, (cnt, H), "el").copy_(x)
                    xf = x.float()

                    def bias(ptr, n):
                        return self._wrap(ptr + e * n * eb, (n,), "el").float() if ptr else 0.0

                    g = xf @ self._wrap(expert_up + e * I * H * eb, (I, H), "el").float().T + bias(bias_up, I)
                    if self.gated:
                        t = (swish_alpha * self._activate(g * swish_beta)).to(el)
                        v = xf @ self._wrap(expert_up_v + e * I * H * eb, (I, H), "el").float().T + bias(bias_up_v, I)
                        y = (v * t.float()).to(el)
                    else:
                        y = self._activate(g).to(el)
                    self._wrap(ref_interim0, (cnt, I), "el").copy_(y)
                    o = (y.float() @ self._wrap(expert_down + e * H * I * eb, (H, I), "el").float().T
                         + bias(bias_down, H)).to(el)
                    self._wrap(ref_interim1, (cnt, H), "el").copy_(o)
                    if k == 1:
                        out[tok] = o                        # bindings.py:481-485
                    else:                                   # Element arithmetic, bindings.py:487-498
                        out[tok] = (o.float() * prob[:, None]).to(el) + out[tok]
        finally:
            torch.backends.cuda.matmul.allow_tf32 = tf32


def initialize(arg: InitArgs) -> ContextHandle:
    mod = _ReferenceModule(arg)
    mod.initialize(device_id=arg.device_id)
    return ContextHandle(mod, None)


def forward(handle: ContextHandle, token_ids: int, f_args: ForwardArgs, r_args: RefForwardArgs) -> None:
    handle.mod.forward(token_ids=token_ids, tokens=f_args.tokens, ref_input=r_args.ref_input,
                       expert_up=r_args.expert_up, expert_up_v=r_args.expert_up_v or 0,
                       expert_down=r_args.expert_down, bias_up=r_args.bias_up or 0,
                       bias_up_v=r_args.bias_up_v or 0, bias_down=r_args.bias_down or 0,
                       ref_interim0=r_args.ref_interim0, ref_interim1=r_args.ref_interim1,
                       expert_counts=f_args.expert_counts, ref_out=r_args.ref_out,
                       swish_alpha=f_args.swish_alpha, swish_beta=f_args.swish_beta,
                       stream_ptr=f_args.stream_ptr)
