"""Model-description types of the layer's public API, and the in-tree native build.

The names, constructor arguments, defaults and enum values mirror the reference's
flashmoe/jit.py:7-151 so that a script written against `flashmoe` runs against this package
unchanged (`import flashmoe_b200 as flashmoe`).  Where the reference compiles one shared
object per model description at `initialize` time (flashmoe/jit.py:153-296), this package
ships one ahead-of-time library whose kernels take the shapes at run time; `_get_compiled`
therefore only locates (and, if asked, builds) that library.
"""
from __future__ import annotations

import math
from enum import IntEnum
from typing import List, Optional


class Topology(IntEnum):
    NVLINK_ONLY = 0
    MIXED = 1


class MLPType(IntEnum):
    GATED = 0
    VANILLA = 1


class DataType(IntEnum):
    BF16 = 0
    FP16 = 1
    FP32 = 2
    FP64 = 3


class ActivationType(IntEnum):
    IDENTITY = 0
    SILU = 1
    GELU = 2
    RELU = 3


class ContextHandle:
    """Pairs the native module with the opaque context it created (jit.py:7-20)."""
    __slots__ = ("_mod", "_ctx")

    def __init__(self, mod, ctx):
        self._mod, self._ctx = mod, ctx

    @property
    def context(self):
        return self._ctx

    @property
    def mod(self):
        return self._mod


class ForwardArgs:
    """Device addresses (ints) of the contiguous buffers one forward reads and writes.

    tokens [S, H]; expert_counts [E] int32; local_expert_up / local_expert_up_v stored
    [nLx, I, H]; local_expert_down stored [nLx, H, I]; biases [nLx, I], [nLx, I], [nLx, H];
    moe_out [S, H].  `local_expert_up` is the activated branch, `_v` the linear one.
    A gated MLP must supply both `_v` buffers (jit.py:72-73); for a plain MLP they stay None
    and are handed to the library as null.  A null bias address means a zero bias
    (an addition of this package; the reference always reads its biases).
    """

    def __init__(self, mt: MLPType, tokens: int, expert_counts: int, local_expert_up: int,
                 local_bias_up: int, local_expert_down: int, local_bias_down: int, moe_out: int,
                 stream_ptr: int, *, swish_alpha: float = 1.0, swish_beta: float = 1.0,
                 local_expert_up_v: Optional[int] = None, local_bias_up_v: Optional[int] = None):
        if mt == MLPType.GATED:
            assert local_expert_up_v is not None, "a gated MLP needs local_expert_up_v"
            assert local_bias_up_v is not None, "a gated MLP needs local_bias_up_v"
        self.tokens = tokens
        self.expert_counts = expert_counts
        self.local_expert_up = local_expert_up
        self.local_expert_up_v = local_expert_up_v
        self.local_bias_up = local_bias_up
        self.local_bias_up_v = local_bias_up_v
        self.local_expert_down = local_expert_down
        self.local_bias_down = local_bias_down
        self.moe_out = moe_out
        self.swish_alpha = swish_alpha
        self.swish_beta = swish_beta
        self.stream_ptr = stream_ptr


class InitArgs:
    """Description of the layer and of this rank's place in the expert-parallel group.

    `gpu_arch` is the compute capability times 100 (1000 for sm_100), as in the reference
    (quickstart.py:50).  `expert_peer_capacity` defaults to ceil(S / E) * k (jit.py:148-151):
    the most tokens one rank may send to one expert; later ones are dropped.  Pass
    `expert_peer_capacity=tokens_per_rank` to drop nothing.  `initialize` fills the fields
    left at None (ep_world, ep_rank, my_pe, num_local_experts, expert_map, rank_map, topo).
    """
    topo: Topology = Topology.MIXED

    def __init__(self, data_type: DataType, tokens_per_rank: int, token_dim: int, ffn_size: int,
                 num_experts: int, top_k: int, gpu_arch: int, mlp_type: MLPType,
                 act_type: ActivationType, stream_ptr: int, device_id: int, *,
                 ep_world: Optional[int] = None, num_local_experts: Optional[int] = None,
                 ep_rank: Optional[int] = None, my_pe: Optional[int] = None,
                 expert_map: Optional[List[int]] = None, rank_map: Optional[List[int]] = None,
                 expert_peer_capacity: Optional[int] = None) -> None:
        assert gpu_arch >= 700
        self.data_type = data_type
        self.tokens_per_rank = tokens_per_rank
        self.token_dim = token_dim
        self.ffn_size = ffn_size
        self.num_experts = num_experts
        self.top_k = top_k
        self.gpu_arch = gpu_arch
        self.mlp_type = mlp_type
        self.act_type = act_type
        self.stream_ptr = stream_ptr
        self.device_id = device_id
        self.ep_world = ep_world
        self.num_local_experts = num_local_experts
        self.ep_rank = ep_rank
        self.my_pe = my_pe
        self.expert_map = expert_map
        self.rank_map = rank_map
        if expert_peer_capacity is None:
            expert_peer_capacity = math.ceil(float(tokens_per_rank) / num_experts) * top_k
        self.expert_peer_capacity = expert_peer_capacity


def _get_compiled(arg: Optional[InitArgs] = None, src=None, mod_prefix: str = "", mod_name: str = ""):
    """Return the loaded native library (the reference's per-model JIT collapses to this).

    Raises if the library has not been built: there is no fallback implementation.
    """
    from . import _native
    return _native.lib()
