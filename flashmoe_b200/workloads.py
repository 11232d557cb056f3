"""Seeded synthetic workloads at the shapes the benchmarks and parity tests name.

Everything is drawn on the CPU from `torch.Generator().manual_seed(...)` in fp32 and then
cast, so that every device and every checker sees identical bits.  Weights come from
`seed` on every rank (the reference's test broadcasts its weight seeds,
csrc/tests/flashmoe.cu:435-471); a rank's tokens come from `seed * 1000 + rank`.

Storage layouts are the reference's (B operands are [N, K] row-major,
csrc/include/flashmoe/tile.cuh:344-346; quickstart.py:231-235):
router weight [E, H]; up / up_v [E, I, H]; down [E, H, I]; biases [E, I], [E, I], [E, H].
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from math import ceil, log
from typing import Optional

import torch

from .jit import ActivationType, DataType, MLPType

TORCH_DTYPE = {DataType.BF16: torch.bfloat16, DataType.FP16: torch.float16,
               DataType.FP32: torch.float32}


@dataclass(frozen=True)
class Workload:
    name: str
    tokens_per_rank: int
    token_dim: int
    ffn_size: int
    num_experts: int
    top_k: int
    data_type: DataType = DataType.BF16
    mlp_type: MLPType = MLPType.GATED
    act_type: ActivationType = ActivationType.SILU
    seed: int = 1234
    zipf_bias: bool = False          # per-expert logit bias 1.5*log(Zipf(s=1.2) rank pmf)
    bias_std: float = 0.0            # expert biases; 0 = zero biases
    capacity: Optional[int] = None   # None = tokens_per_rank (no token is dropped)

    @property
    def expert_peer_capacity(self) -> int:
        return self.tokens_per_rank if self.capacity is None else self.capacity

    @property
    def reference_default_capacity(self) -> int:
        # flashmoe/jit.py:148-151
        return ceil(float(self.tokens_per_rank) / self.num_experts) * self.top_k

    def scaled(self, **kw) -> "Workload":
        return replace(self, **kw)


# The five configurations of the benchmark description, in its order.
CONFIGS = {
    "cpu_ref_fp32": Workload("cpu_ref_fp32", 128, 1024, 2048, 8, 2, DataType.FP32),
    "scout": Workload("scout", 1024, 5120, 8192, 16, 1),
    "mixtral": Workload("mixtral", 4096, 4096, 14336, 8, 2),
    "deepseek_v3": Workload("deepseek_v3", 2048, 7168, 2048, 256, 8, zipf_bias=True),
    "qwen3": Workload("qwen3", 1024, 2048, 768, 128, 8),
    "qwen3_fp32_gelu": Workload("qwen3_fp32_gelu", 1024, 2048, 768, 128, 8, DataType.FP32,
                                MLPType.VANILLA, ActivationType.GELU),
}
QWEN3_SWEEP = (1, 16, 128, 1024, 8192)


@dataclass
class LayerWeights:
    router: torch.Tensor                 # [E, H]
    up: torch.Tensor                     # [E, I, H]  (activated branch, "W_gate")
    up_v: Optional[torch.Tensor]         # [E, I, H]  (linear branch, "W_up"); None if vanilla
    down: torch.Tensor                   # [E, H, I]
    bias_up: torch.Tensor                # [E, I]
    bias_up_v: Optional[torch.Tensor]    # [E, I]
    bias_down: torch.Tensor              # [E, H]
    logit_bias: Optional[torch.Tensor]   # [E] fp32 or None


def _normal(gen: torch.Generator, shape, std: float, dtype: torch.dtype) -> torch.Tensor:
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(dtype)


def make_weights(w: Workload, experts: Optional[range] = None) -> LayerWeights:
    """All E experts (or the slice `experts`) of the layer; identical on every rank.

    Each expert's tensors come from their own generator seeded by (seed, expert) so that a
    rank can materialise just its slice and still agree with a checker holding all of them.
    """
    dt = TORCH_DTYPE[w.data_type]
    E, H, I = w.num_experts, w.token_dim, w.ffn_size
    g = torch.Generator().manual_seed(w.seed)
    router = _normal(g, (E, H), (1.0 / H) ** 0.5, dt)
    ids = list(range(E) if experts is None else experts)
    gated = w.mlp_type == MLPType.GATED
    up, up_v, down, b_up, b_up_v, b_down = [], [], [], [], [], []
    for e in ids:
        ge = torch.Generator().manual_seed(w.seed * 7919 + 17 * e + 1)
        # drawn as [H, I] / [I, H] (the model's orientation) then stored transposed
        up.append(_normal(ge, (H, I), 0.02, dt).t().contiguous())
        v = _normal(ge, (H, I), 0.02, dt).t().contiguous()
        if gated:
            up_v.append(v)
        down.append(_normal(ge, (I, H), 0.02, dt).t().contiguous())
        b_up.append(_normal(ge, (I,), w.bias_std, dt))
        bv = _normal(ge, (I,), w.bias_std, dt)
        if gated:
            b_up_v.append(bv)
        b_down.append(_normal(ge, (H,), w.bias_std, dt))
    logit_bias = None
    if w.zipf_bias:
        perm = torch.randperm(E, generator=torch.Generator().manual_seed(w.seed + 99))
        pmf = torch.tensor([(1.0 + int(perm[e])) ** -1.2 for e in range(E)], dtype=torch.float64)
        pmf = pmf / pmf.sum()
        logit_bias = (1.5 * pmf.log()).float()
    return LayerWeights(router, torch.stack(up), torch.stack(up_v) if gated else None,
                        torch.stack(down), torch.stack(b_up),
                        torch.stack(b_up_v) if gated else None, torch.stack(b_down), logit_bias)


def make_tokens(w: Workload, rank: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(w.seed * 1000 + rank)
    return _normal(g, (w.tokens_per_rank, w.token_dim), 1.0, TORCH_DTYPE[w.data_type])


def flops_per_rank(w: Workload, routed_pairs: int) -> float:
    """Algorithmic work of one rank's forward: c*H*I per routed (token, expert) pair executed
    there (c = 6 gated, 4 plain) plus the router's 2*S*H*E.  No padding, no dropped tokens."""
    c = 6 if w.mlp_type == MLPType.GATED else 4
    return float(routed_pairs) * c * w.token_dim * w.ffn_size + \
        2.0 * w.tokens_per_rank * w.token_dim * w.num_experts


def weight_bytes_per_rank(w: Workload, local_experts: int) -> float:
    eb = 4 if w.data_type == DataType.FP32 else 2
    c = 3 if w.mlp_type == MLPType.GATED else 2
    return float(local_experts) * c * w.token_dim * w.ffn_size * eb
