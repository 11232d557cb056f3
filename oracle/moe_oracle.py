"""CPU restatement of the FlashMoE MoE-layer forward (router + experts + combine).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is the
checker for the CUDA path (tests, the smoke check and the bench's CPU-baseline leg).

PARITY UNPINNED: the reference holds no golden vectors or known-answer tests for this
path (all of its tests draw unseeded inputs and compare two GPU pipelines run side by
side), and none of its code can execute without a GPU, cuBLASDx and NVSHMEM.  This file
therefore restates the reference's algorithm from its sources and is cross-checked
against an independent float64 evaluation plus the structural invariants the
reference's own tests assert (each token appears exactly k times, at most once per
expert; the counts sum to S*k).

What follows what (paths inside the reference project):

* router semantics      csrc/include/flashmoe/gate.cuh:395-565 (single-block main loop:
                        fp32 logits, fp32 softmax over all E, k rounds of arg-max on the
                        probabilities with strict '>' so ties go to the lowest expert id,
                        combine weight p / sum(selected p), counts not clamped, a routing
                        table entry only when slot < EC)
* routing table layout  csrc/include/flashmoe/infra/packed.cuh:8-11 (TPS = {u32 token,
                        f32 probability}), [E, roundEC] row-major
* expert MLP            flashmoe/bindings.py:346-422 (tile epilogue = rounding points),
                        csrc/include/flashmoe/processor.cuh:97-136
* per-expert pipeline   flashmoe/bindings.py:560-626 (clamp min(count, EC), zero-init out)
* combine               flashmoe/bindings.py:464-501
* activations           csrc/include/flashmoe/infra/activation.cuh:30-49

Two things are pinned down here that the reference leaves open, so that integer
results (expert ids, counts, slots) can be compared bit for bit:

1. The fp32 summation order of the logits and of the softmax denominator, and the
   exp() used by the softmax, are spelled out operation by operation (see
   `router_logits` and `det_exp`).  The CUDA router performs exactly the same fp32
   operations in exactly the same order, so its probabilities are bit-identical.
2. Slots inside an expert's routing-table row are handed out in ascending token order.
   The reference yields that order whenever S <= its tile height and an arbitrary
   arrival order otherwise (atomicAdd between tiles, gate.cuh:365).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

# enum values follow flashmoe/jit.py:22-40
GATED, VANILLA = 0, 1
BF16, FP16, FP32, FP64 = 0, 1, 2, 3
IDENTITY, SILU, GELU, RELU = 0, 1, 2, 3

TORCH_DTYPE = {BF16: torch.bfloat16, FP16: torch.float16, FP32: torch.float32}

_F = np.float32
LANES = 32     # partial sums per dot product
VEC = 8        # consecutive elements a partial sum consumes per step

# 2^f on [-0.5, 0.5] as a degree-7 Taylor polynomial in f*ln2, coefficients (ln2)^k/k!
# rounded to fp32 once, here, and spelled as hex floats in the CUDA source.
EXP2_COEF = [_F(float.fromhex(c)) for c in (
    "0x1.0p+0", "0x1.62e43p-1", "0x1.ebfbep-3", "0x1.c6b08ep-5",
    "0x1.3b2ab6p-7", "0x1.5d87fep-10", "0x1.430912p-13", "0x1.ffcbfcp-17",
)]
LOG2E = _F(float.fromhex("0x1.715476p+0"))
EXP_CLAMP = _F(-100.0)


def det_exp(x: np.ndarray) -> np.ndarray:
    """exp(x) for x <= 0, as a fixed sequence of fp32 multiplies and adds (no FMA).

    t = max(x*log2(e), -100); n = rint(t); f = t - n; Horner on EXP2_COEF; times 2^n.
    """
    x = np.asarray(x, dtype=_F)
    t = np.maximum(x * LOG2E, EXP_CLAMP).astype(_F)
    n = np.rint(t).astype(_F)
    f = (t - n).astype(_F)
    p = np.full_like(f, EXP2_COEF[7])
    for c in EXP2_COEF[6::-1]:
        p = (p * f).astype(_F)
        p = (p + c).astype(_F)
    scale = np.ldexp(_F(1.0), n.astype(np.int32)).astype(_F)
    return (p * scale).astype(_F)


def _butterfly(acc: np.ndarray) -> np.ndarray:
    """xor-butterfly over the last axis (length 32): offsets 16, 8, 4, 2, 1."""
    idx = np.arange(LANES)
    for off in (16, 8, 4, 2, 1):
        acc = (acc + acc[..., idx ^ off]).astype(_F)
    return acc[..., 0]


def router_logits(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """logits[s, e] = sum_h x[s, h] * w[e, h] in the router's fixed fp32 order.

    x: [S, H] fp32 (already holding Element-rounded values), w: [E, H] fp32.
    The H axis is cut into vectors of 8 elements; vector v belongs to partial sum
    (v mod 32); a partial sum consumes its vectors in ascending v and, inside a vector,
    ascending h, each step being acc = acc + x*w with the product rounded to fp32 first
    (exact for 16-bit inputs, so equal to an FMA there).  The 32 partial sums are then
    folded by an xor-butterfly with offsets 16, 8, 4, 2, 1.
    """
    x = np.ascontiguousarray(x, dtype=_F)
    w = np.ascontiguousarray(w, dtype=_F)
    S, H = x.shape
    E = w.shape[0]
    assert H % VEC == 0
    nvec = H // VEC
    iters = -(-nvec // LANES)
    pad = iters * LANES * VEC - H
    if pad:
        x = np.concatenate([x, np.zeros((S, pad), _F)], axis=1)
        w = np.concatenate([w, np.zeros((E, pad), _F)], axis=1)
    xv = x.reshape(S, iters, LANES, VEC)
    wv = w.reshape(E, iters, LANES, VEC)
    acc = np.zeros((S, E, LANES), _F)
    for it in range(iters):
        for j in range(VEC):
            prod = (xv[:, None, it, :, j] * wv[None, :, it, :, j]).astype(_F)
            acc = (acc + prod).astype(_F)
    return _butterfly(acc)


def router_softmax(logits: np.ndarray) -> np.ndarray:
    """Row softmax in fp32: p = det_exp(x - max) / d, d summed lane-interleaved.

    Element j belongs to partial sum (j mod 32); partial sums run over ascending j and
    are folded by the same butterfly as the logits; the division is IEEE fp32.
    """
    logits = np.asarray(logits, dtype=_F)
    S, E = logits.shape
    m = logits.max(axis=1, keepdims=True)
    e = det_exp((logits - m).astype(_F))
    groups = -(-E // LANES)
    pad = groups * LANES - E
    ep = np.concatenate([e, np.zeros((S, pad), _F)], axis=1) if pad else e
    ep = ep.reshape(S, groups, LANES)
    acc = np.zeros((S, LANES), _F)
    for g in range(groups):
        acc = (acc + ep[:, g, :]).astype(_F)
    d = _butterfly(acc)
    return (e / d[:, None]).astype(_F)


@dataclass
class Routing:
    probs: np.ndarray          # [S, E] fp32 softmax
    topk_idx: np.ndarray       # [S, k] int32, selection order (descending probability)
    topk_w: np.ndarray         # [S, k] fp32 combine weights p / sum(selected p)
    topk_slot: np.ndarray      # [S, k] int32 slot inside the expert's row (may be >= EC)
    counts: np.ndarray         # [E] int32, not clamped
    table_tok: np.ndarray      # [E, round_ec] uint32 (entries >= min(count, EC) undefined -> 0)
    table_w: np.ndarray        # [E, round_ec] fp32


def route(x: np.ndarray, w: np.ndarray, k: int, ec: int, round_ec: Optional[int] = None,
          logit_bias: Optional[np.ndarray] = None) -> Routing:
    """Full router: logits -> softmax -> top-k -> slot assignment (gate.cuh:395-565)."""
    logits = router_logits(x, w)
    if logit_bias is not None:
        logits = (logits + np.asarray(logit_bias, _F)[None, :]).astype(_F)
    return route_from_logits(logits, k, ec, round_ec)


def route_from_logits(logits: np.ndarray, k: int, ec: int,
                      round_ec: Optional[int] = None) -> Routing:
    S, E = logits.shape
    if round_ec is None:
        round_ec = -(-ec // 128) * 128
    p = router_softmax(logits)
    masked = p.copy()
    topk_idx = np.zeros((S, k), np.int32)
    topk_p = np.zeros((S, k), _F)
    rows = np.arange(S)
    wsum = np.zeros(S, _F)
    for j in range(k):
        # np.argmax returns the first maximum: strict '>' scan, lowest index wins ties
        sel = np.argmax(masked, axis=1)
        topk_idx[:, j] = sel
        topk_p[:, j] = p[rows, sel]
        wsum = (wsum + topk_p[:, j]).astype(_F)
        masked[rows, sel] = -np.inf
    topk_w = (topk_p / wsum[:, None]).astype(_F)

    counts = np.zeros(E, np.int32)
    topk_slot = np.zeros((S, k), np.int32)
    table_tok = np.zeros((E, round_ec), np.uint32)
    table_w = np.zeros((E, round_ec), _F)
    for e in range(E):
        t_idx, j_idx = np.nonzero(topk_idx == e)      # row-major => ascending token order
        counts[e] = len(t_idx)
        slots = np.arange(len(t_idx), dtype=np.int32)
        topk_slot[t_idx, j_idx] = slots
        keep = slots < ec
        table_tok[e, slots[keep]] = t_idx[keep]
        table_w[e, slots[keep]] = topk_w[t_idx[keep], j_idx[keep]]
    return Routing(p, topk_idx, topk_w, topk_slot, counts, table_tok, table_w)


def activation(x: torch.Tensor, act: int) -> torch.Tensor:
    """fp32 activations (infra/activation.cuh:30-49; CUTLASS functors)."""
    if act == SILU:
        return x * torch.sigmoid(x)
    if act == GELU:
        return 0.5 * x * (1.0 + torch.erf(x * 0.7071067811865476))
    if act == RELU:
        return torch.relu(x)
    return x


@dataclass
class ExpertWeights:
    """Storage layout of the reference (B operand is [N, K] row-major, tile.cuh:344-346):
    up / up_v: [E, I, H]; down: [E, H, I]; biases [E, I], [E, I], [E, H]; all Element."""
    up: torch.Tensor
    up_v: Optional[torch.Tensor]
    down: torch.Tensor
    bias_up: torch.Tensor
    bias_up_v: Optional[torch.Tensor]
    bias_down: torch.Tensor


def expert_mlp(xe: torch.Tensor, wts: ExpertWeights, e: int, mlp: int, act: int,
               alpha: float = 1.0, beta: float = 1.0):
    """One expert on its gathered rows; rounding points follow bindings.py:373-401.

    gated:   g = (x Wu^T + b) * beta;  t = Element(alpha * act(g));
             v = x Wv^T + bv;          y = Element(v * float(t))
    vanilla: y = Element(act(x Wu^T + b))
    then     o = Element(y Wd^T + bd)
    Returns (y, o).
    """
    dt = xe.dtype
    xf = xe.float()
    g = xf @ wts.up[e].float().T + wts.bias_up[e].float()
    if mlp == GATED:
        t = (alpha * activation(g * beta, act)).to(dt)
        v = xf @ wts.up_v[e].float().T + wts.bias_up_v[e].float()
        y = (v * t.float()).to(dt)
    else:
        y = activation(g, act).to(dt)
    o = (y.float() @ wts.down[e].float().T + wts.bias_down[e].float()).to(dt)
    return y, o


def moe_forward(tokens: torch.Tensor, r: Routing, wts: ExpertWeights, k: int, ec: int,
                mlp: int = GATED, act: int = SILU, alpha: float = 1.0, beta: float = 1.0,
                combine: str = "fp32", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Experts + combine for one rank's tokens against ALL experts (bindings.py:560-626).

    combine="fp32" (oracle of record): for k > 1 the k weighted rows of a token are summed
    in fp32 in selection order and rounded to Element once.  combine="element" follows
    the reference's arithmetic literally: out = Element(v * w) + out in Element, experts
    ascending (bindings.py:487-498).  For k == 1 rows are copied unscaled and rows of
    dropped tokens keep whatever `out` held (zero when `out` is None).
    """
    S, H = tokens.shape
    dt = tokens.dtype
    E = r.counts.shape[0]
    if out is None:
        out = torch.zeros(S, H, dtype=dt)
    elif k > 1:
        out.zero_()
    acc = torch.zeros(S, H, dtype=torch.float32) if (k > 1 and combine == "fp32") else None
    contrib = {}
    for e in range(E):
        cnt = int(min(r.counts[e], ec))
        if cnt == 0:
            continue
        ids = torch.from_numpy(r.table_tok[e, :cnt].astype(np.int64))
        _, o = expert_mlp(tokens[ids], wts, e, mlp, act, alpha, beta)
        if k == 1:
            out[ids] = o
        elif combine == "element":
            w = torch.from_numpy(r.table_w[e, :cnt])[:, None]
            out[ids] = (o.float() * w).to(dt) + out[ids]
        else:
            contrib[e] = o
    if acc is not None:
        # selection order j = 0..k-1, one fp32 fma-free accumulate per choice
        for j in range(k):
            for e in contrib:
                sel = np.nonzero((r.topk_idx[:, j] == e) & (r.topk_slot[:, j] < ec))[0]
                if len(sel) == 0:
                    continue
                slots = torch.from_numpy(r.topk_slot[sel, j].astype(np.int64))
                w = torch.from_numpy(r.topk_w[sel, j])[:, None]
                acc[torch.from_numpy(sel)] += contrib[e][slots].float() * w
        out.copy_(acc.to(dt))
    return out


def layer_forward(tokens: torch.Tensor, router_w: torch.Tensor, wts: ExpertWeights, k: int,
                  ec: int, mlp: int = GATED, act: int = SILU, alpha: float = 1.0,
                  beta: float = 1.0, logit_bias: Optional[np.ndarray] = None,
                  combine: str = "fp32"):
    """Router + experts + combine for one rank.  Returns (out, Routing)."""
    r = route(tokens.float().numpy(), router_w.float().numpy(), k, ec, logit_bias=logit_bias)
    return moe_forward(tokens, r, wts, k, ec, mlp, act, alpha, beta, combine), r


def dense_f64(tokens: torch.Tensor, r: Routing, wts: ExpertWeights, k: int, ec: int,
              mlp: int, act: int, alpha: float = 1.0, beta: float = 1.0) -> torch.Tensor:
    """Independent float64 evaluation with no intermediate rounding (cross-check only)."""
    S, H = tokens.shape
    out = torch.zeros(S, H, dtype=torch.float64)
    x = tokens.double()
    for t in range(S):
        for j in range(k):
            e = int(r.topk_idx[t, j])
            if r.topk_slot[t, j] >= ec:
                continue
            g = wts.up[e].double() @ x[t] + wts.bias_up[e].double()
            if mlp == GATED:
                y = (wts.up_v[e].double() @ x[t] + wts.bias_up_v[e].double()) * \
                    (alpha * activation(g * beta, act))
            else:
                y = activation(g, act)
            o = wts.down[e].double() @ y + wts.bias_down[e].double()
            out[t] += o if k == 1 else o * float(r.topk_w[t, j])
    return out
