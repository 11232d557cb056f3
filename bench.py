#!/usr/bin/env python
"""Benchmark of the MoE-layer forward (router + dispatch + experts + combine).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload scout]
                    [--impl flashmoe_b200|reference|nccl_unfused]

N > 1 is launched by torchrun (one rank per GPU); experts are sharded over the ranks and every
rank keeps `tokens_per_rank` tokens (weak scaling).  Rank 0 prints ONE JSON line.

A step = one pass of the hot path over one batch of synthetic tokens: the router (2 launches)
and the fused forward (1 launch).  `value` is whole-job tokens/s with the batch resident in
HBM; `e2e` is the same through the C ABI's host-buffer entry point (H2D of the tokens from
pinned memory, router + forward, D2H of the result, every step).  `roofline` describes the
fused forward kernel, timed with CUDA events on its own stream inside the timed loop.
`parity` is an output check made outside the timed region on EVERY rank: spot tokens of the rank
are routed by the CPU oracle, run through the experts they chose on the host (weights fetched
from, or re-drawn for, the experts' owners) and compared with the kernel's rows; two launches
must give the same bits.  A rank that fails makes the run exit non-zero.
`other_workloads` repeats a short measurement + parity check for the other benchmark shapes.

`--impl reference` times the CPU restatement of the reference (the oracle) on the host cores:
the reference itself has no CPU path and needs cuBLASDx + NVSHMEM to build.
`--impl nccl_unfused` times the same layer as the usual unfused pipeline (router, all_to_all of
counts and rows over NCCL, per-expert torch GEMMs, all_to_all back, weighted sum): the GPU-side
baseline that shows what fusing the exchange into the kernel buys.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
CPU_SAMPLE_TOKENS = 256
NVLINK_PEER_COPY_GBS = 770.0      # measured peer copy, per direction per GPU
OTHER_WORKLOADS = (("mixtral", None), ("deepseek_v3", None), ("qwen3", 1), ("qwen3", 16), ("qwen3", 128),
                   ("qwen3", 1024), ("qwen3", 8192), ("qwen3_fp32_gelu", 1024), ("cpu_ref_fp32", None))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


def load_traffic(workload: str, n_gpus: int):
    """DRAM bytes per launch of the fused kernel from a committed ncu capture, or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get(f"{workload}@{n_gpus}")
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms while the timed regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1])); mx.append(float(f[2]))
                for name, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return None
        # samples under load: the upper half of what was seen (idle samples bracket the region)
        hi = sorted(sm)[len(sm) // 2:]
        return {"sm_mhz": statistics.median(hi), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def device_weights(w, dev, experts):
    """Random-init weights drawn ON the device (fast at multi-GB sizes) with the benchmark's
    distributions: router N(0, 1/H), expert matrices N(0, 0.02), zero biases.  Every expert has a
    generator of its own, seeded by (seed, expert id), so any rank can re-draw any expert."""
    import torch
    from flashmoe_b200.workloads import TORCH_DTYPE, LayerWeights
    from flashmoe_b200.jit import MLPType
    dt = TORCH_DTYPE[w.data_type]
    E, H, I = w.num_experts, w.token_dim, w.ffn_size
    g = torch.Generator(device=dev).manual_seed(w.seed)
    router = (torch.randn(E, H, generator=g, device=dev) * (1.0 / H) ** 0.5).to(dt)
    n = len(experts)
    gated = w.mlp_type == MLPType.GATED
    up = torch.empty(n, I, H, dtype=dt, device=dev)
    up_v = torch.empty(n, I, H, dtype=dt, device=dev) if gated else None
    down = torch.empty(n, H, I, dtype=dt, device=dev)
    for i, e in enumerate(experts):   # one matrix at a time keeps the fp32 temporary small
        ge = torch.Generator(device=dev).manual_seed(w.seed * 7919 + 17 * int(e) + 1)
        up[i] = (torch.randn(I, H, generator=ge, device=dev) * 0.02).to(dt)
        if gated:
            up_v[i] = (torch.randn(I, H, generator=ge, device=dev) * 0.02).to(dt)
        down[i] = (torch.randn(H, I, generator=ge, device=dev) * 0.02).to(dt)
    z = lambda *s: torch.zeros(*s, dtype=dt, device=dev)
    logit_bias = None
    if w.zipf_bias:
        from flashmoe_b200.workloads import make_weights
        logit_bias = make_weights(w.scaled(token_dim=64, ffn_size=64)).logit_bias
    return LayerWeights(router, up, up_v, down, z(n, I), z(n, I) if gated else None, z(n, H), logit_bias)


def cpu_sample(w, lw_host, x_host, threads):
    """One pass of the CPU oracle over the first CPU_SAMPLE_TOKENS tokens; returns seconds."""
    import torch
    from oracle import moe_oracle as O
    torch.set_num_threads(threads)
    n = min(CPU_SAMPLE_TOKENS, x_host.shape[0])
    wts = O.ExpertWeights(lw_host.up, lw_host.up_v, lw_host.down, lw_host.bias_up, lw_host.bias_up_v,
                          lw_host.bias_down)
    bias = None if lw_host.logit_bias is None else lw_host.logit_bias.numpy()
    t0 = time.perf_counter()
    O.layer_forward(x_host[:n], lw_host.router, wts, w.top_k, n, int(w.mlp_type), int(w.act_type),
                    logit_bias=bias)
    return time.perf_counter() - t0, n


def to_host(lw):
    import dataclasses
    return dataclasses.replace(lw, **{f.name: (getattr(lw, f.name).cpu() if getattr(lw, f.name) is not None
                                               else None) for f in dataclasses.fields(lw)})


def describe(w, world, capacity_kind):
    """The `config` object: identical for every arm run on the same workload and N."""
    from flashmoe_b200.jit import MLPType
    from flashmoe_b200.workloads import weight_bytes_per_rank
    S, H, I, E, k = w.tokens_per_rank, w.token_dim, w.ffn_size, w.num_experts, w.top_k
    weights_mb = weight_bytes_per_rank(w, E // world) / 1e6
    return {"workload": f"{w.name}: tokens_per_rank={S} H={H} I={I} E={E} k={k} "
                        f"{'gated' if w.mlp_type == MLPType.GATED else 'plain'} {w.act_type.name} "
                        f"{w.data_type.name}, expert_peer_capacity={w.expert_peer_capacity} "
                        f"({'no drop' if capacity_kind == 'nodrop' else 'reference default, drops'})",
            "parallelism": f"ep{world}xdp{world}", "experts_per_gpu": E // world,
            "step": "router (2 launches) + fused dispatch/experts/combine (1 launch)",
            "timing": "the K steps replayed from a CUDA graph (plain launches if capture fails; see timing_used)",
            "l2": (f"no flush: each step streams {weights_mb:.0f} MB of expert weights per GPU, "
                   f"larger than the 126 MB L2") if weights_mb * 1e6 > L2_BYTES else
                  "no flush: the working set fits L2 (decode-sized case)"}


def spot_parity(w, layer, lw, mine, x, dev, n_spot):
    """Output check of this rank, outside any timed region.  `n_spot` tokens, evenly spaced, are
    routed by the CPU oracle (bit-compared with the route records the GPU router left) and pushed
    through the experts they chose on the host; the result is compared with the kernel's rows.
    Weights of experts another rank owns are re-drawn from the owner's seed."""
    import numpy as np
    import torch
    from oracle import moe_oracle as O
    S, k, E = w.tokens_per_rank, w.top_k, w.num_experts
    dt = int(w.data_type)
    tol = 1e-5 if dt == 2 else 2e-2
    layer.tokens.copy_(x)
    with torch.cuda.stream(layer.stream):
        layer.step()
    layer.check()
    first = layer.out.clone()
    with torch.cuda.stream(layer.stream):
        layer.step()
    layer.check()
    deterministic = bool(torch.equal(first.view(torch.uint8), layer.out.view(torch.uint8)))
    out = layer.out.cpu()
    n_spot = min(n_spot, S)
    sel = torch.linspace(0, S - 1, n_spot).round().long().unique()
    bias = None if lw.logit_bias is None else lw.logit_bias.cpu().numpy()
    r = O.route(x[sel].float().numpy(), lw.router.cpu().float().numpy(), k, len(sel), logit_bias=bias)
    routes = layer.debug(4, torch.int32, (S, k, 4)).cpu()[sel]
    routing_exact = bool(np.array_equal(routes[:, :, 0].numpy(), r.topk_idx.astype(np.int32)) and
                         np.array_equal(routes[:, :, 2].numpy().view(np.float32), r.topk_w.astype(np.float32)))
    slots = routes[:, :, 1].numpy()
    cache = {}

    def expert(e):
        if e not in cache:
            if e in mine:
                i = mine.index(e)
                one = (lw.up[i:i + 1], None if lw.up_v is None else lw.up_v[i:i + 1], lw.down[i:i + 1])
            else:
                d = device_weights(w, dev, [e])
                one = (d.up, d.up_v, d.down)
            H, I = w.token_dim, w.ffn_size
            zt = lambda n: torch.zeros(1, n, dtype=lw.up.dtype)
            cache[e] = O.ExpertWeights(one[0].cpu(), None if one[1] is None else one[1].cpu(), one[2].cpu(),
                                       zt(I), None if one[1] is None else zt(I), zt(H))
            if len(cache) > 24:                       # bound the host copies
                cache.pop(next(iter(cache)))
        return cache[e]

    got, want = [], []
    order = sorted(((int(r.topk_idx[i, j]), i, j) for i in range(len(sel)) for j in range(k)))
    partial = {}
    for e, i, j in order:                             # expert by expert, so that each is fetched once
        if slots[i, j] >= w.expert_peer_capacity:
            continue                                  # a dropped pair contributes nothing
        t = int(sel[i])
        _, o = O.expert_mlp(x[t:t + 1], expert(e), 0, int(w.mlp_type), int(w.act_type))
        partial[(i, j)] = o[0].float()
    for i in range(len(sel)):
        rows = [(j, partial[(i, j)]) for j in range(k) if (i, j) in partial]
        if k == 1:
            if not rows:
                continue                              # dropped: the output row is left untouched
            ref = rows[0][1]
        else:
            ref = torch.zeros(w.token_dim)
            for j, o in rows:                         # selection order, fp32, one rounding
                ref = ref + o * float(r.topk_w[i, j])
        want.append(ref.to(out.dtype).double())
        got.append(out[int(sel[i])].double())
    if not got:
        return {"ok": deterministic and routing_exact, "max_rel_err": 0.0, "elementwise_mismatch_frac": 0.0,
                "tokens_checked": 0, "routing_bit_exact": routing_exact, "deterministic": deterministic}
    a, b = torch.stack(got), torch.stack(want)
    err = float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
    rms = float(b.pow(2).mean().sqrt().clamp_min(1e-30))
    frac = float(((a - b).abs() > tol * b.abs() + tol * rms).double().mean())
    finite = bool(torch.isfinite(out.float()).all())
    ok = finite and deterministic and routing_exact and err <= tol and frac <= 1e-4
    return {"ok": ok, "max_rel_err": err, "elementwise_mismatch_frac": frac, "tokens_checked": len(got),
            "routing_bit_exact": routing_exact, "deterministic": deterministic, "tolerance": tol}


def roofline_of(w, world, mine, allc, ms_kernel, peaks, peaks_kind):
    """The fused kernel against the slower of its tensor and HBM bounds.  The launch time is the
    maximum over ranks, so the work is that of the rank with the most routed pairs (with balanced
    routing every rank has about the same; with a skewed router one rank carries the layer)."""
    from flashmoe_b200.jit import DataType, MLPType
    from flashmoe_b200.workloads import weight_bytes_per_rank
    S, H, I = w.tokens_per_rank, w.token_dim, w.ffn_size
    eb = 4 if w.data_type == DataType.FP32 else 2
    cap = w.expert_peer_capacity
    nlx = len(mine)
    per_rank = [sum(min(c[e], cap) for c in allc for e in range(r * nlx, (r + 1) * nlx)) for r in range(world)]
    busiest = max(range(world), key=lambda r: per_rank[r])
    mine = list(range(busiest * nlx, (busiest + 1) * nlx))
    pairs_here = per_rank[busiest]
    active = sum(1 for e in mine if any(c[e] > 0 for c in allc))   # experts whose weights are read
    c_mlp = 6 if w.mlp_type == MLPType.GATED else 4
    flops = float(pairs_here) * c_mlp * H * I
    hbm_bytes = weight_bytes_per_rank(w, active) + 2.0 * S * H * eb
    # fp32 layers run as six BF16 plane products per fp32 product
    tensor_flops = flops * (6 if eb == 4 else 1)
    t_tensor = tensor_flops / (peaks["bf16_tflops_sustained"] * 1e12)
    t_hbm = hbm_bytes / (peaks["hbm_gbs"] * 1e9)
    sec = ms_kernel * 1e-3
    if t_hbm >= t_tensor:
        ach, peak, unit, bound = hbm_bytes / sec / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
    else:
        ach, peak, unit, bound = tensor_flops / sec / 1e12, peaks["bf16_tflops_sustained"], "TFLOP/s", "tensor"
    return {"kernel": "moe_forward_kernel", "bound": bound, "achieved": ach, "peak": peak, "unit": unit,
            "frac": ach / peak, "peak_source": f"of {peaks_kind}",
            "traffic": load_traffic(w.name, world), "ms_per_launch": ms_kernel,
            "algorithmic_flops": flops, "algorithmic_hbm_bytes": hbm_bytes,
            "active_local_experts": active, "routed_pairs": pairs_here, "routed_pairs_per_rank": per_rank,
            "t_tensor_us": t_tensor * 1e6, "t_hbm_us": t_hbm * 1e6,
            "pct_dense_bf16_peak_burst": 100.0 * tensor_flops / sec / (peaks["bf16_tflops"] * 1e12)}


def nvlink_of(w, mine, counts, phases, ms_kernel):
    """Bytes this rank pushed to other GPUs: dispatched rows during the dispatch phase, returned
    rows (the same number come back) spread over the GEMM phase."""
    from flashmoe_b200.jit import DataType
    eb = 4 if w.data_type == DataType.FP32 else 2
    cap = w.expert_peer_capacity
    remote_rows = sum(min(int(counts[e]), cap) for e in range(w.num_experts) if e not in mine)
    out_bytes = float(remote_rows) * w.token_dim * (6 if eb == 4 else 2)   # fp32 rows travel as 3 BF16 planes
    ret_bytes = float(remote_rows) * w.token_dim * eb
    gemm_us = max(phases["gemm_tickets"] + phases["drain_last_task"], 1e-9)
    return {"dispatch_bytes_out": out_bytes, "return_bytes_in": ret_bytes,
            "dispatch_us": phases["dispatch"],
            "dispatch_gbs": out_bytes / max(phases["dispatch"], 1e-9) / 1e3,
            "return_gbs_over_gemm_phase": ret_bytes / gemm_us / 1e3,
            "peak_nominal_gbs": 900.0, "peak_measured_peer_copy_gbs": NVLINK_PEER_COPY_GBS,
            "t_nvlink_us": out_bytes / (NVLINK_PEER_COPY_GBS * 1e3),
            "note": "rank 0, per direction; the dispatch runs on the epilogue warps under the first "
                    "GEMM tickets and also copies the local rows; returned rows are written by the GEMM1 "
                    "epilogues while the GEMM phase runs"}


def short_measure(name, tokens, world, rank, local_rank, dev, dist, peaks, peaks_kind, capacity_kind):
    """A bounded pass over another benchmark shape at the same N: 10 timed steps of plain launches
    (CUDA events per step and per fused launch), the phase stamps, the output check."""
    import torch
    from flashmoe_b200.workloads import CONFIGS, make_tokens
    from flashmoe_b200.layer import MoELayer
    w = CONFIGS[name]
    if tokens:
        w = w.scaled(tokens_per_rank=tokens)
    if capacity_kind == "reference":
        w = w.scaled(capacity=w.reference_default_capacity)
    E = w.num_experts
    if E % world:
        return {"workload": f"{name}@{w.tokens_per_rank}", "skipped": f"E={E} does not divide over {world} ranks"}
    nlx = E // world
    mine = list(range(rank * nlx, (rank + 1) * nlx))
    lw = device_weights(w, dev, mine)
    layer = MoELayer(w, lw, local_rank, local_experts=range(nlx))
    x = make_tokens(w, rank)
    layer.tokens.copy_(x)
    st = layer.stream
    steps = 10

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def mx(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    try:
        with torch.cuda.stream(st):
            for _ in range(3):
                layer.step()
        sync()
        layer.check()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
        with torch.cuda.stream(st):
            for i in range(steps):
                ev[i][0].record(st); layer.route(); ev[i][1].record(st); layer.experts(); ev[i][2].record(st)
        sync()
        layer.check()
        router_us = mx(statistics.mean(e[0].elapsed_time(e[1]) for e in ev) * 1e3)
        fwd_us = mx(statistics.mean(e[1].elapsed_time(e[2]) for e in ev) * 1e3)
        phases = layer.phases()
        counts = layer.counts.cpu().numpy()
        # decode-sized batches: the same step as ONE launch (the router as the kernel's first phase)
        one_launch_us = None
        if w.tokens_per_rank <= 128:
            with torch.cuda.stream(st):
                for _ in range(3):
                    layer.step_one_launch()
            sync()
            o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(st):
                o0.record(st)
                for _ in range(steps):
                    layer.step_one_launch()
                o1.record(st)
            sync()
            layer.check()
            one_launch_us = mx(o0.elapsed_time(o1) / steps * 1e3)
        if world > 1:
            allc = [None] * world
            dist.all_gather_object(allc, counts.tolist())
        else:
            allc = [counts.tolist()]
        roof = roofline_of(w, world, mine, allc, fwd_us / 1e3, peaks, peaks_kind)
        par = spot_parity(w, layer, lw, mine, x, dev, max(4, 16 // w.top_k))
        oks = [par["ok"]]
        if world > 1:
            oks = [None] * world
            dist.all_gather_object(oks, par["ok"])
        res = {"workload": f"{name}@{w.tokens_per_rank}", "dtype": w.data_type.name.lower(),
               "specialised_kernel": bool(layer.geometry().specialised),
               "fwd_us": fwd_us, "router_us": router_us, "step_as_one_launch_us": one_launch_us,
               "tokens_per_s": w.tokens_per_rank * world / ((fwd_us + router_us) * 1e-6),
               "bound": roof["bound"], "frac": roof["frac"],
               "pct_dense_bf16_peak_burst": roof["pct_dense_bf16_peak_burst"],
               "exposed_comm_frac": phases["exposed_comm_frac"],
               "nvlink_gbs": (nvlink_of(w, mine, counts, phases, fwd_us / 1e3)["dispatch_gbs"] if world > 1 else None),
               "parity_max_rel_err": par["max_rel_err"], "parity_mismatch_frac": par["elementwise_mismatch_frac"],
               "parity_ranks_ok": int(sum(bool(o) for o in oks))}
    finally:
        layer.close()
        del layer, lw
        torch.cuda.empty_cache()
    return res


def unfused_arm(a, w, world, rank, local_rank, dev, dist, cfg):
    """The usual unfused expert-parallel pipeline, as the GPU-side baseline: this package's router
    (its route records give every token's experts and weights), then in torch: sort the (token,
    choice) pairs by expert, all_to_all_single of the per-expert counts and of the rows over NCCL,
    one GEMM chain per local expert, all_to_all_single back, weighted sum.  Split sizes travel
    through the host every step, as such pipelines do."""
    import torch
    import torch.nn.functional as F
    from flashmoe_b200.jit import ActivationType, MLPType
    from flashmoe_b200.layer import MoELayer
    from flashmoe_b200.workloads import make_tokens
    S, H, E, k = w.tokens_per_rank, w.token_dim, w.num_experts, w.top_k
    nlx = E // world
    mine = list(range(rank * nlx, (rank + 1) * nlx))
    lw = device_weights(w, dev, mine)
    layer = MoELayer(w, lw, local_rank, local_experts=range(nlx))   # for its router and route records
    x = make_tokens(w, rank).to(dev)
    layer.tokens.copy_(x)
    routes_ptr, routes_bytes = layer.handle.mod.debug_buffer(layer.handle.context, 4)

    class _Raw:
        __cuda_array_interface__ = {"shape": (S, k, 4), "typestr": "<i4", "data": (routes_ptr, False), "version": 2}
    routes = torch.as_tensor(_Raw(), device=dev)
    gated = w.mlp_type == MLPType.GATED
    act = {ActivationType.SILU: F.silu, ActivationType.GELU: F.gelu, ActivationType.RELU: F.relu,
           ActivationType.IDENTITY: (lambda t: t)}[w.act_type]
    cap = w.expert_peer_capacity

    def step():
        with torch.cuda.stream(layer.stream):
            layer.route()
        layer.stream.synchronize()
        e_id = routes[:, :, 0].reshape(-1).long()
        keep = routes[:, :, 1].reshape(-1) < cap
        wgt = routes[:, :, 2].reshape(-1).view(torch.float32)
        pair = torch.nonzero(keep).squeeze(1)
        order = pair[torch.argsort(e_id[pair], stable=True)]
        send_counts = torch.bincount(e_id[order], minlength=E)
        rows = x[order // k]
        if world > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts)
            sc, rc = send_counts.view(world, nlx).sum(1).tolist(), recv_counts.view(world, nlx).sum(1).tolist()
            landed = torch.empty(sum(rc), H, dtype=x.dtype, device=dev)
            dist.all_to_all_single(landed, rows, rc, sc)
            per = recv_counts.view(world, nlx).cpu()
        else:
            landed, per, sc, rc = rows, send_counts.view(1, nlx).cpu(), None, None
        # rows arrive grouped by source rank, then by local expert: regroup per local expert
        offs, o = [[0] * nlx for _ in range(world)], 0
        for s in range(world):
            for lx in range(nlx):
                offs[s][lx] = o; o += int(per[s, lx])
        result = torch.empty_like(landed)
        for lx in range(nlx):
            idx = torch.cat([torch.arange(offs[s][lx], offs[s][lx] + int(per[s, lx]), device=dev) for s in range(world)])
            if idx.numel() == 0:
                continue
            xe = landed[idx]
            h = act(xe @ lw.up[lx].t())
            if gated:
                h = h * (xe @ lw.up_v[lx].t())
            result[idx] = h @ lw.down[lx].t()
        if world > 1:
            back = torch.empty(len(order), H, dtype=x.dtype, device=dev)
            dist.all_to_all_single(back, result, sc, rc)
        else:
            back = result
        out = torch.zeros(S, H, dtype=torch.float32, device=dev)
        scale = wgt[order].unsqueeze(1) if k > 1 else 1.0
        out.index_add_(0, order // k, back.float() * scale)
        return out.to(x.dtype)

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(a.steps):
        out = step()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / a.steps
    # the unfused pipeline against the fused one on the same tokens (both are this library's router)
    with torch.cuda.stream(layer.stream):
        layer.step()
    layer.check()
    agree = float((out.double() - layer.out.double()).abs().max() / layer.out.double().abs().max().clamp_min(1e-30))
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    layer.close()
    if rank != 0:
        return None
    return {"impl": "nccl_unfused", "metric": "moe_layer_tokens_per_s", "value": S * world / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.data_type.name.lower(),
            "data": "synthetic", "config": cfg, "max_rel_diff_vs_fused": agree,
            "pipeline": "router (this library) -> all_to_all_single(counts, rows) over NCCL -> per-expert "
                        "torch GEMMs -> all_to_all_single back -> weighted sum; split sizes via the host"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="scout")
    ap.add_argument("--tokens", type=int, default=None, help="override tokens_per_rank")
    ap.add_argument("--impl", default="flashmoe_b200", choices=["flashmoe_b200", "reference", "nccl_unfused"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time plain launches instead of a CUDA-graph replay")
    ap.add_argument("--others", dest="others", action="store_true", default=None,
                    help="also run the short pass over the other benchmark shapes (default: with the scout workload)")
    ap.add_argument("--no-others", dest="others", action="store_false")
    ap.add_argument("--capacity", default="nodrop", choices=["nodrop", "reference"],
                    help="expert_peer_capacity: tokens_per_rank (nothing dropped, default) or the "
                         "reference's default ceil(S/E)*k (tokens beyond it are dropped)")
    ap.add_argument("--proxy-ep", type=int, default=0,
                    help="development aid, one GPU: a logit bias routes every token to the first E/W experts, "
                         "which gives one GPU the expert load of one rank at EP=W (not a reported number)")
    a = ap.parse_args()

    import torch
    from flashmoe_b200.workloads import CONFIGS, make_tokens
    from flashmoe_b200.jit import DataType

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus and not (world == 1 and a.gpus == 1):
        print(f"bench.py: --gpus {a.gpus} but WORLD_SIZE={world}; launch with torchrun", file=sys.stderr)
        return 2
    w = CONFIGS[a.workload]
    if a.tokens:
        w = w.scaled(tokens_per_rank=a.tokens)
    if a.capacity == "reference":
        w = w.scaled(capacity=w.reference_default_capacity)
    if a.others is None:
        a.others = a.workload == "scout" and not a.tokens and not a.proxy_ep and a.capacity == "nodrop"
    a.warmup = max(a.warmup, 3)
    S, H, I, E, k = w.tokens_per_rank, w.token_dim, w.ffn_size, w.num_experts, w.top_k
    eb = 4 if w.data_type == DataType.FP32 else 2
    dtype_name = w.data_type.name.lower()
    cfg = describe(w, world, a.capacity)
    dev = torch.device("cuda", local_rank)
    have_gpu = torch.cuda.is_available()

    # ------------------------------------------------------------------ reference arm (CPU)
    if a.impl == "reference":
        if rank != 0:
            return 0
        threads = os.cpu_count() or 1
        experts = list(range(E))
        if have_gpu:
            lw_host = to_host(device_weights(w, dev, experts))
        else:
            from flashmoe_b200.workloads import make_weights
            lw_host = make_weights(w)
        x = make_tokens(w, 0)
        times = []
        for i in range(a.warmup + a.steps):
            t, n = cpu_sample(w, lw_host, x, threads)
            if i >= a.warmup:
                times.append(t)
            if sum(times) > 150:
                break
        sec = statistics.mean(times)
        val = n / sec
        line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": val, "unit": "tokens/s",
                "n_gpus": a.gpus, "steps": len(times), "warmup": a.warmup, "ms_per_step": sec * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name,
                "data": "synthetic", "config": cfg,
                "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port",
                                 "sample": f"first {n} tokens of the batch through all {E} experts "
                                           f"(CPU restatement of the reference; it has no CPU path)"},
                "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    # ------------------------------------------------------------------ this library
    if not have_gpu:
        print("bench.py: no CUDA device; the library has no CPU path", file=sys.stderr)
        return 2
    import torch.distributed as dist
    from flashmoe_b200 import _native
    from flashmoe_b200.layer import MoELayer
    torch.cuda.set_device(dev)
    if world > 1:
        import datetime
        dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=240))

    if a.impl == "nccl_unfused":
        line = unfused_arm(a, w, world, rank, local_rank, dev, dist, cfg)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        if line is not None:
            print(json.dumps(line))
        return 0

    nlx = E // world
    mine = list(range(rank * nlx, (rank + 1) * nlx))
    lw = device_weights(w, dev, mine)
    if a.proxy_ep:
        assert world == 1, "--proxy-ep is a one-GPU aid"
        bias = torch.full((E,), -1e30, dtype=torch.float32)
        bias[:E // a.proxy_ep] = 0.0
        lw.logit_bias = bias
    layer = MoELayer(w, lw, local_rank, local_experts=range(nlx))
    x = make_tokens(w, rank)
    x_pinned = x.clone().pin_memory()
    out_pinned = torch.empty_like(x_pinned).pin_memory()
    layer.tokens.copy_(x)
    torch.cuda.synchronize()
    lib = _native.lib()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    st = layer.stream
    # true when the forward runs the kernel compiled for this layer's description (built ahead of
    # time into flashmoe_b200/lib/spec by __graft_entry__.build(); the generic kernel otherwise)
    specialised = bool(layer.geometry().specialised)
    with torch.cuda.stream(st):
        for _ in range(a.warmup):
            layer.step()
    barrier()
    layer.check()
    counts = layer.counts.cpu().numpy()

    # --- device-resident timing ------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    launches0 = lib.fmoe_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.steps)]
    with torch.cuda.stream(st):
        ev0.record(st)
        for i in range(a.steps):
            layer.route()
            kev[i][0].record(st)
            layer.experts()
            kev[i][1].record(st)
        ev1.record(st)
    barrier()
    launches = lib.fmoe_launch_count() - launches0
    layer.check()
    phases = layer.phases()   # in-kernel %globaltimer stamps of the last timed launch
    ms_step_plain = max_over_ranks(ev0.elapsed_time(ev1) / a.steps)
    ms_kernel = max_over_ranks(statistics.mean(s.elapsed_time(e) for s, e in kev))

    # --- the same K steps replayed from a CUDA graph (the reference's own timing protocol,
    # quickstart.py:264-291): no host launch gaps between the kernels of a step -----------------
    ms_step, timing = ms_step_plain, "plain launches"
    if not a.no_graph:
        per_graph = 50 if a.steps % 50 == 0 else a.steps
        ok_local = 1
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                for _ in range(per_graph):
                    layer.step()
        except Exception as exc:   # capture is an optimisation of the measurement, not of the product
            ok_local = 0
            print(f"bench.py: graph capture failed ({exc}); timing plain launches", file=sys.stderr)
        if int(max_over_ranks(float(1 - ok_local))) == 0:
            with torch.cuda.stream(st):
                graph.replay()
            barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(st):
                g0.record(st)
                for _ in range(a.steps // per_graph):
                    graph.replay()
                g1.record(st)
            barrier()
            layer.check()
            launches = 3 * a.steps   # router (2) + fused forward (1) per replayed step
            ms_step = max_over_ranks(g0.elapsed_time(g1) / a.steps)
            timing = f"{a.steps} steps replayed from a CUDA graph of {per_graph} steps"

    # --- end to end through the C ABI with host buffers --------------------------------------
    # every step: H2D of that step's tokens from pinned memory, router + forward, D2H of the result.
    # (a) one step at a time (fmoe_forward_host synchronises); (b) pipelined (fmoe_forward_host_async:
    # the copies of neighbouring steps overlap the kernels), the figure reported as e2e.
    xs = [x_pinned, x.clone().pin_memory()]
    outs = [out_pinned, torch.empty_like(x_pinned).pin_memory()]
    for _ in range(2):
        layer.forward_host(x_pinned, out_pinned)
    barrier()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        layer.forward_host(x_pinned, out_pinned)
    torch.cuda.synchronize()
    e2e_sync_s = max_over_ranks((time.perf_counter() - t0) / a.steps)
    for i in range(4):
        layer.forward_host(xs[i & 1], outs[i & 1], wait=False)
    layer.host_wait()
    barrier()
    t0 = time.perf_counter()
    for i in range(a.steps):
        layer.forward_host(xs[i & 1], outs[i & 1], wait=False)
    layer.host_wait()
    e2e_s = max_over_ranks((time.perf_counter() - t0) / a.steps)
    if rank == 0:
        time.sleep(0.3)
    clocks = sampler.stop() if rank == 0 else None
    layer.check()

    # --- what the host link gives while every rank copies at once: the ceiling of the e2e figure ---
    pcie = {}
    big = layer.tokens
    for name, src, dst in (("h2d", x_pinned, big), ("d2h", big, out_pinned)):
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(10):
            dst.copy_(src, non_blocking=True)
        c1.record()
        torch.cuda.synchronize()
        pcie[name + "_gbs_per_gpu_all_ranks_copying"] = S * H * eb * 10 / (max_over_ranks(c0.elapsed_time(c1)) * 1e-3) / 1e9
    pcie["copy_ms_per_step_at_that_rate"] = S * H * eb / 1e6 * (1 / pcie["h2d_gbs_per_gpu_all_ranks_copying"] +
                                                                 1 / pcie["d2h_gbs_per_gpu_all_ranks_copying"])

    # --- roofline of the fused kernel ----------------------------------------------------------
    peaks, peaks_kind = load_peaks()
    # routed (token, expert) pairs executed on this rank: gather the counts of every rank
    if world > 1:
        allc = [None] * world
        dist.all_gather_object(allc, counts.tolist())
    else:
        allc = [counts.tolist()]
    roofline = roofline_of(w, world, mine, allc, ms_kernel, peaks, peaks_kind)
    nvlink = nvlink_of(w, mine, counts, phases, ms_kernel) if world > 1 else None
    if nvlink is not None:
        # the slower of the compute roofline and the NVLink roofline, as a fraction
        t_bound = max(roofline["t_tensor_us"], roofline["t_hbm_us"], nvlink["t_nvlink_us"])
        roofline["frac_of_slower_of_compute_and_nvlink"] = t_bound / (ms_kernel * 1e3)

    # --- output check on every rank (outside every timed region) ---------------------------------
    par = spot_parity(w, layer, lw, mine, x, dev, max(8, 32 // k))
    pars = [par]
    if world > 1:
        pars = [None] * world
        dist.all_gather_object(pars, par)
    parity = {"max_rel_err": max(p_["max_rel_err"] for p_ in pars),
              "elementwise_mismatch_frac": max(p_["elementwise_mismatch_frac"] for p_ in pars),
              "tokens_checked": sum(p_["tokens_checked"] for p_ in pars),
              "ranks_ok": sum(1 for p_ in pars if p_["ok"]), "ranks": world,
              "routing_bit_exact": all(p_["routing_bit_exact"] for p_ in pars),
              "two_launches_same_bits": all(p_["deterministic"] for p_ in pars),
              "tolerance": par.get("tolerance"),
              "method": "spot tokens of every rank: CPU-oracle routing (bit-compared with the GPU router's route "
                        "records) and the chosen experts on the host, against the kernel's output rows"}
    all_ok = parity["ranks_ok"] == world

    # --- CPU baseline on a bounded sample (rank 0, N = 1 only) ----------------------------------
    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        threads = os.cpu_count() or 1
        lw_host = to_host(lw)
        cpu_sample(w, lw_host, x, threads)     # warm-up
        ts = []
        while len(ts) < 3 and sum(ts) < 20:
            t, n = cpu_sample(w, lw_host, x, threads)
            ts.append(t)
        cpu = {"value": n / statistics.median(ts), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"first {n} tokens of the batch through all {E} experts, median of {len(ts)} runs "
                         f"(CPU restatement of the reference; the reference has no CPU path)"}
        del lw_host

    layer.close()
    del layer, lw
    torch.cuda.empty_cache()

    # --- the unfused NCCL pipeline on the same GPUs, briefly (5 timed steps), for the ratio ----------
    vs_unfused = None
    if not a.proxy_ep:
        try:
            u = unfused_arm(argparse.Namespace(steps=5, warmup=3), w, world, rank, local_rank, dev, dist, cfg)
            if u is not None:
                vs_unfused = {"unfused_ms_per_step": u["ms_per_step"], "fused_ms_per_step": ms_step,
                              "ratio": u["ms_per_step"] / ms_step, "max_rel_diff_vs_fused": u["max_rel_diff_vs_fused"],
                              "what": "bench.py --impl nccl_unfused, 5 timed steps in this run"}
        except Exception as exc:
            vs_unfused = {"error": f"{type(exc).__name__}: {exc}"[:200]}
        torch.cuda.empty_cache()

    # --- the other benchmark shapes, briefly, at the same N -----------------------------------------
    others = None
    if a.others:
        others = []
        t_start = time.perf_counter()
        for name, tokens in OTHER_WORKLOADS:
            spent = max_over_ranks(time.perf_counter() - t_start)
            if spent > 150:
                others.append({"workload": f"{name}@{tokens}", "skipped": "time budget of the short pass used up"})
                continue
            try:
                others.append(short_measure(name, tokens, world, rank, local_rank, dev, dist, peaks, peaks_kind,
                                            a.capacity))
            except Exception as exc:    # one shape failing must not lose the headline line
                others.append({"workload": f"{name}@{tokens}", "error": f"{type(exc).__name__}: {exc}"[:300]})
        # (the exit code follows the headline workload's check; the short pass reports its own
        # `parity_ranks_ok` per shape)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return 0 if all_ok else 1
    tokens_job = S * world
    line = {"metric": "moe_layer_tokens_per_s", "value": tokens_job / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name,
            "data": "synthetic", "config": cfg, "timing_used": timing,
            "tokens_per_s_per_gpu": S / (ms_step * 1e-3), "fwd_us": ms_kernel * 1e3,
            "ms_per_step_plain_launches": ms_step_plain,
            "router_us": (ms_step_plain - ms_kernel) * 1e3,
            "e2e": {"value": tokens_job / e2e_s, "unit": "tokens/s", "ms_per_step": e2e_s * 1e3,
                    "h2d_bytes_per_step": S * H * eb, "d2h_bytes_per_step": S * H * eb,
                    "ms_per_step_one_at_a_time": e2e_sync_s * 1e3, "host_link": pcie,
                    "api": "fmoe_forward_host_async + fmoe_forward_host_wait (C ABI, pinned host buffers; "
                           "copies of neighbouring steps overlap the kernels)"},
            "gpu_launches": int(launches), "specialised_kernel": specialised, "parity": parity, "phases_us": phases, "nvlink": nvlink,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks, "vs_unfused": vs_unfused,
            "other_workloads": others}
    if a.proxy_ep:
        line["proxy"] = f"one GPU carrying the expert load of one rank at EP={a.proxy_ep}; not a reported number"
    print(json.dumps(line))
    return 0 if all_ok else 1


if __name__ == "__main__":
    sys.exit(main())
