#!/usr/bin/env python
"""Benchmark of the MoE-layer forward (router + dispatch + experts + combine).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload scout] [--impl reference]

N > 1 is launched by torchrun (one rank per GPU); experts are sharded over the ranks and every
rank keeps `tokens_per_rank` tokens (weak scaling).  Rank 0 prints ONE JSON line.

A step = one pass of the hot path over one batch of synthetic tokens: the router (2 launches)
and the fused forward (1 launch).  `value` is whole-job tokens/s with the batch resident in
HBM; `e2e` is the same through the C ABI's host-buffer entry point (H2D of the tokens from
pinned memory, router + forward, D2H of the result, every step).  `roofline` describes the
fused forward kernel, timed with CUDA events on its own stream inside the timed loop.
`--impl reference` times the CPU restatement of the reference (the oracle) on the host cores:
the reference itself has no CPU path and needs cuBLASDx + NVSHMEM to build.
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
    distributions: router N(0, 1/H), expert matrices N(0, 0.02), zero biases."""
    import torch
    from flashmoe_b200.workloads import TORCH_DTYPE, LayerWeights
    from flashmoe_b200.jit import MLPType
    dt = TORCH_DTYPE[w.data_type]
    E, H, I = w.num_experts, w.token_dim, w.ffn_size
    g = torch.Generator(device=dev).manual_seed(w.seed)
    router = (torch.randn(E, H, generator=g, device=dev) * (1.0 / H) ** 0.5).to(dt)
    n = len(experts)
    ge = torch.Generator(device=dev).manual_seed(w.seed * 7919 + experts[0])

    def mat(*shape):
        out = torch.empty(*shape, dtype=dt, device=dev)
        for i in range(shape[0]):   # one expert at a time keeps the fp32 temporary small
            out[i] = (torch.randn(*shape[1:], generator=ge, device=dev) * 0.02).to(dt)
        return out
    gated = w.mlp_type == MLPType.GATED
    z = lambda *s: torch.zeros(*s, dtype=dt, device=dev)
    logit_bias = None
    if w.zipf_bias:
        from flashmoe_b200.workloads import make_weights
        logit_bias = make_weights(w.scaled(token_dim=64, ffn_size=64)).logit_bias
    return LayerWeights(router, mat(n, I, H), mat(n, I, H) if gated else None, mat(n, H, I), z(n, I),
                        z(n, I) if gated else None, z(n, H), logit_bias)


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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="scout")
    ap.add_argument("--tokens", type=int, default=None, help="override tokens_per_rank")
    ap.add_argument("--impl", default="flashmoe_b200", choices=["flashmoe_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time plain launches instead of a CUDA-graph replay")
    ap.add_argument("--capacity", default="nodrop", choices=["nodrop", "reference"],
                    help="expert_peer_capacity: tokens_per_rank (nothing dropped, default) or the "
                         "reference's default ceil(S/E)*k (tokens beyond it are dropped)")
    a = ap.parse_args()

    import torch
    from flashmoe_b200.workloads import CONFIGS, make_tokens, weight_bytes_per_rank
    from flashmoe_b200.jit import MLPType

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
    a.warmup = max(a.warmup, 3)
    S, H, I, E, k = w.tokens_per_rank, w.token_dim, w.ffn_size, w.num_experts, w.top_k
    eb = 2
    cfg = {"workload": f"{w.name}: tokens_per_rank={S} H={H} I={I} E={E} k={k} "
                       f"{'gated' if w.mlp_type == MLPType.GATED else 'plain'} {w.act_type.name} "
                       f"{w.data_type.name}, expert_peer_capacity={w.expert_peer_capacity} "
                       f"({'no drop' if a.capacity == 'nodrop' else 'reference default, drops'})",
           "parallelism": f"ep{world}xdp{world}", "experts_per_gpu": E // world,
           "step": "router (2 launches) + fused dispatch/experts/combine (1 launch)"}
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
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
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
        dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    nlx = E // world
    mine = list(range(rank * nlx, (rank + 1) * nlx))
    lw = device_weights(w, dev, mine)
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

    # --- roofline of the fused kernel ----------------------------------------------------------
    peaks, peaks_kind = load_peaks()
    # routed (token, expert) pairs executed on this rank: gather the counts of every rank
    if world > 1:
        allc = [None] * world
        dist.all_gather_object(allc, counts.tolist())
    else:
        allc = [counts.tolist()]
    cap = w.expert_peer_capacity
    pairs_here = sum(min(c[e], cap) for c in allc for e in mine)
    active = sum(1 for e in mine if any(c[e] > 0 for c in allc))   # experts whose weights are read
    c_mlp = 6 if w.mlp_type == MLPType.GATED else 4
    flops = float(pairs_here) * c_mlp * H * I
    hbm_bytes = weight_bytes_per_rank(w, active) + 2.0 * S * H * eb
    t_tensor = flops / (peaks["bf16_tflops_sustained"] * 1e12)
    t_hbm = hbm_bytes / (peaks["hbm_gbs"] * 1e9)
    sec_kernel = ms_kernel * 1e-3
    if t_hbm >= t_tensor:
        ach, peak, unit, bound = hbm_bytes / sec_kernel / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
    else:
        ach, peak, unit, bound = flops / sec_kernel / 1e12, peaks["bf16_tflops_sustained"], "TFLOP/s", "tensor"
    roofline = {"kernel": "moe_forward_kernel", "bound": bound, "achieved": ach, "peak": peak, "unit": unit,
                "frac": ach / peak, "peak_source": f"of {peaks_kind}",
                "traffic": load_traffic(w.name, world), "ms_per_launch": ms_kernel,
                "algorithmic_flops": flops, "algorithmic_hbm_bytes": hbm_bytes,
                "active_local_experts": active, "routed_pairs": pairs_here,
                "t_tensor_us": t_tensor * 1e6, "t_hbm_us": t_hbm * 1e6,
                "pct_dense_bf16_peak_burst": 100.0 * flops / sec_kernel / (peaks["bf16_tflops"] * 1e12)}

    # --- NVLink: bytes this rank pushed to other GPUs during the dispatch phase -------------------
    nvlink = None
    if world > 1:
        remote_rows = sum(min(counts[e], cap) for e in range(E) if e not in mine)
        out_bytes = float(remote_rows) * H * eb
        nvlink = {"dispatch_bytes_out": out_bytes, "return_bytes_in": out_bytes,
                  "dispatch_us": phases["dispatch"],
                  "dispatch_gbs": out_bytes / max(phases["dispatch"], 1e-9) / 1e3,
                  "peak_nominal_gbs": 900.0, "peak_measured_peer_copy_gbs": 770.0,
                  "note": "rank 0, per direction; the dispatch phase also copies the local rows; "
                          "returned rows travel during the GEMM phase (GEMM1 epilogues store them remotely)"}

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

    layer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return 0
    tokens_job = S * world
    weights_mb = weight_bytes_per_rank(w, nlx) / 1e6
    cfg["timing"] = timing
    cfg["l2"] = (f"no flush: each step streams {weights_mb:.0f} MB of expert weights per GPU, "
                 f"larger than the 126 MB L2") if weights_mb * 1e6 > L2_BYTES else "working set fits L2"
    line = {"metric": "moe_layer_tokens_per_s", "value": tokens_job / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": cfg,
            "tokens_per_s_per_gpu": S / (ms_step * 1e-3), "fwd_us": ms_kernel * 1e3,
            "ms_per_step_plain_launches": ms_step_plain,
            "router_us": (ms_step_plain - ms_kernel) * 1e3,
            "e2e": {"value": tokens_job / e2e_s, "unit": "tokens/s", "ms_per_step": e2e_s * 1e3,
                    "h2d_bytes_per_step": S * H * eb, "d2h_bytes_per_step": S * H * eb,
                    "ms_per_step_one_at_a_time": e2e_sync_s * 1e3,
                    "api": "fmoe_forward_host_async + fmoe_forward_host_wait (C ABI, pinned host buffers; "
                           "copies of neighbouring steps overlap the kernels)"},
            "gpu_launches": int(launches), "phases_us": phases, "nvlink": nvlink, "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
