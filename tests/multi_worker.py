"""One rank of a multi-GPU parity run (launched by torchrun from test_gpu_multi.py).

Every rank holds its own tokens and its slice of the experts, runs router + fused forward three
times (new tokens each time, so the epoch protocol and the packed landing layout change between
launches) and checks its output against the single-rank CPU oracle evaluated on its tokens with
ALL experts -- the reference's own multi-rank test does the same (csrc/tests/flashmoe.cu:435-471).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

from cases import GOLDEN_CASES  # noqa: E402
from helpers import REL_TOL, elementwise_mismatch, max_rel_err, oracle_layer  # noqa: E402
from flashmoe_b200.workloads import CONFIGS, make_tokens, make_weights  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--tokens", type=int, default=None)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", local))
    from flashmoe_b200.layer import MoELayer
    w = GOLDEN_CASES.get(a.case) or CONFIGS[a.case]
    if a.tokens:
        w = w.scaled(tokens_per_rank=a.tokens)
    lw = make_weights(w)
    layer = MoELayer(w, lw, local)
    worst, worst_frac = 0.0, 0.0
    ok = True
    try:
        for step in range(3):
            x = make_tokens(w.scaled(seed=w.seed + 7 * step), rank)
            ref, _ = oracle_layer(w, x=x, lw=lw)
            out = layer.forward(x).cpu()
            err = max_rel_err(out, ref)
            frac, _ = elementwise_mismatch(out, ref, w.data_type)
            worst, worst_frac = max(worst, err), max(worst_frac, frac)
            ok = ok and bool(torch.isfinite(out.float()).all()) and err <= REL_TOL[int(w.data_type)] and frac == 0.0
        # the same step as ONE launch per rank (the router as the kernel's first phase): same bits
        layer.out.zero_()
        layer.step_one_launch()
        layer.check()
        ok = ok and bool(torch.equal(layer.out.cpu(), out))
    finally:
        layer.close()
    res = [None] * world
    dist.all_gather_object(res, {"rank": rank, "ok": ok, "err": worst, "mismatch_frac": worst_frac})
    if rank == 0:
        print("MULTI_RESULT " + json.dumps(res))
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
