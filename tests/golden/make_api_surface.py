"""Records the reference's public Python surface as a fixture (tests/golden/api_surface.json).

Run where a checkout of the reference is at hand:

    python tests/golden/make_api_surface.py <path to the reference checkout>

The reference's package imports without a GPU (its NVSHMEM, CUDA and JIT imports are all inside
functions), so its own classes and functions are inspected, not a transcription of them: names,
order, kind and default of every parameter of the public functions and constructors
(flashmoe/__init__.py, jit.py, router.py, reference.py, cb.py), the members of the four enums,
the fields each argument object ends up with, and the capacity the reference's InitArgs derives
when none is given, over a sweep of (tokens, experts, top-k).  tests/test_abi.py holds this
package to the fixture.
"""
from __future__ import annotations

import inspect
import json
import sys
from enum import IntEnum
from pathlib import Path

OUT = Path(__file__).resolve().parent / "api_surface.json"


def params(fn):
    out = []
    for p in inspect.signature(fn).parameters.values():
        if p.name == "self":
            continue
        out.append({"name": p.name, "kind": p.kind.name,
                    "default": None if p.default is inspect.Parameter.empty else repr(p.default),
                    "required": p.default is inspect.Parameter.empty})
    return out


def functions(mod):
    return {n: params(f) for n, f in vars(mod).items()
            if inspect.isfunction(f) and not n.startswith("_") and f.__module__ == mod.__name__}


def main() -> None:
    ref_root = Path(sys.argv[1]).resolve()
    sys.path.insert(0, str(ref_root))
    import flashmoe as ref   # the reference itself
    from flashmoe import cb, jit, reference, router

    surface = {
        "package_names": sorted(n for n in vars(ref) if not n.startswith("_") and n not in ("jit", "SHOULD_FINALIZE_NVSHMEM")),
        "functions": {"flashmoe": functions(ref), "flashmoe.router": functions(router),
                      "flashmoe.reference": functions(reference), "flashmoe.cb": functions(cb)},
        "enums": {n: {m.name: int(m) for m in c} for n, c in vars(jit).items()
                  if inspect.isclass(c) and issubclass(c, IntEnum) and c is not IntEnum},
        "constructors": {"InitArgs": params(jit.InitArgs.__init__), "ForwardArgs": params(jit.ForwardArgs.__init__),
                         "RouterForwardArgs": params(router.RouterForwardArgs.__init__),
                         "RefForwardArgs": params(reference.RefForwardArgs.__init__),
                         "ContextHandle": params(jit.ContextHandle.__init__)},
    }
    # the fields every argument object carries after construction, with the values the reference's
    # own constructors leave in them for one fixed call each
    init = jit.InitArgs(jit.DataType.BF16, 1024, 5120, 8192, 16, 1, 1000, jit.MLPType.GATED, jit.ActivationType.SILU, 11, 3)
    fwd = jit.ForwardArgs(jit.MLPType.VANILLA, 1, 2, 3, 4, 5, 6, 7, 8)
    rfa = router.RouterForwardArgs(1, 2, 3, 4)
    rra = reference.RefForwardArgs(1, 2, 3, 4, 5, 6, 7, 8, expert_up_v=9, bias_up_v=10)
    plain = lambda o: {k: (int(v) if isinstance(v, IntEnum) else v) for k, v in sorted(vars(o).items())}
    surface["fields"] = {"InitArgs": plain(init), "ForwardArgs": plain(fwd), "RouterForwardArgs": plain(rfa),
                         "RefForwardArgs": plain(rra)}
    surface["context_handle_properties"] = sorted(n for n, v in vars(jit.ContextHandle).items() if isinstance(v, property))
    # derived expert capacity: [tokens_per_rank, num_experts, top_k, capacity]
    sweep = []
    for s in (1, 2, 7, 16, 100, 128, 1000, 1024, 2048, 4096, 8192, 16384):
        for e in (8, 16, 24, 64, 128, 256):
            for k in (1, 2, 3, 4, 6, 8):
                a = jit.InitArgs(jit.DataType.BF16, s, 64, 64, e, k, 1000, jit.MLPType.GATED, jit.ActivationType.SILU, 0, 0)
                sweep.append([s, e, k, int(a.expert_peer_capacity)])
    surface["derived_capacity"] = sweep
    # assertions the reference's constructors make
    def raises(fn):
        try:
            fn()
        except AssertionError:
            return True
        return False
    surface["asserts"] = {
        "gated_forward_args_need_up_v": raises(lambda: jit.ForwardArgs(jit.MLPType.GATED, 1, 2, 3, 4, 5, 6, 7, 8)),
        "gpu_arch_below_700": raises(lambda: jit.InitArgs(jit.DataType.BF16, 8, 64, 64, 8, 1, 600, 0, 0, 0, 0)),
    }
    OUT.write_text(json.dumps(surface, indent=1, sort_keys=True) + "\n")
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
