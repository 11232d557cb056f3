"""The shared library loads, exports every entry point the header declares, and rejects bad
descriptions with a status code (no GPU is touched: validation comes before any CUDA call)."""
import ctypes as C
import os
import re

import pytest

import flashmoe_b200 as flashmoe
from flashmoe_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "flashmoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fmoe_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = N.lib()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(N.SIGNATURES)


def test_strerror_and_launch_count():
    lib = N.lib()
    assert lib.fmoe_strerror(0) == b"success"
    assert b"device-side" in lib.fmoe_strerror(5)
    assert lib.fmoe_launch_count() == 0


def _desc(**kw):
    d = dict(tokens_per_rank=128, token_dim=256, ffn_size=256, num_experts=8, top_k=2,
             expert_peer_capacity=128, data_type=0, mlp_type=0, act_type=1, gpu_arch=1000)
    d.update(kw)
    return N.ModelDesc(*[d[n] for n, _ in N.ModelDesc._fields_])


def _create(desc, world=1, nlx=None, emap=None):
    E = desc.num_experts
    emap = emap if emap is not None else [i // (E // world) for i in range(E)]
    ep = N.EpDesc(world, 0, 0, 0, nlx if nlx is not None else E // world, 0,
                  (C.c_int32 * len(emap))(*emap), (C.c_int32 * world)(*range(world)))
    ctx = C.c_void_p()
    rc = N.lib().fmoe_ctx_create(C.byref(desc), C.byref(ep), None, C.byref(ctx))
    return rc, N.lib().fmoe_last_error().decode()


@pytest.mark.parametrize("kw,code,needle", [
    (dict(gpu_arch=900), 2, "sm_100a"),
    (dict(token_dim=100), 1, "token dimension"),
    (dict(ffn_size=72), 1, "Intermediate size"),
    (dict(top_k=9), 1, "top_k"),
    (dict(num_experts=12), 1, "multiple of 8"),
    (dict(data_type=3), 2, "FP64 is not built"),
    (dict(expert_peer_capacity=0), 1, "expert_peer_capacity"),
])
def test_bad_descriptions_are_rejected(kw, code, needle):
    rc, msg = _create(_desc(**kw))
    assert rc == code, msg
    assert needle in msg


def test_bad_expert_maps_are_rejected():
    rc, msg = _create(_desc(), world=2, emap=[0] * 8)
    assert rc == 1 and "expert_map" in msg
    rc, msg = _create(_desc(), world=2, nlx=3)
    assert rc == 1


def test_workspace_bytes_follow_the_description_without_a_device():
    """fmoe_workspace_bytes / flashmoe.get_workspace_bytes (the reference's getWorkspaceBytes): host
    arithmetic only.  Scout shapes on 8 ranks, no drop: the landing area holds every rank's 1024
    rows plus one tile of slack per local expert, the return area this rank's 1024 rows."""
    S, H, I, E, W = 1024, 5120, 8192, 16, 8
    arg = flashmoe.InitArgs(flashmoe.DataType.BF16, S, H, I, E, 1, 1000, flashmoe.MLPType.GATED,
                            flashmoe.ActivationType.SILU, 0, 0, expert_peer_capacity=S)
    b = flashmoe.get_workspace_bytes(arg, ep_world=W)
    rows = W * S + (E // W) * 128
    assert rows * H * 2 + S * H * 2 <= b["symmetric"] <= rows * H * 2 + S * H * 2 + (1 << 20)
    # GEMM0 output, plus the fp32 partial sums of the GEMM1 tiles the closing wave cuts along K
    # (160 tiles x 2 parts x 128 x 256 floats)
    split = 160 * 2 * 128 * 256 * 4
    assert rows * I * 2 + split <= b["workspace"] <= rows * I * 2 + split + (4 << 20)
    one = flashmoe.get_workspace_bytes(arg, ep_world=1)
    assert one["symmetric"] < b["symmetric"]
    # FP32 layers add the three BF16 planes of the local experts' weights
    arg32 = flashmoe.InitArgs(flashmoe.DataType.FP32, 128, 1024, 2048, 8, 2, 1000, flashmoe.MLPType.GATED,
                              flashmoe.ActivationType.SILU, 0, 0, expert_peer_capacity=128)
    assert flashmoe.get_workspace_bytes(arg32)["workspace"] >= 8 * 1024 * 2048 * 2 * 3 * 3
    # the same checks as create
    desc, ep = _desc(token_dim=100), N.EpDesc(1, 0, 0, 0, 8, 0, None, None)
    out = C.c_int64()
    assert N.lib().fmoe_workspace_bytes(C.byref(desc), C.byref(ep), C.byref(out), None) == 1
    assert "token dimension" in N.lib().fmoe_last_error().decode()


def test_python_api_surface_matches_the_reference():
    a = flashmoe.InitArgs(flashmoe.DataType.BF16, 1024, 5120, 8192, 16, 1, 1000, flashmoe.MLPType.GATED,
                          flashmoe.ActivationType.SILU, 0, 0)
    assert a.expert_peer_capacity == 64          # ceil(1024 / 16) * 1
    assert a.ep_rank is None and a.expert_map is None
    assert (int(flashmoe.MLPType.GATED), int(flashmoe.MLPType.VANILLA)) == (0, 1)
    assert [int(x) for x in flashmoe.DataType] == [0, 1, 2, 3]
    assert [int(x) for x in flashmoe.ActivationType] == [0, 1, 2, 3]
    assert (int(flashmoe.Topology.NVLINK_ONLY), int(flashmoe.Topology.MIXED)) == (0, 1)
    with pytest.raises(AssertionError):
        flashmoe.ForwardArgs(flashmoe.MLPType.GATED, 1, 2, 3, 4, 5, 6, 7, 0)
    f = flashmoe.ForwardArgs(flashmoe.MLPType.VANILLA, 1, 2, 3, 4, 5, 6, 7, 0)
    assert f.local_expert_up_v is None and f.swish_alpha == 1.0
    with pytest.raises(AssertionError):
        flashmoe.InitArgs(flashmoe.DataType.BF16, 8, 64, 64, 8, 1, 600, 0, 0, 0, 0)
    for name in ("initialize", "forward", "finalize", "router", "cb", "get_local_rank"):
        assert hasattr(flashmoe, name)
    for name in ("initialize", "forward", "finalize", "RouterForwardArgs"):
        assert hasattr(flashmoe.router, name)
    for name in ("initialize", "forward", "RefForwardArgs"):
        assert hasattr(flashmoe.reference, name)
    r = flashmoe.reference.RefForwardArgs(1, 2, 3, 4, 5, 6, 7, 8, expert_up_v=9, bias_up_v=10)
    assert (r.expert_up, r.expert_down, r.bias_up, r.bias_down, r.ref_input, r.ref_interim0, r.ref_interim1,
            r.ref_out, r.expert_up_v, r.bias_up_v) == (1, 2, 3, 4, 5, 6, 7, 8, 9, 10)


def _params(fn):
    import inspect
    out = []
    for q in inspect.signature(fn).parameters.values():
        if q.name != "self":
            out.append({"name": q.name, "kind": q.kind.name,
                        "default": None if q.default is inspect.Parameter.empty else repr(q.default),
                        "required": q.default is inspect.Parameter.empty})
    return out


def _holds(ours, theirs, where):
    """Every parameter of the reference's callable is here under the same name, at the same position
    among the positional ones, of the same kind and with the same default; what this package adds
    must be optional, so that a call written for the reference means the same thing here."""
    ours_by = {q["name"]: q for q in ours}
    for q in theirs:
        assert q["name"] in ours_by, f"{where}: parameter {q['name']} is missing"
        mine = ours_by[q["name"]]
        assert (mine["kind"], mine["default"], mine["required"]) == (q["kind"], q["default"], q["required"]), \
            f"{where}: {q['name']} is {mine}, the reference has {q}"
    positional = lambda ps: [q["name"] for q in ps if q["kind"] in ("POSITIONAL_ONLY", "POSITIONAL_OR_KEYWORD")]
    assert positional(ours)[:len(positional(theirs))] == positional(theirs), f"{where}: positional order differs"
    for q in ours:
        if q["name"] not in {t["name"] for t in theirs}:
            assert not q["required"], f"{where}: added parameter {q['name']} must be optional"


def test_python_api_follows_the_surface_recorded_from_the_reference():
    """tests/golden/api_surface.json was written by tests/golden/make_api_surface.py from the
    reference's own modules (flashmoe/__init__.py, jit.py, router.py, reference.py, cb.py)."""
    import json
    from enum import IntEnum
    surface = json.load(open(os.path.join(ROOT, "tests", "golden", "api_surface.json")))
    for name in surface["package_names"]:
        assert hasattr(flashmoe, name), f"flashmoe.{name} is missing"
    modules = {"flashmoe": flashmoe, "flashmoe.router": flashmoe.router, "flashmoe.reference": flashmoe.reference,
               "flashmoe.cb": flashmoe.cb}
    for mod_name, fns in surface["functions"].items():
        for fn_name, theirs in fns.items():
            fn = getattr(modules[mod_name], fn_name, None)
            assert callable(fn), f"{mod_name}.{fn_name} is missing"
            _holds(_params(fn), theirs, f"{mod_name}.{fn_name}")
    for enum_name, members in surface["enums"].items():
        ours = getattr(flashmoe, enum_name)
        assert {m.name: int(m) for m in ours} == members
    classes = {"InitArgs": flashmoe.InitArgs, "ForwardArgs": flashmoe.ForwardArgs,
               "RouterForwardArgs": flashmoe.router.RouterForwardArgs,
               "RefForwardArgs": flashmoe.reference.RefForwardArgs, "ContextHandle": flashmoe.ContextHandle}
    for cls_name, theirs in surface["constructors"].items():
        _holds(_params(classes[cls_name].__init__), theirs, f"{cls_name}()")
    # the same constructor calls leave the same values in the same fields
    D, M, A = flashmoe.DataType, flashmoe.MLPType, flashmoe.ActivationType
    made = {
        "InitArgs": flashmoe.InitArgs(D.BF16, 1024, 5120, 8192, 16, 1, 1000, M.GATED, A.SILU, 11, 3),
        "ForwardArgs": flashmoe.ForwardArgs(M.VANILLA, 1, 2, 3, 4, 5, 6, 7, 8),
        "RouterForwardArgs": flashmoe.router.RouterForwardArgs(1, 2, 3, 4),
        "RefForwardArgs": flashmoe.reference.RefForwardArgs(1, 2, 3, 4, 5, 6, 7, 8, expert_up_v=9, bias_up_v=10),
    }
    for cls_name, fields in surface["fields"].items():
        for field, value in fields.items():
            got = getattr(made[cls_name], field)
            got = int(got) if isinstance(got, IntEnum) else got
            assert got == value, f"{cls_name}.{field}: {got!r}, the reference leaves {value!r}"
    for prop in surface["context_handle_properties"]:
        assert isinstance(getattr(flashmoe.ContextHandle, prop), property)
    for s, e, k, cap in surface["derived_capacity"]:
        a = flashmoe.InitArgs(D.BF16, s, 64, 64, e, k, 1000, M.GATED, A.SILU, 0, 0)
        assert a.expert_peer_capacity == cap, (s, e, k)
    assert surface["asserts"]["gated_forward_args_need_up_v"] and surface["asserts"]["gpu_arch_below_700"]
    with pytest.raises(AssertionError):
        flashmoe.ForwardArgs(M.GATED, 1, 2, 3, 4, 5, 6, 7, 8)
    with pytest.raises(AssertionError):
        flashmoe.InitArgs(D.BF16, 8, 64, 64, 8, 1, 600, 0, 0, 0, 0)


def test_initialize_without_a_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    a = flashmoe.InitArgs(flashmoe.DataType.BF16, 128, 256, 256, 8, 2, 1000, flashmoe.MLPType.GATED,
                          flashmoe.ActivationType.SILU, 0, 0)
    with pytest.raises(flashmoe.FlashMoEError):
        flashmoe.initialize(a)
    with pytest.raises(RuntimeError):          # the checker has no CPU path either
        flashmoe.reference.initialize(a)
