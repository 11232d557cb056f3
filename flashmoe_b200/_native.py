"""ctypes view of libflashmoe_b200.so (the C ABI in include/flashmoe_b200.h) and its build.

The library is built in-tree with nvcc for sm_100a only.  There is no fallback: if the shared
object is missing, every entry point of the package raises.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "lib" / "libflashmoe_b200.so"
SOURCES = ("router.cu", "moe_kernel.cu", "abi.cu")
NVCC_FLAGS = ("-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared", "-ldl")

IPC_HANDLE_BYTES = 64
MAX_WORLD = 8


class ModelDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "tokens_per_rank", "token_dim", "ffn_size", "num_experts", "top_k",
        "expert_peer_capacity", "data_type", "mlp_type", "act_type", "gpu_arch")]


class EpDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "ep_world", "ep_rank", "my_pe", "device_id", "num_local_experts", "topology")] + [
        ("expert_map", C.POINTER(C.c_int32)), ("rank_map", C.POINTER(C.c_int32))]


class ForwardArgsC(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "tokens", "expert_counts", "local_expert_up", "local_expert_up_v", "local_bias_up",
        "local_bias_up_v", "local_expert_down", "local_bias_down", "moe_out")] + [
        ("swish_alpha", C.c_float), ("swish_beta", C.c_float)]


class RouterArgsC(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "tokens", "weights", "routing", "expert_counts", "logit_bias")]


class Status(C.Structure):
    _fields_ = [("code", C.c_int32), ("phase", C.c_int32), ("rank", C.c_int32), ("cta", C.c_int32),
                ("detail", C.c_int64), ("epoch", C.c_uint64)]


class Geometry(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "tile_m", "tile_n0", "tile_n1", "tile_k", "stages", "round_ec", "landing_rows", "grid",
        "threads", "smem_bytes", "cta_pairs", "split_parts")] + [("symm_bytes", C.c_int64),
                                                                  ("workspace_bytes", C.c_int64),
                                                                  ("specialised", C.c_int32),
                                                                  ("reserved", C.c_int32)]


# name -> (restype, argtypes); the single source of truth for the symbol-export test too
SIGNATURES = {
    "fmoe_ctx_create": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(EpDesc), C.c_void_p,
                                  C.POINTER(C.c_void_p)]),
    "fmoe_ctx_create_in": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(EpDesc), C.c_void_p, C.c_void_p, C.c_size_t,
                                     C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "fmoe_workspace_bytes": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(EpDesc), C.POINTER(C.c_int64),
                                       C.POINTER(C.c_int64)]),
    "fmoe_symm_bytes": (C.c_int, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "fmoe_symm_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fmoe_symm_import": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "fmoe_symm_base": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "fmoe_symm_set_peer": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "fmoe_ctx_commit": (C.c_int, [C.c_void_p]),
    "fmoe_token_indices": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "fmoe_ctx_destroy": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fmoe_forward": (C.c_int, [C.c_void_p, C.POINTER(ForwardArgsC), C.c_void_p]),
    "fmoe_forward_routed": (C.c_int, [C.c_void_p, C.POINTER(RouterArgsC), C.POINTER(ForwardArgsC), C.c_void_p]),
    "fmoe_weights_changed": (C.c_int, [C.c_void_p]),
    "fmoe_ctx_load_specialised": (C.c_int, [C.c_void_p, C.c_char_p]),
    "fmoe_router_create": (C.c_int, [C.POINTER(ModelDesc), C.c_int32, C.c_int32, C.c_void_p,
                                     C.POINTER(C.c_void_p)]),
    "fmoe_router_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(RouterArgsC), C.c_void_p]),
    "fmoe_router_destroy": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fmoe_router_forward_static": (C.c_int, [C.POINTER(ModelDesc), C.c_int32, C.POINTER(RouterArgsC),
                                            C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "fmoe_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.POINTER(RouterArgsC), C.POINTER(ForwardArgsC), C.c_void_p]),
    "fmoe_forward_host_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.POINTER(RouterArgsC), C.POINTER(ForwardArgsC), C.c_void_p]),
    "fmoe_forward_host_wait": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fmoe_last_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(Status)]),
    "fmoe_strerror": (C.c_char_p, [C.c_int]),
    "fmoe_last_error": (C.c_char_p, []),
    "fmoe_launch_count": (C.c_uint64, []),
    "fmoe_get_geometry": (C.c_int, [C.c_void_p, C.POINTER(Geometry)]),
    "fmoe_debug_buffer": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p),
                                    C.POINTER(C.c_size_t)]),
}

_lib = None


class FlashMoEError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str):
        super().__init__(f"{what}: {detail} [status {code}]")
        self.code = code


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources into the in-tree shared object (sm_100a, -lineinfo)."""
    srcs = [SRC_DIR / s for s in SOURCES]
    deps = srcs + sorted(SRC_DIR.glob("*.cuh")) + [PKG_DIR.parent / "include" / "flashmoe_b200.h"]
    if not force and LIB_PATH.exists() and all(
            LIB_PATH.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libflashmoe_b200.so")
    LIB_PATH.parent.mkdir(parents=True, exist_ok=True)
    tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(tmp),
           *map(str, srcs)]
    proc = subprocess.run(cmd, cwd=SRC_DIR, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    os.replace(tmp, LIB_PATH)   # atomic publish
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m flashmoe_b200.build` "
                "(needs nvcc; targets sm_100a). There is no non-CUDA implementation.")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        l = lib()
        raise FlashMoEError(code, what, (l.fmoe_last_error() or l.fmoe_strerror(code)).decode())
