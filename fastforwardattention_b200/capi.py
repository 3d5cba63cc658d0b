"""ctypes view of libffa_b200.so (include/ffa_c_api.h) for hosts without the torch extension.

This is the binding a non-torch caller writes; the GPU parity tests drive the C ABI through
it with raw device pointers (the benchmark goes through the torch extension instead).  No computation happens in Python.
"""
from __future__ import annotations

import ctypes as C
import os

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libffa_b200.so")

F32, F16, BF16 = 0, 1, 2
MODE_EXACT, MODE_ROUND_LIKE_TORCH = 0, 1

SYMBOLS = ["ffa_cache_bytes", "ffa_cache_init", "ffa_plan_create", "ffa_plan_destroy", "ffa_plan_get_launch",
           "ffa_plan_set_launch", "ffa_plan_set_mode", "ffa_workspace_bytes", "ffa_workspace_bind", "ffa_attention",
           "ffa_device_status", "ffa_launch_count", "ffa_last_error", "ffa_attention_static_scratch", "ffa_static_scratch_status", "ffa_static_scratch_selftest_wait_timeout", "ffa_selftest_wait_timeout", "ffa_plan_set_prune_path", "ffa_plan_create_offline",
           "ffa_plan_get_prune_launch", "ffa_plan_get_prune_path", "ffa_cache_copy", "ffa_attention_paged", "ffa_peer_gather_bytes",
           "ffa_peer_mem_alloc", "ffa_peer_mem_open", "ffa_peer_mem_close", "ffa_peer_mem_free", "ffa_peer_gather_attach",
           "ffa_peer_gather", "ffa_plan_set_cluster_merge", "ffa_peer_push_target"]


class Launch(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("tile_rows", "stages", "consumer_warps", "ctas_per_sm", "grid", "smem_bytes",
                                        "parts_per_bh")]


class FfaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"ffa error {code}: {msg}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m fastforwardattention_b200.build`")
        L = C.CDLL(LIB_PATH)
        vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
        L.ffa_cache_bytes.argtypes = [i, i, i, i, i, C.POINTER(sz), C.POINTER(sz)]
        L.ffa_cache_init.argtypes = [i, i, i, i, i, i, vp, vp, vp, vp, vp]
        L.ffa_cache_copy.argtypes = [i, i, i, i, i, i, i, vp, vp, vp, vp, vp]
        L.ffa_plan_create.argtypes = [i, i, i, i, i, i, i, C.POINTER(vp)]
        L.ffa_plan_create_offline.argtypes = [i, i, i, i, i, i, i, i, i, C.POINTER(vp)]
        L.ffa_plan_get_prune_launch.argtypes = [vp, i] + [C.POINTER(i)] * 5
        L.ffa_plan_get_prune_path.argtypes = [vp, i, C.c_float, i, C.POINTER(i)]
        L.ffa_plan_destroy.argtypes = [vp]
        L.ffa_plan_destroy.restype = None
        L.ffa_plan_get_launch.argtypes = [vp, i, C.POINTER(Launch)]
        L.ffa_plan_set_launch.argtypes = [vp, C.POINTER(Launch)]
        L.ffa_plan_set_mode.argtypes = [vp, i]
        L.ffa_plan_set_prune_path.argtypes = [vp, i]
        L.ffa_plan_set_cluster_merge.argtypes = [vp, i]
        L.ffa_workspace_bytes.argtypes = [vp, i]
        L.ffa_workspace_bytes.restype = sz
        L.ffa_workspace_bind.argtypes = [vp, vp, sz, vp]
        L.ffa_attention.argtypes = [vp, vp, vp, vp, vp, vp, vp, f, i, vp, i, f, vp, vp]
        L.ffa_attention_paged.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, vp, f, i, vp, i, f, vp, vp]
        L.ffa_device_status.argtypes = [vp, vp, C.POINTER(i)]
        L.ffa_attention_static_scratch.argtypes = [i, i, i, i, i, vp, vp, vp, vp, vp, vp, f, i, vp, vp, C.c_char_p, sz]
        L.ffa_selftest_wait_timeout.argtypes = [vp, C.c_uint, vp]
        L.ffa_static_scratch_status.argtypes = [vp, C.POINTER(i)]
        L.ffa_static_scratch_selftest_wait_timeout.argtypes = [C.c_uint, vp]
        L.ffa_peer_gather_bytes.argtypes = [vp, i]
        L.ffa_peer_gather_bytes.restype = sz
        L.ffa_peer_mem_alloc.argtypes = [sz, C.POINTER(vp), C.c_char_p]
        L.ffa_peer_mem_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.ffa_peer_mem_close.argtypes = [vp]
        L.ffa_peer_mem_free.argtypes = [vp]
        L.ffa_peer_gather_attach.argtypes = [vp, i, i, C.POINTER(vp), sz]
        L.ffa_peer_gather.argtypes = [vp, vp, vp, i, C.c_uint, vp]
        L.ffa_peer_push_target.argtypes = [vp, vp]
        L.ffa_launch_count.restype = C.c_ulonglong
        L.ffa_last_error.restype = C.c_char_p
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise FfaError(rc, lib().ffa_last_error().decode())
