"""Loads libglmserve_b200.so (the C ABI in include/glmserve_b200.h).  No fallback: if the
library is missing the import of any operator raises."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libglmserve_b200.so")

STATUS = {0: "ok", 1: "invalid argument", 2: "unsupported shape or format", 3: "kernel launch failed",
          4: "device-side wait timed out", 5: "CUDA runtime call failed", 6: "workspace too small",
          7: "problem larger than the built-in fixed-size buffer"}


class GsbError(RuntimeError):
    def __init__(self, status: int, where: str):
        super().__init__(f"{where}: status {status} ({STATUS.get(status, 'unknown')})")
        self.status = status


class MoeConfig(C.Structure):
    """Mirror of struct gsb_moe_config."""
    _fields_ = [("hidden", C.c_int), ("n_experts", C.c_int), ("topk", C.c_int), ("moe_inter", C.c_int),
                ("shared_inter", C.c_int), ("group", C.c_int), ("norm_topk", C.c_int),
                ("routed_scale", C.c_float), ("router_w", C.c_void_p), ("e_bias", C.c_void_p),
                ("gate_q", C.c_void_p), ("gate_sc", C.c_void_p), ("up_q", C.c_void_p),
                ("up_sc", C.c_void_p), ("down_q", C.c_void_p), ("down_sc", C.c_void_p),
                ("sg_q", C.c_void_p), ("sg_sc", C.c_void_p), ("su_q", C.c_void_p), ("su_sc", C.c_void_p),
                ("sd_q", C.c_void_p), ("sd_sc", C.c_void_p), ("gate_up_packed", C.c_void_p),
                ("down_packed", C.c_void_p), ("shared_gate_up_packed", C.c_void_p),
                ("shared_down_packed", C.c_void_p), ("ep_size", C.c_int), ("ep_rank", C.c_int),
                ("fixed_routing", C.c_int), ("down_inter", C.c_int), ("shared_down_inter", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m glmserve_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        L = C.CDLL(LIB_PATH)
        L.gsb_status_string.restype = C.c_char_p
        L.gsb_build_info.restype = C.c_char_p
        L.gsb_prepack_bytes.restype = C.c_size_t
        L.gsb_moe_workspace_bytes.restype = C.c_size_t
        L.gsb_moe_workspace_bytes.argtypes = [C.c_void_p, C.c_int]
        L.gsb_moe_layer_create.argtypes = [C.POINTER(MoeConfig), C.POINTER(C.c_void_p)]
        L.gsb_moe_layer_destroy.argtypes = [C.c_void_p]
        L.gsb_moe_layer_destroy.restype = None
        L.gsb_comm_heap.restype = C.c_void_p
        L.gsb_comm_heap_bytes.restype = C.c_size_t
        L.gsb_comm_allreduce_reserve.restype = C.c_size_t
        L.gsb_moe_ep_heap_bytes.restype = C.c_size_t
        L.gsb_moe_ep_workspace_bytes.restype = C.c_size_t
        L.gsb_comm_destroy.restype = None
        L.gsb_comm_set_wait_cycles.argtypes = [C.c_void_p, C.c_longlong]
        L.gsb_comm_open_loopback.argtypes = [C.c_void_p]
        L.gsb_prefill_wait_profile.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise GsbError(status, where)
