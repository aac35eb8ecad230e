"""ctypes access to the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import this
package; the shipped library (``glmserve_b200``) never does.

``liboracle.so`` is the plain-C restatement (``moe_oracle.c``); ``_ref/libglmref.so`` is
the reference's own CPU code built by ``make -C oracle ref`` where the reference sources
are present.  Arrays are numpy, C-contiguous; scales are float32 holding fp16-representable
values.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def ref_root():
    """The reference checkout: $REF_ROOT, else a folder named ``reference`` beside this repository
    (None when neither exists)."""
    cand = os.environ.get("REF_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src")) else None


def build(with_ref: bool = True) -> None:
    """Compile liboracle.so and, when the reference tree exists, _ref/libglmref.so."""
    env = dict(os.environ, CC="gcc", CXX="g++")
    subprocess.run(["make", "-C", _HERE, "all"], check=True, env=env, capture_output=True)
    ref_root_ = ref_root()
    if with_ref and ref_root_:
        subprocess.run(["make", "-C", _HERE, "ref", f"REF_ROOT={ref_root_}"], check=True, env=env,
                       capture_output=True)


def _opt(a, dtype):
    if a is None:
        return None
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        _lib = C.CDLL(path)
        _lib.orc_max_threads.restype = C.c_int
    return _lib


def max_threads() -> int:
    return int(lib().orc_max_threads())


def dequant_int4(packed, scales, count, group):
    out = np.empty(count, np.float32)
    p = np.ascontiguousarray(packed, np.uint8)
    s = np.ascontiguousarray(scales, np.float32)
    lib().orc_dequant_int4(_ptr(p), _ptr(s), C.c_int64(count), C.c_int64(group), _ptr(out))
    return out


def linear(w, x, bias=None):
    w = np.ascontiguousarray(w, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    n, inn = x.shape
    out = w.shape[0]
    y = np.empty((n, out), np.float32)
    b = _opt(bias, np.float32)
    lib().orc_linear(_ptr(w), _ptr(b), _ptr(x), _ptr(y), C.c_int64(n), C.c_int64(inn), C.c_int64(out))
    return y


def rmsnorm_rows(x, w, eps):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty_like(x)
    lib().orc_rmsnorm_rows(_ptr(x), _ptr(w), _ptr(out), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]),
                           C.c_float(eps))
    return out


def router(logits, e_bias, topk, norm_topk=True, routed_scale=2.5):
    """Returns (ids int32 [n,topk], weights f32 [n,topk], tokens_with_ties)."""
    logits = np.ascontiguousarray(logits, np.float32)
    n, E = logits.shape
    ids = np.empty((n, topk), np.int32)
    w = np.empty((n, topk), np.float32)
    b = _opt(e_bias, np.float32)
    f = lib().orc_router
    f.restype = C.c_int
    ties = f(_ptr(logits), _ptr(b), n, E, topk, int(bool(norm_topk)), C.c_float(routed_scale),
             _ptr(ids), _ptr(w))
    return ids, w, int(ties)


def dispatch(topk_ids, E):
    """Returns (expert_offsets [E+1], sorted_token_ids [P], sorted_row [P])."""
    ids = np.ascontiguousarray(topk_ids, np.int32)
    n, topk = ids.shape
    offs = np.empty(E + 1, np.int32)
    tok = np.empty(max(n * topk, 1), np.int32)
    row = np.empty(max(n * topk, 1), np.int32)
    lib().orc_dispatch(_ptr(ids), n, topk, E, _ptr(offs), _ptr(tok), _ptr(row))
    return offs, tok[: n * topk], row[: n * topk]


def gemm_w4a16(x, qW, scales, group, bias=None, nthreads=0):
    x = np.ascontiguousarray(x, np.float32)
    qW = np.ascontiguousarray(qW, np.uint8)
    scales = np.ascontiguousarray(scales, np.float32)
    n, inn = x.shape
    out = qW.shape[0]
    y = np.empty((n, out), np.float32)
    b = _opt(bias, np.float32)
    lib().orc_gemm_w4a16(_ptr(x), _ptr(qW), _ptr(scales), _ptr(b), _ptr(y), C.c_int64(n),
                         C.c_int64(inn), C.c_int64(out), C.c_int64(group),
                         nthreads or max_threads())
    return y


def _wargs(L):
    """The twelve weight pointers of a layer dict (see glmserve_b200.synth.make_layer)."""
    keys = ["gate_q", "gate_sc", "up_q", "up_sc", "down_q", "down_sc",
            "sg_q", "sg_sc", "su_q", "su_sc", "sd_q", "sd_sc"]
    arrs = []
    for k in keys:
        a = L.get(k)
        if a is None:
            arrs.append(None)
        else:
            arrs.append(np.ascontiguousarray(a, np.uint8 if k.endswith("_q") else np.float32))
    return arrs


def moe_experts_w4(x, topk_ids, topk_w, L, nthreads=0, return_slots=False):
    x = np.ascontiguousarray(x, np.float32)
    ids = np.ascontiguousarray(topk_ids, np.int32)
    w = np.ascontiguousarray(topk_w, np.float32)
    n, H = x.shape
    topk = ids.shape[1]
    a = _wargs(L)
    out = np.empty((n, H), np.float32)
    ys = np.empty((n * topk, H), np.float32) if return_slots else None
    lib().orc_moe_experts_w4(_ptr(x), _ptr(ids), _ptr(w), *[_ptr(t) for t in a[:6]], n, topk, H,
                             int(L["I"]), int(L["E"]), int(L["group"]), _ptr(out), _ptr(ys),
                             nthreads or max_threads())
    return (out, ys) if return_slots else out


def moe_layer_w4(x, L, logits_in=None, nthreads=0):
    """Whole layer on the CPU.  Returns dict(logits, ids, w, out, ties)."""
    x = np.ascontiguousarray(x, np.float32)
    n, H = x.shape
    E, topk = int(L["E"]), int(L["topk"])
    a = _wargs(L)
    rw = np.ascontiguousarray(L["router_w"], np.float32)
    eb = _opt(L.get("e_bias"), np.float32)
    li = _opt(logits_in, np.float32)
    logits = np.empty((n, E), np.float32)
    ids = np.empty((n, topk), np.int32)
    w = np.empty((n, topk), np.float32)
    out = np.empty((n, H), np.float32)
    f = lib().orc_moe_layer_w4
    f.restype = C.c_int
    ties = f(_ptr(x), n, H, int(L["I"]), int(L["Is"]), E, topk, int(L["group"]), _ptr(rw), _ptr(eb),
             int(bool(L["norm_topk"])), C.c_float(L["routed_scale"]), *[_ptr(t) for t in a],
             _ptr(li), _ptr(logits), _ptr(ids), _ptr(w), _ptr(out), nthreads or max_threads())
    return dict(logits=logits, ids=ids, w=w, out=out, ties=int(ties))


def moe_block_layer_w4(hidden, norm_w, eps, L, logits_in=None, nthreads=0):
    """h <- h + moe(rmsnorm(h)) in place on a float32 copy; returns (hidden, ids)."""
    h = np.array(hidden, np.float32, order="C")
    n, H = h.shape
    E, topk = int(L["E"]), int(L["topk"])
    a = _wargs(L)
    rw = np.ascontiguousarray(L["router_w"], np.float32)
    eb = _opt(L.get("e_bias"), np.float32)
    li = _opt(logits_in, np.float32)
    nw = np.ascontiguousarray(norm_w, np.float32)
    ids = np.empty((n, topk), np.int32)
    f = lib().orc_moe_block_layer_w4
    f.restype = C.c_int
    f(_ptr(h), _ptr(nw), C.c_float(eps), n, H, int(L["I"]), int(L["Is"]), E, topk, int(L["group"]),
      _ptr(rw), _ptr(eb), int(bool(L["norm_topk"])), C.c_float(L["routed_scale"]),
      *[_ptr(t) for t in a], _ptr(li), _ptr(ids), nthreads or max_threads())
    return h, ids


# ---- the reference's own code (oracle/_ref) -------------------------------------------
_ref = None


def ref_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libglmref.so"))


def ref():
    global _ref
    if _ref is None:
        _ref = C.CDLL(os.path.join(_HERE, "_ref", "libglmref.so"))
        _ref.ref_moe_mlp_w4.restype = C.c_double
        _ref.ref_moe_run.restype = C.c_double
        _ref.ref_moe_run.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        _ref.ref_moe_create.restype = C.c_void_p
        _ref.ref_moe_destroy.argtypes = [C.c_void_p]
        _ref.ref_moe_destroy.restype = None
    return _ref


def ref_dequant_int4(packed, scales, count, group):
    out = np.empty(count, np.float32)
    p = np.ascontiguousarray(packed, np.uint8)
    s = np.ascontiguousarray(scales, np.float32)
    ref().ref_dequant_int4(_ptr(p), _ptr(s), C.c_int64(count), C.c_int64(group), _ptr(out))
    return out


def ref_rmsnorm_rows(x, w, eps):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty_like(x)
    ref().ref_rmsnorm_rows(_ptr(x), _ptr(w), _ptr(out), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]),
                           C.c_float(eps))
    return out


def ref_linear_forward(w, x):
    w = np.ascontiguousarray(w, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty((x.shape[0], w.shape[0]), np.float32)
    ref().ref_linear_forward(_ptr(w), _ptr(x), _ptr(y), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]),
                             C.c_int64(w.shape[0]))
    return y


def ref_moe_mlp_w4(x, L, active=None):
    """The reference's GLM52Model::moe_mlp.  Returns (out, seconds inside moe_mlp)."""
    x = np.ascontiguousarray(x, np.float32)
    n, H = x.shape
    a = _wargs(L)
    rw = np.ascontiguousarray(L["router_w"], np.float32)
    eb = _opt(L.get("e_bias"), np.float32)
    act = _opt(active, np.uint8)
    out = np.empty((n, H), np.float32)
    secs = ref().ref_moe_mlp_w4(_ptr(x), n, H, int(L["I"]), int(L["Is"]), int(L["E"]), int(L["topk"]),
                                int(L["group"]), _ptr(rw), _ptr(eb), int(bool(L["norm_topk"])),
                                C.c_double(L["routed_scale"]), *[_ptr(t) for t in a], _ptr(act),
                                _ptr(out))
    if secs < 0:
        raise RuntimeError("reference moe_mlp failed (an inactive expert was routed to?)")
    return out, float(secs)


class RefLayer:
    """The reference's MoE layer with fp32 weights dequantised once (as after its load);
    ``run`` calls GLM52Model::moe_mlp and returns (out, seconds inside moe_mlp)."""

    def __init__(self, L, active=None):
        a = _wargs(L)
        rw = np.ascontiguousarray(L["router_w"], np.float32)
        eb = _opt(L.get("e_bias"), np.float32)
        act = _opt(active, np.uint8)
        self.H = int(L["H"])
        self._h = ref().ref_moe_create(self.H, int(L["I"]), int(L["Is"]), int(L["E"]), int(L["topk"]),
                                       int(L["group"]), _ptr(rw), _ptr(eb), int(bool(L["norm_topk"])),
                                       C.c_double(L["routed_scale"]), *[_ptr(t) for t in a], _ptr(act))
        if not self._h:
            raise RuntimeError("reference layer construction failed")

    def run(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty((x.shape[0], self.H), np.float32)
        secs = ref().ref_moe_run(self._h, _ptr(x), x.shape[0], _ptr(out))
        if secs < 0:
            raise RuntimeError("reference moe_mlp failed (an inactive expert was routed to?)")
        return out, float(secs)

    def close(self):
        if self._h:
            ref().ref_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()
