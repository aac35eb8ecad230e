"""Host-side mirror of the reference's operator surface (cuda/kernels.cuh, namespace
glmserve::cuda) on top of the C ABI.  Same names, argument meaning and error behaviour:
the reference's wrappers return nothing and leave errors to the caller's later check; here
a non-zero status from the C ABI raises ``GsbError`` at the call.  Tensors are torch CUDA
tensors used only as device buffers; every call runs on torch's current stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import MoeConfig, check, lib

PATH_AUTO, PATH_DIRECT, PATH_DECODE, PATH_PREFILL, PATH_DECODE_SMEM = 0, 1, 2, 3, 4


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, dtype, name):
    if t is None:
        return
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous CUDA tensor of {dtype}")


def moe_router(logits, e_bias, topk, norm_topk=True, routed_scale=2.5):
    """cuda/kernels.cuh:243 moe_router.  Returns (topk_ids int32 [n,topk], topk_w f32)."""
    _need(logits, torch.float32, "logits"); _need(e_bias, torch.float32, "e_bias")
    n, E = logits.shape
    ids = torch.empty((n, topk), dtype=torch.int32, device=logits.device)
    w = torch.empty((n, topk), dtype=torch.float32, device=logits.device)
    check(lib().gsb_moe_router(_p(logits), _p(e_bias), n, E, topk, int(bool(norm_topk)),
                               C.c_float(routed_scale), _p(ids), _p(w), _stream()), "moe_router")
    return ids, w


def moe_dispatch_ws(topk_ids, E):
    """moe_dispatch with scratch: the many-block form above 8192 slots (same permutation)."""
    _need(topk_ids, torch.int32, "topk_ids")
    n, topk = topk_ids.shape
    dev = topk_ids.device
    offs = torch.empty(E + 1, dtype=torch.int32, device=dev)
    tok = torch.empty(n * topk, dtype=torch.int32, device=dev)
    row = torch.empty(n * topk, dtype=torch.int32, device=dev)
    lib().gsb_moe_dispatch_scratch_bytes.restype = C.c_size_t
    nb = int(lib().gsb_moe_dispatch_scratch_bytes(n, topk, E))
    scratch = torch.empty(max(nb, 4), dtype=torch.uint8, device=dev)
    check(lib().gsb_moe_dispatch_ws(_p(topk_ids), n, topk, E, _p(offs), _p(tok), _p(row), _p(scratch),
                                    C.c_size_t(scratch.numel()), _stream()), "moe_dispatch_ws")
    return offs, tok, row


def moe_dispatch(topk_ids, E):
    """cuda/kernels.cuh:249 moe_dispatch.  Returns (expert_offsets [E+1], sorted_token_ids,
    sorted_row), all int32."""
    _need(topk_ids, torch.int32, "topk_ids")
    n, topk = topk_ids.shape
    dev = topk_ids.device
    offs = torch.empty(E + 1, dtype=torch.int32, device=dev)
    tok = torch.empty(n * topk, dtype=torch.int32, device=dev)
    row = torch.empty(n * topk, dtype=torch.int32, device=dev)
    check(lib().gsb_moe_dispatch(_p(topk_ids), n, topk, E, _p(offs), _p(tok), _p(row), _stream()),
          "moe_dispatch")
    return offs, tok, row


def moe_expert_ffn_w4a16(x, topk_ids, topk_w, gate_q, gate_sc, up_q, up_sc, down_q, down_sc, group):
    """cuda/kernels.cuh:259 moe_expert_ffn_w4a16 (fp32 activations and scales)."""
    for t, d, nm in ((x, torch.float32, "x"), (topk_ids, torch.int32, "ids"), (topk_w, torch.float32, "w"),
                     (gate_q, torch.uint8, "gate_q"), (gate_sc, torch.float32, "gate_sc"),
                     (up_q, torch.uint8, "up_q"), (up_sc, torch.float32, "up_sc"),
                     (down_q, torch.uint8, "down_q"), (down_sc, torch.float32, "down_sc")):
        _need(t, d, nm)
    n, H = x.shape
    E, I = gate_q.shape[0], gate_q.shape[1]
    out = torch.empty((n, H), dtype=torch.float32, device=x.device)
    check(lib().gsb_moe_expert_ffn_w4a16(_p(x), _p(topk_ids), _p(topk_w), _p(gate_q), _p(gate_sc),
                                         _p(up_q), _p(up_sc), _p(down_q), _p(down_sc), n,
                                         topk_ids.shape[1], H, I, E, group, _p(out), _stream()),
          "moe_expert_ffn_w4a16")
    return out


def moe_expert_ffn(x, topk_ids, topk_w, gate_w, up_w, down_w):
    """cuda/kernels.cuh:254 moe_expert_ffn (fp32 weights)."""
    for t, nm in ((x, "x"), (topk_w, "w"), (gate_w, "gate_w"), (up_w, "up_w"), (down_w, "down_w")):
        _need(t, torch.float32, nm)
    _need(topk_ids, torch.int32, "ids")
    n, H = x.shape
    E, I = gate_w.shape[0], gate_w.shape[1]
    out = torch.empty((n, H), dtype=torch.float32, device=x.device)
    check(lib().gsb_moe_expert_ffn(_p(x), _p(topk_ids), _p(topk_w), _p(gate_w), _p(up_w), _p(down_w), n,
                                   topk_ids.shape[1], H, I, E, _p(out), _stream()), "moe_expert_ffn")
    return out


def gemm_w4a16(x, qW, scales, group, bias=None):
    """cuda/kernels.cuh:48 gemm_w4a16: y[n,out] = x W^T (+ bias)."""
    _need(x, torch.float32, "x"); _need(qW, torch.uint8, "qW"); _need(scales, torch.float32, "scales")
    _need(bias, torch.float32, "bias")
    n, inn = x.shape
    out = qW.shape[0]
    y = torch.empty((n, out), dtype=torch.float32, device=x.device)
    check(lib().gsb_gemm_w4a16(_p(x), _p(qW), _p(scales), _p(bias), _p(y), C.c_int64(n), C.c_int64(inn),
                               C.c_int64(out), C.c_int64(group), _stream()), "gemm_w4a16")
    return y


def operator_cache_enable(max_weight_bytes: int) -> None:
    """Fast path behind moe_expert_ffn_w4a16 / gemm_w4a16 called with the reference's signatures: weights are
    repacked once per set of pointers and the tile-stream kernels run (0 = off, frees everything)."""
    check(lib().gsb_operator_cache_enable(C.c_size_t(max_weight_bytes)), "operator_cache_enable")


def operator_cache_bytes() -> int:
    lib().gsb_operator_cache_bytes.restype = C.c_size_t
    return int(lib().gsb_operator_cache_bytes())


def silu_mul(g, u):
    out = torch.empty_like(g)
    check(lib().gsb_silu_mul(_p(g), _p(u), _p(out), C.c_int64(g.numel()), _stream()), "silu_mul")
    return out


def add_inplace(y, x):
    check(lib().gsb_add_inplace(_p(y), _p(x), C.c_int64(y.numel()), _stream()), "add_inplace")
    return y


def rmsnorm(x, w, eps):
    _need(x, torch.float32, "x"); _need(w, torch.float32, "w")
    out = torch.empty_like(x)
    check(lib().gsb_rmsnorm(_p(x), _p(w), _p(out), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]),
                            C.c_float(eps), _stream()), "rmsnorm")
    return out


def quantize_act_q8(x):
    """cuda/kernels.cuh:77 quantize_act_q8: returns (xq int8 [n,in], xs f32 [n,in/32])."""
    _need(x, torch.float32, "x")
    n, inn = x.shape
    xq = torch.empty((n, inn), dtype=torch.int8, device=x.device)
    xs = torch.empty((n, inn // 32), dtype=torch.float32, device=x.device)
    check(lib().gsb_quantize_act_q8(_p(x), C.c_int64(n), C.c_int64(inn), _p(xq), _p(xs), _stream()),
          "quantize_act_q8")
    return xq, xs


def router_logits(x_bf16, router_w_bf16):
    _need(x_bf16, torch.bfloat16, "x"); _need(router_w_bf16, torch.bfloat16, "router_w")
    n, H = x_bf16.shape
    E = router_w_bf16.shape[0]
    logits = torch.empty((n, E), dtype=torch.float32, device=x_bf16.device)
    check(lib().gsb_router_logits(_p(x_bf16), _p(router_w_bf16), n, H, E, _p(logits), _stream()),
          "router_logits")
    return logits


def prepack_gate_up(gate_q, gate_sc, up_q, up_sc, group=128):
    """One-time repack of [E, I, H/2] gate and up tensors into the tile stream."""
    if gate_q.dim() == 2:
        gate_q, gate_sc, up_q, up_sc = (t.unsqueeze(0) for t in (gate_q, gate_sc, up_q, up_sc))
    E, I, hb = gate_q.shape
    H = hb * 2
    nbytes = lib().gsb_prepack_bytes(E, 2 * I, H)
    if nbytes == 0:
        raise ValueError("shape not supported by the tile stream (needs I % 16 == 0, H % 512 == 0)")
    out = torch.empty(nbytes, dtype=torch.uint8, device=gate_q.device)
    f32 = int(gate_sc.dtype == torch.float32)
    check(lib().gsb_prepack_gate_up(_p(gate_q.contiguous()), _p(gate_sc.contiguous()), _p(up_q.contiguous()),
                                    _p(up_sc.contiguous()), f32, E, I, H, group, _p(out), _stream()),
          "prepack_gate_up")
    return out


def prepack_down(down_q, down_sc, group=128):
    if down_q.dim() == 2:
        down_q, down_sc = down_q.unsqueeze(0), down_sc.unsqueeze(0)
    E, H, ib = down_q.shape
    I = ib * 2
    nbytes = lib().gsb_prepack_bytes(E, H, I)
    if nbytes == 0:
        raise ValueError("shape not supported by the tile stream (needs H % 32 == 0, I % 512 == 0)")
    out = torch.empty(nbytes, dtype=torch.uint8, device=down_q.device)
    f32 = int(down_sc.dtype == torch.float32)
    check(lib().gsb_prepack_down(_p(down_q.contiguous()), _p(down_sc.contiguous()), f32, E, H, I, group,
                                 _p(out), _stream()), "prepack_down")
    return out


class MoELayer:
    """One MoE layer resident on the current GPU: the native whole-layer entry point.

    ``L`` is a layer dict of torch CUDA tensors (see glmserve_b200.synth).  With
    ``prepack=True`` (default when the shapes allow) the int4 tensors are repacked once into
    the tile stream and ``keep_raw=False`` drops the raw copies, like an engine would after
    upload.
    """

    def __init__(self, L: dict, prepack: bool | None = None, keep_raw: bool = True, share_from=None,
                 fixed_routing: bool = False):
        """``share_from``: another MoELayer over the same weight tensors whose prepacked
        streams are reused (only router weight / bias / flags are taken from ``L``)."""
        self.H, self.E, self.topk, self.I, self.Is, self.group = (int(L[k]) for k in
                                                                   ("H", "E", "topk", "I", "Is", "group"))
        shared = L.get("sg_q") is not None
        # input dims of the down matrices as given (larger than I / Is when a tensor-parallel shard padded them)
        self.Id = int(L.get("Id") or self.I)
        self.Isd = int(L.get("Isd") or self.Is)
        can_pack = self.group == 128 and self.H % 512 == 0 and self.I % 64 == 0 and self.Id % 512 == 0 and \
            (not shared or (self.Is % 64 == 0 and self.Isd % 512 == 0))
        if prepack is None:
            prepack = can_pack
        if prepack and not can_pack:
            raise ValueError("these shapes cannot use the tile-stream kernels")
        self._keep = {}
        cfg = MoeConfig()
        cfg.hidden, cfg.n_experts, cfg.topk, cfg.moe_inter = self.H, self.E, self.topk, self.I
        cfg.shared_inter = self.Is if shared else 0
        cfg.group, cfg.norm_topk, cfg.routed_scale = self.group, int(bool(L["norm_topk"])), float(L["routed_scale"])
        self.ep_rank, self.ep_size = L.get("ep", (0, 1))
        cfg.ep_rank, cfg.ep_size = self.ep_rank, self.ep_size

        def hold(name, t):
            self._keep[name] = t
            return t.data_ptr()

        cfg.fixed_routing = int(fixed_routing)
        cfg.down_inter = self.Id if self.Id != self.I else 0
        cfg.shared_down_inter = self.Isd if (shared and self.Isd != self.Is) else 0
        if not fixed_routing:
            cfg.router_w = hold("router_w", L["router_w"].to(torch.bfloat16).contiguous())
        if L.get("e_bias") is not None:
            cfg.e_bias = hold("e_bias", L["e_bias"].float().contiguous())
        names = ["gate", "up", "down"] + (["sg", "su", "sd"] if shared else [])
        if prepack and share_from is not None:
            for nm, fld in (("gup", "gate_up_packed"), ("dp", "down_packed"), ("sgup", "shared_gate_up_packed"),
                            ("sdp", "shared_down_packed")):
                if nm in share_from._keep:
                    setattr(cfg, fld, hold(nm, share_from._keep[nm]))
        elif prepack:
            cfg.gate_up_packed = hold("gup", prepack_gate_up(L["gate_q"], L["gate_sc"], L["up_q"], L["up_sc"]))
            cfg.down_packed = hold("dp", prepack_down(L["down_q"], L["down_sc"]))
            if shared:
                cfg.shared_gate_up_packed = hold("sgup", prepack_gate_up(L["sg_q"], L["sg_sc"], L["su_q"], L["su_sc"]))
                cfg.shared_down_packed = hold("sdp", prepack_down(L["sd_q"], L["sd_sc"]))
        if (keep_raw and share_from is None) or not prepack:
            for nm in names:
                setattr(cfg, nm + "_q", hold(nm + "_q", L[nm + "_q"].contiguous()))
                setattr(cfg, nm + "_sc", hold(nm + "_sc", L[nm + "_sc"].to(torch.float16).contiguous()))
        self.cfg = cfg
        self.prepacked = bool(prepack)
        handle = C.c_void_p()
        check(lib().gsb_moe_layer_create(C.byref(cfg), C.byref(handle)), "moe_layer_create")
        self._h = handle
        self._ws = None
        self._ws_n = -1
        self.device = L["gate_q"].device if L.get("gate_q") is not None else L["router_w"].device

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib().gsb_moe_layer_destroy(h)
            self._h = None

    def workspace_bytes(self, n: int) -> int:
        return int(lib().gsb_moe_workspace_bytes(self._h, n))

    def _workspace(self, n: int):
        if self._ws is None or n > self._ws_n:
            self._ws = torch.zeros(self.workspace_bytes(n) + 256, dtype=torch.uint8, device=self.device)
            self._ws_n = n
        return self._ws

    def forward(self, x_bf16, out=None, path=PATH_AUTO, return_routing=False):
        """x bf16 [n,H] -> out f32 [n,H] (overwritten).  Asynchronous on the current stream."""
        _need(x_bf16, torch.bfloat16, "x")
        n = x_bf16.shape[0]
        if out is None:
            out = torch.empty((n, self.H), dtype=torch.float32, device=x_bf16.device)
        ws = self._workspace(n)
        logits = ids = w = None
        if return_routing:
            logits = torch.empty((n, self.E), dtype=torch.float32, device=x_bf16.device)
            ids = torch.empty((n, self.topk), dtype=torch.int32, device=x_bf16.device)
            w = torch.empty((n, self.topk), dtype=torch.float32, device=x_bf16.device)
        check(lib().gsb_moe_layer_forward(self._h, _p(x_bf16), n, _p(out), _p(ws), C.c_size_t(ws.numel()),
                                          path, _p(logits), _p(ids), _p(w), _stream()), "moe_layer_forward")
        return (out, logits, ids, w) if return_routing else out

    def block_forward(self, hidden_f32, norm_w, eps=1e-5, path=PATH_AUTO, ids_out=None):
        """hidden <- hidden + moe(rmsnorm(hidden)) in place (f32 [n,H])."""
        _need(hidden_f32, torch.float32, "hidden"); _need(norm_w, torch.float32, "norm_w")
        n = hidden_f32.shape[0]
        ws = self._workspace(n)
        check(lib().gsb_moe_block_layer_forward(self._h, _p(hidden_f32), _p(norm_w), C.c_float(eps), n,
                                                _p(ws), C.c_size_t(ws.numel()), path, _p(ids_out), _stream()),
              "moe_block_layer_forward")
        return hidden_f32

    def forward_ep(self, comm, x_bf16, out=None, recv_cap=None, heap_offset=None, ids_out=None, path=PATH_AUTO):
        """Expert-parallel forward over the communicator's ranks (this layer holds the experts
        of rank ``comm.rank``).  x bf16 [n,H] = this GPU's tokens -> out f32 [n,H].  ``path``: the
        tcgen05 kernels, the split-K kernels, or AUTO (by ``recv_cap``); the same on every rank.
        Without ``recv_cap`` the ranks agree on the largest n (one small all-reduce on the host)."""
        _need(x_bf16, torch.bfloat16, "x")
        n = x_bf16.shape[0]
        if out is None:
            out = torch.empty((n, self.H), dtype=torch.float32, device=x_bf16.device)
        if recv_cap is None:
            recv_cap = comm.max_over_ranks(n) * self.topk * self.ep_size
        if heap_offset is None:
            heap_offset = (comm.reserved + 1023) // 1024 * 1024
        need = int(lib().gsb_moe_ep_workspace_bytes(self._h, n, recv_cap))
        if getattr(self, "_ep_ws", None) is None or self._ep_ws.numel() < need + 256:
            self._ep_ws = torch.zeros(need + 256, dtype=torch.uint8, device=self.device)
        check(lib().gsb_moe_layer_forward_ep(self._h, comm._h, _p(x_bf16), n, _p(out), _p(self._ep_ws),
                                             C.c_size_t(self._ep_ws.numel()), C.c_size_t(heap_offset), recv_cap,
                                             path, _p(ids_out), _stream()), "moe_layer_forward_ep")
        return out

    def block_forward_ep(self, comm, hidden_f32, norm_w, eps=1e-5, recv_cap=None, heap_offset=None, ids_out=None,
                         path=PATH_AUTO):
        """hidden <- hidden + moe(rmsnorm(hidden)) in place over the communicator's ranks (f32 [n,H] = this
        GPU's tokens): ``forward_ep`` with the pre-norm inside the router-logits launch and the residual add
        inside the combine."""
        _need(hidden_f32, torch.float32, "hidden"); _need(norm_w, torch.float32, "norm_w")
        n = hidden_f32.shape[0]
        if recv_cap is None:
            recv_cap = comm.max_over_ranks(n) * self.topk * self.ep_size
        if heap_offset is None:
            heap_offset = (comm.reserved + 1023) // 1024 * 1024
        need = int(lib().gsb_moe_ep_workspace_bytes(self._h, n, recv_cap))
        if getattr(self, "_ep_ws", None) is None or self._ep_ws.numel() < need + 256:
            self._ep_ws = torch.zeros(need + 256, dtype=torch.uint8, device=self.device)
        check(lib().gsb_moe_block_layer_forward_ep(self._h, comm._h, _p(hidden_f32), _p(norm_w), C.c_float(eps), n,
                                                   _p(self._ep_ws), C.c_size_t(self._ep_ws.numel()),
                                                   C.c_size_t(heap_offset), recv_cap, path, _p(ids_out), _stream()),
              "moe_block_layer_forward_ep")
        return hidden_f32

    def ep_heap_bytes(self, n: int, recv_cap: int) -> int:
        return int(lib().gsb_moe_ep_heap_bytes(self._h, n, recv_cap))

    def status(self) -> int:
        """After a stream synchronise: 0, or 4 when a bounded device wait gave up."""
        torch.cuda.current_stream().synchronize()
        return int(lib().gsb_moe_layer_status(self._h, _p(self._ws))) if self._ws is not None else 0

    def forward_host(self, x_host, out_host, path=PATH_AUTO):
        """The call an engine with host-resident activations makes: pinned host bf16 [n,H] in,
        pinned host f32 [n,H] out; copies ride the current stream around the layer."""
        n = x_host.shape[0]
        if getattr(self, "_hx", None) is None or self._hx.shape[0] < n:
            self._hx = torch.empty((n, self.H), dtype=torch.bfloat16, device=self.device)
            self._ho = torch.empty((n, self.H), dtype=torch.float32, device=self.device)
        xd, od = self._hx[:n], self._ho[:n]
        xd.copy_(x_host, non_blocking=True)
        self.forward(xd, out=od, path=path)
        out_host.copy_(od, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host


STAGES = ("moe.router", "moe.dispatch", "moe.gate_up", "moe.down", "moe.combine")
# the same five marks of an expert-parallel forward: routing + count exchange + plan (the push is launched on
# a side stream), the shared expert on local tokens, waiting for the peers' rows, the routed GEMMs (the down
# kernel stores to the tokens' home GPUs), waiting for the returned rows + combine
EP_STAGES = ("ep.route_plan", "ep.shared", "ep.wait_rows", "ep.routed_gemms", "ep.return_combine")


class DenseMLP:
    """A dense W4A16 SwiGLU MLP (the model's first, non-MoE layers: gate/up ``[I, H]``, down
    ``[H, I]``, src/model_gpu.cpp:1432-1445) on the grouped MoE kernels.  SwiGLU is elementwise
    over the intermediate dim, so ``down(silu(gate x) * up x)`` is the sum over slices of I of the
    same expression on the slice: the I columns are cut into ``I / slice`` experts that every
    token visits with weight 1 (``fixed_routing``), and the combine adds the slices in order.

    gate_q/up_q uint8 ``[I, H/2]``, down_q uint8 ``[H, I/2]``, scales ``[rows, cols/128]``."""

    def __init__(self, gate_q, gate_sc, up_q, up_sc, down_q, down_sc, slice_cols: int = 2048):
        I, hb = gate_q.shape
        H = hb * 2
        if I % slice_cols:
            slice_cols = I
        E = I // slice_cols
        gs = slice_cols // 128
        L = dict(H=H, E=E, topk=E, I=slice_cols, Is=0, group=128, norm_topk=False, routed_scale=1.0,
                 router_w=None, e_bias=None,
                 gate_q=gate_q.reshape(E, slice_cols, hb), gate_sc=gate_sc.reshape(E, slice_cols, -1),
                 up_q=up_q.reshape(E, slice_cols, hb), up_sc=up_sc.reshape(E, slice_cols, -1),
                 down_q=down_q.reshape(H, E, slice_cols // 2).permute(1, 0, 2).contiguous(),
                 down_sc=down_sc.reshape(H, E, gs).permute(1, 0, 2).contiguous())
        self.layer = MoELayer(L, keep_raw=False, fixed_routing=True)
        self.H, self.I = H, I

    def forward(self, x_bf16, out=None, path=PATH_AUTO):
        return self.layer.forward(x_bf16, out=out, path=path)


def profile_enable(layer: MoELayer, max_forwards: int) -> None:
    check(lib().gsb_moe_layer_profile_enable(layer._h, max_forwards), "profile_enable")


def profile_read(layer: MoELayer, names=STAGES) -> dict:
    """Average stage times (ms) of the forwards since the last read; sync first."""
    torch.cuda.current_stream().synchronize()
    ms = (C.c_float * len(STAGES))()
    n = C.c_int(0)
    check(lib().gsb_moe_layer_profile_read(layer._h, ms, C.byref(n)), "profile_read")
    return dict(forwards=n.value, **{k: float(ms[i]) for i, k in enumerate(names)})
