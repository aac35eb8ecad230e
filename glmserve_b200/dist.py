"""One process per GPU: the NVLink peer-memory communicator of the C ABI (gsb_comm_*), driven
through torch.distributed only for the one-time exchange of IPC handles.  Also host mirrors
of the expert-parallel plan and of the tensor-parallel shard rule, used by the CPU tests.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib


class Comm:
    """Symmetric heap + flags over all ranks of the default process group (one box).

    ``loopback_world``: no process group at all - a single-process communicator of that many
    "ranks" whose peer slots all map this rank's own heap.  Nothing ever posts the peers' flags, so
    every device-side wait runs out: the way the bounded waits are tested on one GPU."""

    def __init__(self, heap_bytes: int, allreduce_max_count: int = 0, loopback_world: int = 0):
        import torch
        if loopback_world:
            self.rank, self.world = 0, loopback_world
            self._dist = None
        else:
            import torch.distributed as dist
            self._dist = dist
            self.rank, self.world = dist.get_rank(), dist.get_world_size()
        hb = lib().gsb_comm_handle_bytes()
        handle = (C.c_ubyte * hb)()
        h = C.c_void_p()
        check(lib().gsb_comm_create(self.rank, self.world, C.c_size_t(heap_bytes), handle, C.byref(h)), "comm_create")
        self._h = h
        self._dev = torch.device("cuda", torch.cuda.current_device())
        if loopback_world:
            check(lib().gsb_comm_open_loopback(self._h), "comm_open_loopback")
        else:
            dist, dev = self._dist, self._dev
            mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=dev)
            allh = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(allh, mine)
            buf = b"".join(bytes(t.cpu().numpy().tobytes()) for t in allh)
            self._handles = (C.c_ubyte * len(buf)).from_buffer_copy(buf)
            st = lib().gsb_comm_open(self._h, self._handles)
            ok = torch.tensor([1 if st == 0 else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)          # all-or-none, like the reference's bring-up
            if int(ok) == 0:
                self.close()
                raise RuntimeError("peer memory could not be opened on every rank")
        self.reserved = int(lib().gsb_comm_allreduce_reserve(self._h, C.c_int64(allreduce_max_count)))
        if not loopback_world:
            self._dist.barrier()

    @staticmethod
    def reserve_bytes(world: int, allreduce_max_count: int) -> int:
        """Bytes at the start of the heap the all-reduce takes: add them when sizing ``heap_bytes``."""
        lib().gsb_comm_allreduce_reserve_bytes.restype = C.c_size_t
        return int(lib().gsb_comm_allreduce_reserve_bytes(int(world), C.c_int64(allreduce_max_count)))

    def set_wait_cycles(self, cycles: int) -> None:
        """Budget of every device-side wait in SM clock cycles (0 = default, about two seconds)."""
        check(lib().gsb_comm_set_wait_cycles(self._h, C.c_longlong(cycles)), "comm_set_wait_cycles")

    def max_over_ranks(self, value: int) -> int:
        """Host-side agreement on the largest ``value`` over the ranks (a small all-reduce)."""
        if self._dist is None:
            return int(value)
        import torch
        t = torch.tensor([int(value)], device=self._dev)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX)
        return int(t)

    def heap_bytes(self) -> int:
        return int(lib().gsb_comm_heap_bytes(self._h))

    def allreduce_one_shot_limit(self, total_floats: int) -> None:
        """count * world up to which the all-reduce is a one-shot pull (0 = default 2**21)."""
        check(lib().gsb_comm_allreduce_one_shot_limit(self._h, C.c_int64(total_floats)), "allreduce_one_shot_limit")

    def allreduce_ll_limit(self, floats: int) -> None:
        """Messages up to ``floats`` floats take the flag-in-data form (0 = default 65536, 1 = off)."""
        check(lib().gsb_comm_allreduce_ll_limit(self._h, C.c_int64(floats)), "allreduce_ll_limit")

    def allreduce_sum(self, t):
        """In-place sum of a contiguous float32 CUDA tensor over all ranks (rank order)."""
        import torch
        assert t.dtype == torch.float32 and t.is_contiguous() and t.is_cuda
        check(lib().gsb_comm_allreduce_sum(self._h, C.c_void_p(t.data_ptr()), C.c_int64(t.numel()),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream)), "allreduce_sum")
        return t

    def allreduce_sum_n(self, t, n: int):
        """``n`` in-place sums launched from one host call (timing aid: no per-call host cost in between)."""
        import torch
        assert t.dtype == torch.float32 and t.is_contiguous() and t.is_cuda
        check(lib().gsb_comm_allreduce_sum_n(self._h, C.c_void_p(t.data_ptr()), C.c_int64(t.numel()), int(n),
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream)), "comm_allreduce_sum_n")
        return t

    def allreduce_sum_rows(self, t):
        """Row-by-row form (include/nccl_comm.hpp:53-59 of the reference); same bits as one call."""
        for r in range(t.shape[0]):
            self.allreduce_sum(t[r])
        return t

    def barrier(self):
        import torch
        check(lib().gsb_comm_barrier(self._h, C.c_void_p(torch.cuda.current_stream().cuda_stream)), "comm_barrier")

    def status(self) -> int:
        import torch
        torch.cuda.current_stream().synchronize()
        return int(lib().gsb_comm_status(self._h))

    def close(self):
        if getattr(self, "_h", None):
            lib().gsb_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


class PeerLost(RuntimeError):
    """A rank did not reach a step that its peers reached."""


class StepGuard:
    """Host-side liveness check between steps.  The device-side waits of the collectives are bounded,
    but a rank that has left (crashed, exited, never joined) should be noticed BEFORE its peers launch
    kernels that wait for it.  Every rank posts "I am about to run step s" in a key-value store
    (``torch.distributed.TCPStore`` or anything with ``set`` / ``wait(keys, timeout)``) and waits a short
    time for the others; a missing post raises ``PeerLost`` naming the rank, and the caller stops
    launching instead of running into timeouts on the GPU.  A rank leaves only between steps."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s

    def enter(self, step: int) -> None:
        import datetime
        self.store.set(f"gsb/step/{step}/{self.rank}", "1")
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                self.store.wait([f"gsb/step/{step}/{r}"], datetime.timedelta(seconds=self.timeout_s))
            except Exception as e:  # the store raises its own timeout type
                raise PeerLost(f"rank {r} did not reach step {step} within {self.timeout_s} s") from e


# ---- host mirrors (numpy) ------------------------------------------------------------------

def ep_plan_np(cnt: np.ndarray, rank: int, recv_cap: int | None = None):
    """Mirror of ep_plan_kernel.  cnt[src, e] = rows rank `src` routes to expert e.
    Returns (recv_offsets[El+1], send_base[E], src_pos[world, E]): the receive layout of `rank`
    (local expert major, then source rank), where this rank's rows for expert e start on the
    owner's receive buffer, and where expert e's rows start in each source's sorted order.
    With ``recv_cap`` the receive offsets are clamped to it, as the kernel does on overflow: no
    tile, intermediate row or output pointer index can then lie beyond the capacity (senders drop
    rows whose destination row is not below the OWNER's capacity)."""
    world, E = cnt.shape
    El = E // world
    tot = cnt.sum(axis=0)
    base = np.zeros(E, np.int64)
    for o in range(world):
        base[o * El:(o + 1) * El] = np.concatenate([[0], np.cumsum(tot[o * El:(o + 1) * El])[:-1]])
    send_base = base + cnt[:rank].sum(axis=0)
    recv_offsets = np.concatenate([base[rank * El:(rank + 1) * El], [base[(rank + 1) * El - 1] + tot[(rank + 1) * El - 1]]])
    src_pos = np.concatenate([np.zeros((world, 1), np.int64), np.cumsum(cnt, axis=1)[:, :-1]], axis=1)
    if recv_cap is not None:
        recv_offsets = np.minimum(recv_offsets, recv_cap)
    return recv_offsets.astype(np.int64), send_base.astype(np.int64), src_pos


def shard_layer_tp(L: dict, rank: int, tp: int, pad_to: int = 0, pad_down_to: int = 0) -> dict:
    """Tensor-parallel shard of a numpy layer dict, the reference's rule
    (src/model_glm52.cpp:314-422): gate/up split on their output rows (intermediate dim),
    down on its input columns - contiguous, group-aligned slices; router replicated.
    ``pad_down_to``: only the down matrices' input columns are padded with zero weights (nibble 8,
    scale 1) up to a multiple of it, so that a slice narrower than the tile stream's 512-column
    chunk can be packed; the result carries ``Id`` / ``Isd`` (the padded dims) next to the true
    ``I`` / ``Is``, and gate/up keep their true size.  ``pad_to`` pads gate/up rows as well (twice
    the bytes of what is needed; kept for comparison)."""
    g = int(L["group"])
    out = dict(L)

    def split(name_g, name_u, name_d, I):
        assert I % tp == 0 and (I // tp) % g == 0, "slice must be group aligned"
        Il = I // tp
        r0, r1 = rank * Il, (rank + 1) * Il
        if pad_down_to and not pad_to:
            Ipd = (Il + pad_down_to - 1) // pad_down_to * pad_down_to
            res = {}
            for nm in (name_g, name_u):
                res[nm + "_q"] = np.ascontiguousarray(L[nm + "_q"][..., r0:r1, :])
                res[nm + "_sc"] = np.ascontiguousarray(L[nm + "_sc"][..., r0:r1, :])
            q, sc = L[name_d + "_q"][..., r0 // 2:r1 // 2], L[name_d + "_sc"][..., r0 // g:r1 // g]
            if Ipd > Il:
                padq = np.full(q.shape[:-1] + ((Ipd - Il) // 2,), 0x88, np.uint8)
                pads = np.ones(sc.shape[:-1] + ((Ipd - Il) // g,), np.float32)
                q, sc = np.concatenate([q, padq], axis=-1), np.concatenate([sc, pads], axis=-1)
            res[name_d + "_q"], res[name_d + "_sc"] = np.ascontiguousarray(q), np.ascontiguousarray(sc)
            return res, (Il, Ipd)
        Ip = ((Il + pad_to - 1) // pad_to * pad_to) if pad_to else Il
        res = {}
        for nm in (name_g, name_u):
            q, sc = L[nm + "_q"][..., r0:r1, :], L[nm + "_sc"][..., r0:r1, :]
            if Ip > Il:
                padq = np.full(q.shape[:-2] + (Ip - Il, q.shape[-1]), 0x88, np.uint8)
                pads = np.ones(sc.shape[:-2] + (Ip - Il, sc.shape[-1]), np.float32)
                q, sc = np.concatenate([q, padq], axis=-2), np.concatenate([sc, pads], axis=-2)
            res[nm + "_q"], res[nm + "_sc"] = np.ascontiguousarray(q), np.ascontiguousarray(sc)
        q, sc = L[name_d + "_q"][..., r0 // 2:r1 // 2], L[name_d + "_sc"][..., r0 // g:r1 // g]
        if Ip > Il:
            padq = np.full(q.shape[:-1] + ((Ip - Il) // 2,), 0x88, np.uint8)
            pads = np.ones(sc.shape[:-1] + ((Ip - Il) // g,), np.float32)
            q, sc = np.concatenate([q, padq], axis=-1), np.concatenate([sc, pads], axis=-1)
        res[name_d + "_q"], res[name_d + "_sc"] = np.ascontiguousarray(q), np.ascontiguousarray(sc)
        return res, Ip

    r, Ip = split("gate", "up", "down", int(L["I"]))
    out.update(r)
    if isinstance(Ip, tuple):
        out["I"], out["Id"] = Ip
    else:
        out["I"] = Ip
    if L.get("sg_q") is not None:
        r, Isp = split("sg", "su", "sd", int(L["Is"]))
        out.update(r)
        if isinstance(Isp, tuple):
            out["Is"], out["Isd"] = Isp
        else:
            out["Is"] = Isp
    return out


def shard_layer_ep(L: dict, rank: int, ep: int) -> dict:
    """Expert-parallel shard: experts [rank*E/ep, (rank+1)*E/ep) resident; router, bias and
    the shared expert replicated.  ``E`` stays the global count."""
    E = int(L["E"])
    El = E // ep
    out = dict(L)
    for nm in ("gate", "up", "down"):
        out[nm + "_q"] = L[nm + "_q"][rank * El:(rank + 1) * El]
        out[nm + "_sc"] = L[nm + "_sc"][rank * El:(rank + 1) * El]
    out["ep"] = (rank, ep)
    return out


def shard_layer_tp_torch(L: dict, rank: int, tp: int, pad_to: int = 0, pad_down_to: int = 512) -> dict:
    """torch form of shard_layer_tp for layers generated on the GPU (scales fp16)."""
    import torch
    g = int(L["group"])
    out = dict(L)

    def split(ng, nu, nd, I):
        Il = I // tp
        assert I % tp == 0 and Il % g == 0
        r0, r1 = rank * Il, (rank + 1) * Il
        if pad_down_to and not pad_to:
            Ipd = (Il + pad_down_to - 1) // pad_down_to * pad_down_to
            res = {}
            for nm in (ng, nu):
                res[nm + "_q"], res[nm + "_sc"] = L[nm + "_q"][..., r0:r1, :].contiguous(), L[nm + "_sc"][..., r0:r1, :].contiguous()
            q, sc = L[nd + "_q"][..., r0 // 2:r1 // 2], L[nd + "_sc"][..., r0 // g:r1 // g]
            if Ipd > Il:
                q = torch.cat([q, torch.full(q.shape[:-1] + ((Ipd - Il) // 2,), 0x88, dtype=torch.uint8, device=q.device)], dim=-1)
                sc = torch.cat([sc, torch.ones(sc.shape[:-1] + ((Ipd - Il) // g,), dtype=sc.dtype, device=sc.device)], dim=-1)
            res[nd + "_q"], res[nd + "_sc"] = q.contiguous(), sc.contiguous()
            return res, (Il, Ipd)
        Ip = (Il + pad_to - 1) // pad_to * pad_to if pad_to else Il
        res = {}
        for nm in (ng, nu):
            q, sc = L[nm + "_q"][..., r0:r1, :], L[nm + "_sc"][..., r0:r1, :]
            if Ip > Il:
                q = torch.cat([q, torch.full(q.shape[:-2] + (Ip - Il, q.shape[-1]), 0x88, dtype=torch.uint8, device=q.device)], dim=-2)
                sc = torch.cat([sc, torch.ones(sc.shape[:-2] + (Ip - Il, sc.shape[-1]), dtype=sc.dtype, device=sc.device)], dim=-2)
            res[nm + "_q"], res[nm + "_sc"] = q.contiguous(), sc.contiguous()
        q, sc = L[nd + "_q"][..., r0 // 2:r1 // 2], L[nd + "_sc"][..., r0 // g:r1 // g]
        if Ip > Il:
            q = torch.cat([q, torch.full(q.shape[:-1] + ((Ip - Il) // 2,), 0x88, dtype=torch.uint8, device=q.device)], dim=-1)
            sc = torch.cat([sc, torch.ones(sc.shape[:-1] + ((Ip - Il) // g,), dtype=sc.dtype, device=sc.device)], dim=-1)
        res[nd + "_q"], res[nd + "_sc"] = q.contiguous(), sc.contiguous()
        return res, Ip

    r, Ip = split("gate", "up", "down", int(L["I"]))
    out.update(r)
    if isinstance(Ip, tuple):
        out["I"], out["Id"] = Ip
    else:
        out["I"] = Ip
    if L.get("sg_q") is not None:
        r, Isp = split("sg", "su", "sd", int(L["Is"]))
        out.update(r)
        if isinstance(Isp, tuple):
            out["Is"], out["Isd"] = Isp
        else:
            out["Is"] = Isp
    return out
