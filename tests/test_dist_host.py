"""Host-side logic of the multi-GPU paths on CPU: tensor-parallel shard rule, expert-parallel
plan (mirror of the device kernel) exercised by two gloo ranks exchanging real rows."""
import os
import socket

import numpy as np
import pytest

import oracle
from glmserve_b200.dist import ep_plan_np, shard_layer_ep, shard_layer_tp
from glmserve_b200.synth import CONFIGS, make_layer_np, make_x_np


def test_tp_shards_sum_to_the_full_layer():
    L = make_layer_np(CONFIGS["mid"], seed=3)
    x = make_x_np(10, L["H"], seed=4)
    full = oracle.moe_layer_w4(x, L)
    acc = np.zeros_like(full["out"])
    for r in range(2):
        Ls = shard_layer_tp(L, r, 2)
        assert Ls["I"] == L["I"] // 2 and Ls["down_q"].shape[-1] == L["I"] // 4
        part = oracle.moe_layer_w4(x, Ls, logits_in=full["logits"])
        assert np.array_equal(part["ids"], full["ids"])
        acc = acc + part["out"]
    np.testing.assert_allclose(acc, full["out"], rtol=0, atol=2e-5)


def test_tp_padding_adds_exact_zeros():
    L = make_layer_np(CONFIGS["mid"], seed=5)
    x = make_x_np(6, L["H"], seed=6)
    a = shard_layer_tp(L, 1, 4)              # I_local = 128
    b = shard_layer_tp(L, 1, 4, pad_to=512)  # padded to 512 with zero weights
    assert b["I"] == 512 and a["I"] == 128
    lo = oracle.moe_layer_w4(x, L)["logits"]
    assert np.array_equal(oracle.moe_layer_w4(x, a, logits_in=lo)["out"], oracle.moe_layer_w4(x, b, logits_in=lo)["out"])


def test_ep_plan_layout_is_consistent():
    rng = np.random.default_rng(0)
    world, E = 4, 16
    cnt = rng.integers(0, 7, size=(world, E))
    cnt[2] = 0                                   # a rank with no tokens
    plans = [ep_plan_np(cnt, r) for r in range(world)]
    El = E // world
    for owner in range(world):
        recv_off, _, _ = plans[owner]
        assert recv_off[-1] == cnt[:, owner * El:(owner + 1) * El].sum()
        # every (expert, source) block tiles the receive buffer without gaps or overlap
        covered = np.zeros(recv_off[-1], int)
        for e in range(owner * El, (owner + 1) * El):
            for s in range(world):
                b = plans[s][1][e]
                covered[b:b + cnt[s, e]] += 1
                assert b >= recv_off[e - owner * El] and b + cnt[s, e] <= recv_off[e - owner * El + 1]
        assert np.all(covered == 1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L = make_layer_np(CONFIGS["tiny"], seed=11)
        E, k, H = L["E"], L["topk"], L["H"]
        n = 9 + 4 * rank
        x = make_x_np(n, H, seed=20 + rank)
        full = oracle.moe_layer_w4(x, L)                       # what a single GPU would give
        offs, tok, row = oracle.dispatch(full["ids"], E)
        cnt_local = torch.from_numpy(np.diff(offs).astype(np.int64))
        allc = [torch.empty_like(cnt_local) for _ in range(world)]
        dist.all_gather(allc, cnt_local)
        cnt = np.stack([c.numpy() for c in allc])
        recv_off, send_base, src_pos = ep_plan_np(cnt, rank)
        El = E // world
        # dispatch: rows to their owners at the planned positions
        recv = np.zeros((int(recv_off[-1]), H), np.float32)
        sends = [[] for _ in range(world)]
        for e in range(E):
            rows = x[tok[offs[e]:offs[e + 1]]]
            sends[e // El].append((e, send_base[e], rows))
        gathered = [None] * world
        dist.all_gather_object(gathered, sends)
        for src in range(world):
            for e, base, rows in gathered[src][rank]:
                recv[base:base + len(rows)] = rows
        # local experts on the received rows (oracle arithmetic), outputs back to the sources
        Lloc = shard_layer_ep(L, rank, world)
        ids_loc = np.repeat(np.arange(El), np.diff(recv_off)).astype(np.int32)[:, None]
        Lone = dict(Lloc, E=El, topk=1, sg_q=None, sg_sc=None, su_q=None, su_sc=None, sd_q=None, sd_sc=None)
        y = oracle.moe_experts_w4(recv, ids_loc, np.ones_like(ids_loc, np.float32), Lone) if len(recv) else recv
        back = [[] for _ in range(world)]
        for el in range(El):
            e = rank * El + el
            r0 = recv_off[el]
            for s in range(world):
                back[s].append((int(src_pos[s][e]), y[r0:r0 + cnt[s, e]]))
                r0 += cnt[s, e]
        got_back = [None] * world
        dist.all_gather_object(got_back, back)
        ybuf = np.zeros((n * k, H), np.float32)
        for owner in range(world):
            for pos, rows in got_back[owner][rank]:
                ybuf[pos:pos + len(rows)] = rows
        # deterministic combine in slot order, shared expert last
        pos_of = np.empty(n * k, int)
        pos_of[tok * k + row] = np.arange(n * k)
        Lns = dict(L, sg_q=None, sg_sc=None, su_q=None, su_sc=None, sd_q=None, sd_sc=None)
        routed_only = oracle.moe_layer_w4(x, Lns, logits_in=full["logits"])["out"]
        out = np.zeros((n, H), np.float32)
        for t in range(n):
            for j in range(k):
                out[t] += full["w"][t, j] * ybuf[pos_of[t * k + j]]
        ok = np.array_equal(out, routed_only)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_ep_exchange_with_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=5) for _ in range(2))
    assert res == {0: True, 1: True}


def test_ep_plan_overflow_is_clamped_to_the_receive_capacity():
    """More rows than a rank can receive: the receive offsets stop at the capacity, so no tile, no row of
    the intermediate buffer and no output-pointer index derived from them lies beyond it, and the rows a
    sender keeps (destination row below the OWNER's capacity) all fall inside the clamped layout."""
    rng = np.random.default_rng(1)
    world, E = 4, 16
    El = E // world
    cnt = rng.integers(0, 40, size=(world, E))
    for owner in range(world):
        total = int(cnt[:, owner * El:(owner + 1) * El].sum())
        cap = total // 2
        recv_off, _, _ = ep_plan_np(cnt, owner, recv_cap=cap)
        assert recv_off[-1] == min(total, cap) and np.all(recv_off <= cap) and np.all(np.diff(recv_off) >= 0)
        full_off, _, _ = ep_plan_np(cnt, owner)
        for s in range(world):
            send_base = ep_plan_np(cnt, s)[1]
            for e in range(owner * El, (owner + 1) * El):
                kept = [r for r in range(send_base[e], send_base[e] + cnt[s, e]) if r < cap]
                # a kept row lies in its expert's clamped segment
                el = e - owner * El
                assert all(recv_off[el] <= r < max(recv_off[el + 1], recv_off[el]) or r >= recv_off[el + 1] for r in kept)
                assert all(r < cap for r in kept)
        # different ranks may size their buffers differently: the clamp is per owner
        assert full_off[-1] == total


def _guard_worker(rank, world, port, leave_after, q):
    import datetime

    import torch.distributed as dist
    from glmserve_b200.dist import PeerLost, StepGuard
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    guard = StepGuard(store, rank, world, timeout_s=2.0)
    done = 0
    try:
        for step in range(4):
            if rank == 1 and step == leave_after:
                q.put((rank, "left", done))      # leaves BETWEEN steps, nothing in flight
                return
            guard.enter(step)
            done += 1                            # a step's kernels would be launched here
        q.put((rank, "finished", done))
    except PeerLost as e:
        q.put((rank, "peer lost: " + str(e), done))
    finally:
        if rank == 0:
            import time
            time.sleep(0.5)                      # the store's server outlives the other rank's last request


def test_a_rank_that_leaves_between_steps_is_reported_not_waited_for():
    """Rank 1 leaves after two steps.  Rank 0 learns of it on the host before it launches step 2 (a
    short store wait), reports which rank is missing and stops - it does not run into the device-side
    timeouts of kernels that would wait for the missing peer."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_guard_worker, args=(r, 2, port, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    res = {r: (what, done) for r, what, done in (q.get(timeout=5) for _ in range(2))}
    assert res[1] == ("left", 2)
    assert res[0][0].startswith("peer lost: rank 1 did not reach step 2") and res[0][1] == 2
