"""Worker of tests/test_gpu_multi.py: one rank per GPU (launched by torch.distributed.run), any world
size the layer's 32 / 256 experts divide by (2, 4, 8).  Checks the NVLink all-reduce, the tensor-parallel
layer and the expert-parallel layer against single-GPU results and the CPU oracle, on the mid
configuration and at GLM scale.  Exits non-zero on the first failure."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from glmserve_b200 import ops  # noqa: E402
from glmserve_b200.dist import Comm, shard_layer_ep, shard_layer_tp, shard_layer_tp_torch  # noqa: E402
from glmserve_b200.synth import (CONFIGS, layer_to_np, layer_to_torch, make_layer_np, make_layer_torch,  # noqa: E402
                                 make_x_np, make_x_torch)
from helpers import assert_layer_close, bf16_tensor  # noqa: E402


def check_allreduce(comm, rank, world, dev):
    """Values, determinism, rows parity, one-shot and two-shot sizes."""
    for count in (4, 6144, 8 * 6144, 64 * 6144, 2048 * 1024 + 64):
        gen = torch.Generator(device=dev); gen.manual_seed(100 + rank)
        x = torch.randn(count, generator=gen, device=dev)
        allx = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(allx, x)
        want = torch.zeros_like(x)
        for r in range(world):
            want = want + allx[r]                       # rank order, like the kernel
        for rep in range(3):                            # both parities of the staging, and a reuse
            y = x.clone()
            comm.allreduce_sum(y)
            assert comm.status() == 0
            assert torch.equal(y, want), f"allreduce count={count} rep={rep}"
    # the algorithm switch changes no bit: the same message through both forms
    gen = torch.Generator(device=dev); gen.manual_seed(300 + rank)
    x = torch.randn(64 * 6144, generator=gen, device=dev)
    got = []
    for limit in (1 << 40, 1, 0):                       # one-shot, two-shot, default
        comm.allreduce_one_shot_limit(limit)
        y = x.clone()
        comm.allreduce_sum(y)
        assert comm.status() == 0
        got.append(y)
    assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[2]), "one-shot vs two-shot"
    # decode-sized messages: the flag-in-data form (default) against the flag forms, bit for bit
    for count in (4, 6144, 4 * 6144, 65536):
        gen = torch.Generator(device=dev); gen.manual_seed(500 + rank)
        x = torch.randn(count, generator=gen, device=dev)
        got = []
        for ll in (0, 1, 0):                                 # on, off, on again
            comm.allreduce_ll_limit(ll)
            for rep in range(3):                             # both parities of the slots, and a reuse
                y = x.clone()
                comm.allreduce_sum(y)
                assert comm.status() == 0
                got.append(y)
        assert all(torch.equal(g, got[0]) for g in got), f"flag-in-data all-reduce differs (count={count})"
    comm.allreduce_ll_limit(0)
    rows = torch.randn((5, 6144), generator=torch.Generator(device=dev).manual_seed(7 + rank), device=dev)
    a, b = rows.clone(), rows.clone()
    comm.allreduce_sum(a.view(-1))
    comm.allreduce_sum_rows(b)
    assert comm.status() == 0 and torch.equal(a, b), "rows parity"
    # back-to-back calls without a host sync in between (the staging parities alternate)
    z = torch.ones(6144, device=dev)
    for _ in range(20):
        comm.allreduce_sum(z)
    assert comm.status() == 0 and torch.equal(z, torch.full_like(z, float(world) ** 20))


def check_mid(comm, rank, world, dev):
    cfg = CONFIGS["mid"]
    n = 300
    # ---- tensor parallel: column-split gate/up, row-split down, all-reduce ----
    L = make_layer_np(cfg, seed=51)
    x_np = make_x_np(n, L["H"], seed=52)                # same tokens on every rank
    x = bf16_tensor(x_np, dev)
    if (L["I"] // world) % L["group"] == 0:             # the shard rule wants group-aligned slices
        Lt = shard_layer_tp(L, rank, world, pad_down_to=512)
        layer_tp = ops.MoELayer(layer_to_torch(Lt, dev))
        out, logits, ids, w = layer_tp.forward(x, path=ops.PATH_DECODE, return_routing=True)
        comm.allreduce_sum(out.view(-1))
        assert comm.status() == 0 and layer_tp.status() == 0
        ref = oracle.moe_layer_w4(x_np, L, logits_in=logits.cpu().numpy())
        assert np.array_equal(ids.cpu().numpy(), ref["ids"])
        assert_layer_close(out.cpu().numpy(), ref["out"], "tensor-parallel layer")
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(g, out) for g in gathered), "ranks disagree after all-reduce"

    # ---- expert parallel: in-kernel NVLink dispatch/combine vs the single-GPU layer, both kernel families ----
    x_loc_np = make_x_np(n, L["H"], seed=60 + rank)     # different tokens per rank
    x_loc = bf16_tensor(x_loc_np, dev)
    full = ops.MoELayer(layer_to_torch(L, dev))
    layer_ep = ops.MoELayer(layer_to_torch(shard_layer_ep(L, rank, world), dev))
    ref = oracle.moe_layer_w4(x_loc_np, L, logits_in=ops.router_logits(x_loc, full._keep["router_w"]).cpu().numpy())
    for path in (ops.PATH_PREFILL, ops.PATH_DECODE):
        want = full.forward(x_loc, path=path).clone()
        for rep in range(2):
            got = layer_ep.forward_ep(comm, x_loc, path=path)
            assert comm.status() == 0, "expert-parallel exchange reported an error"
            assert torch.equal(got, want), f"expert-parallel output differs from single GPU (path {path}, rep {rep})"
        assert_layer_close(got.cpu().numpy(), ref["out"], f"expert-parallel layer vs oracle (path {path})")
    # the block entry (pre-norm inside the logits launch, residual inside the combine) against the single-GPU block
    nw = (1.0 + 0.02 * torch.randn(L["H"], generator=torch.Generator(device=dev).manual_seed(5), device=dev)).contiguous()
    for path in (ops.PATH_PREFILL, ops.PATH_DECODE):
        h_want = torch.from_numpy(x_loc_np).to(dev)
        h_got = h_want.clone()
        full.block_forward(h_want, nw, 1e-5, path=path)
        layer_ep.block_forward_ep(comm, h_got, nw, 1e-5, path=path)
        assert comm.status() == 0
        assert torch.equal(h_got, h_want), f"expert-parallel block differs from the single-GPU block (path {path})"
    # ragged: one rank with no tokens at all, and every rank sizing its buffers from its own n
    n2 = 0 if rank == 0 else 77 + rank
    x2 = bf16_tensor(make_x_np(max(n2, 1), L["H"], seed=70 + rank)[:n2], dev)
    for path in (ops.PATH_PREFILL, ops.PATH_DECODE):
        got2 = layer_ep.forward_ep(comm, x2, recv_cap=4096 + 128 * rank, path=path)
        assert comm.status() == 0
        if n2:
            assert torch.equal(got2, full.forward(x2, path=path))
    # a handful of tokens per rank: routing, dispatch and the posting of the counts ride one launch there
    for n3 in (1 + rank % 3, 32):
        x3 = bf16_tensor(make_x_np(n3, L["H"], seed=80 + rank), dev)
        for path in (ops.PATH_PREFILL, ops.PATH_DECODE):
            ids3 = torch.empty((n3, L["topk"]), dtype=torch.int32, device=dev)
            got5 = layer_ep.forward_ep(comm, x3, recv_cap=1024, path=path, ids_out=ids3)
            assert comm.status() == 0
            want5, _, ids_w, _ = full.forward(x3, path=path, return_routing=True)
            assert torch.equal(ids3, ids_w), f"small-batch expert-parallel routing differs (n={n3}, path {path})"
            assert torch.equal(got5, want5), f"small-batch expert-parallel output differs (n={n3}, path {path})"
    # a receive capacity that is too small is reported, and nothing is written out of bounds
    got3 = layer_ep.forward_ep(comm, x_loc, recv_cap=64, path=ops.PATH_PREFILL)
    torch.cuda.synchronize()
    st = torch.tensor([comm.status()], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    assert int(st) == 7, "overflow of the receive capacity was not reported"
    got4 = layer_ep.forward_ep(comm, x_loc, path=ops.PATH_PREFILL)   # and the next call is fine again
    assert comm.status() == 0 and torch.equal(got4, full.forward(x_loc, path=ops.PATH_PREFILL))


def check_glm(comm, rank, world, dev):
    """GLM-scale layer: expert parallel (256 tokens per rank on the split-K kernels, 1024 on the tcgen05
    kernels) bitwise against the single-GPU layer and, on rank 0, within tolerance of the oracle on a
    token sample; tensor parallel at T=64 against the oracle."""
    cfg = CONFIGS["glm"]
    Lt = make_layer_torch(cfg, seed=1, device=dev)
    full = ops.MoELayer(Lt, keep_raw=False)
    layer_ep = ops.MoELayer(shard_layer_ep(Lt, rank, world), keep_raw=False)
    Lnp = layer_to_np(Lt) if rank == 0 else None
    pick = np.array([0, 1, 7, 100, 255])
    for n, path in ((1024, ops.PATH_PREFILL), (256, ops.PATH_DECODE)):
        # rank 0 alone runs the oracle (seconds of host work): the ranks meet on the host before they launch
        # kernels that wait for one another - the device-side waits are bounded (about two seconds)
        dist.barrier()
        x = make_x_torch(n, cfg["H"], seed=900 + rank, device=dev)
        want, logits, ids, _ = full.forward(x, path=path, return_routing=True)
        want, logits = want.clone(), logits.clone()
        got = layer_ep.forward_ep(comm, x, recv_cap=2 * n * cfg["topk"], path=path)
        st = comm.status()
        assert st == 0, f"GLM-scale expert-parallel exchange reported status {st} (n={n})"
        bad = (got != want).any(dim=1).nonzero().flatten()
        assert bad.numel() == 0, (f"GLM-scale expert-parallel output differs from single GPU (n={n}): {bad.numel()} rows, "
                                  f"first {bad[:8].tolist()}, max abs diff {float((got - want).abs().max()):.3e}")
        if rank == 0:
            sel = torch.from_numpy(pick).to(dev)
            r = oracle.moe_layer_w4(x[sel].float().cpu().numpy(), Lnp, logits_in=logits[sel].cpu().numpy())
            assert np.array_equal(ids.cpu().numpy()[pick], r["ids"])
            assert_layer_close(got.cpu().numpy()[pick], r["out"], f"GLM-scale expert-parallel vs oracle (n={n})")
    del layer_ep
    # tensor parallel, decode batch: same tokens on every rank, local intermediate 2048 / world
    layer_tp = ops.MoELayer(shard_layer_tp_torch(Lt, rank, world), keep_raw=False)
    x = make_x_torch(64, cfg["H"], seed=100, device=dev)
    dist.barrier()
    out, logits, ids, _ = layer_tp.forward(x, path=ops.PATH_DECODE, return_routing=True)
    comm.allreduce_sum(out.view(-1))
    assert comm.status() == 0 and layer_tp.status() == 0
    if rank == 0:
        r = oracle.moe_layer_w4(x.float().cpu().numpy()[:12], Lnp, logits_in=logits.cpu().numpy()[:12])
        assert np.array_equal(ids.cpu().numpy()[:12], r["ids"])
        assert_layer_close(out.cpu().numpy()[:12], r["out"], "GLM-scale tensor-parallel layer vs oracle")
    assert comm.status() == 0
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    assert all(torch.equal(g, out) for g in gathered), "ranks disagree after the GLM-scale all-reduce"


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = Comm(heap_bytes=1024 << 20, allreduce_max_count=4096 * 1024)
    check_allreduce(comm, rank, world, dev)
    check_mid(comm, rank, world, dev)
    check_glm(comm, rank, world, dev)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"rank {rank}: multi-GPU checks passed")


if __name__ == "__main__":
    main()
