"""Worker of tests/test_gpu_multi.py: one rank per GPU (launched by torch.distributed.run).
Checks the NVLink all-reduce, the tensor-parallel layer and the expert-parallel layer against
single-GPU results and the CPU oracle.  Exits non-zero on the first failure."""
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
from glmserve_b200.dist import Comm, shard_layer_ep, shard_layer_tp  # noqa: E402
from glmserve_b200.synth import CONFIGS, layer_to_torch, make_layer_np, make_x_np  # noqa: E402
from helpers import assert_layer_close, bf16_tensor  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = CONFIGS["mid"]
    n = 300
    comm = Comm(heap_bytes=512 << 20, allreduce_max_count=4096 * 1024)

    # ---- all-reduce: values, determinism, rows parity, one-shot and two-shot sizes ----
    for count in (4, 6144, 8 * 6144, 64 * 6144, 2048 * 1024 + 64):
        gen = torch.Generator(device=dev); gen.manual_seed(100 + rank)
        x = torch.randn(count, generator=gen, device=dev)
        allx = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(allx, x)
        want = torch.zeros_like(x)
        for r in range(world):
            want = want + allx[r]                       # rank order, like the kernel
        for rep in range(2):                            # both parities
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
    rows = torch.randn((5, 6144), generator=torch.Generator(device=dev).manual_seed(7 + rank), device=dev)
    a, b = rows.clone(), rows.clone()
    comm.allreduce_sum(a.view(-1))
    comm.allreduce_sum_rows(b)
    assert comm.status() == 0 and torch.equal(a, b), "rows parity"

    # ---- tensor parallel: column-split gate/up, row-split down, all-reduce ----
    L = make_layer_np(cfg, seed=51)
    x_np = make_x_np(n, L["H"], seed=52)                # same tokens on every rank
    Lt = shard_layer_tp(L, rank, world, pad_to=512)
    layer_tp = ops.MoELayer(layer_to_torch(Lt, dev))
    x = bf16_tensor(x_np, dev)
    out, logits, ids, w = layer_tp.forward(x, path=ops.PATH_DECODE, return_routing=True)
    comm.allreduce_sum(out.view(-1))
    assert comm.status() == 0 and layer_tp.status() == 0
    ref = oracle.moe_layer_w4(x_np, L, logits_in=logits.cpu().numpy())
    assert np.array_equal(ids.cpu().numpy(), ref["ids"])
    assert_layer_close(out.cpu().numpy(), ref["out"], "tensor-parallel layer")
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    assert all(torch.equal(g, out) for g in gathered), "ranks disagree after all-reduce"

    # ---- expert parallel: in-kernel NVLink dispatch/combine vs the single-GPU layer ----
    x_loc_np = make_x_np(n, L["H"], seed=60 + rank)     # different tokens per rank
    x_loc = bf16_tensor(x_loc_np, dev)
    full = ops.MoELayer(layer_to_torch(L, dev))
    want = full.forward(x_loc, path=ops.PATH_PREFILL)
    layer_ep = ops.MoELayer(layer_to_torch(shard_layer_ep(L, rank, world), dev))
    for rep in range(2):
        got = layer_ep.forward_ep(comm, x_loc)
        assert comm.status() == 0, "expert-parallel exchange reported an error"
        assert torch.equal(got, want), f"expert-parallel output differs from single GPU (rep {rep})"
    ref = oracle.moe_layer_w4(x_loc_np, L, logits_in=ops.router_logits(x_loc, full._keep["router_w"]).cpu().numpy())
    assert_layer_close(got.cpu().numpy(), ref["out"], "expert-parallel layer vs oracle")
    # ragged: one rank with no tokens at all
    n2 = 0 if rank == 0 else 77
    x2 = bf16_tensor(make_x_np(max(n2, 1), L["H"], seed=70 + rank)[:n2], dev)
    got2 = layer_ep.forward_ep(comm, x2, recv_cap=4096)
    assert comm.status() == 0
    if n2:
        assert torch.equal(got2, full.forward(x2, path=ops.PATH_PREFILL))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"rank {rank}: multi-GPU checks passed")


if __name__ == "__main__":
    main()
