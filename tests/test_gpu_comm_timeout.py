"""A bounded device-side wait that actually runs out, on ONE GPU and without faulting anything: a
communicator of two "ranks" whose peer slot maps this process's own heap (gsb_comm_open_loopback),
so the flag a wait is looking for is never posted.  With the budget set to about a millisecond the
kernel gives up, returns, and gsb_comm_status reports GSB_ERR_TIMEOUT; the context stays usable.
The reference's all-reduce spins on such a flag without limit (cuda/custom_ar.cu:77-79)."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GSB_ERR_TIMEOUT = 4


def test_waits_run_out_and_the_context_stays_usable():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import oracle
    from glmserve_b200 import ops
    from glmserve_b200.dist import Comm
    from glmserve_b200.synth import CONFIGS, layer_to_torch, make_layer_np, make_x_np
    from helpers import assert_layer_close, bf16_tensor
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    comm = Comm(heap_bytes=8 << 20, allreduce_max_count=1 << 16, loopback_world=2)
    comm.set_wait_cycles(2_000_000)                     # about a millisecond of SM clocks
    assert comm.status() == 0
    # the barrier's wait kernel looks for the peer's flag, which nothing posts
    t0 = time.perf_counter()
    comm.barrier()
    assert comm.status() == GSB_ERR_TIMEOUT
    assert time.perf_counter() - t0 < 5.0
    assert comm.status() == 0                           # reading the status cleared it
    # the all-reduce kernel (one-shot and two-shot): every block's wait runs out, the kernel returns
    for limit in (1 << 40, 1):
        comm.allreduce_one_shot_limit(limit)
        x = torch.ones(8192, device=dev)
        comm.allreduce_sum(x)
        assert comm.status() == GSB_ERR_TIMEOUT
    # the GPU and the library carry on: a layer forward gives the oracle's result afterwards
    L = make_layer_np(CONFIGS["mid"], seed=3)
    layer = ops.MoELayer(layer_to_torch(L, dev))
    x_np = make_x_np(16, L["H"], seed=4)
    out, logits, ids, w = layer.forward(bf16_tensor(x_np, dev), path=ops.PATH_DECODE, return_routing=True)
    assert layer.status() == 0
    r = oracle.moe_layer_w4(x_np, L, logits_in=logits.cpu().numpy())
    assert np.array_equal(ids.cpu().numpy(), r["ids"])
    assert_layer_close(out.cpu().numpy(), r["out"], "layer after the timeouts")
    comm.close()
