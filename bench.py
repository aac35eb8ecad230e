#!/usr/bin/env python
"""Benchmark of the W4A16 MoE layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]

One "step" is one pass of the whole layer (router GEMM -> top-k -> dispatch -> grouped
gate/up + SwiGLU -> down -> shared expert -> combine) over one batch of T synthetic tokens of a
GLM-scale layer (H=6144, 256 experts top-8, I=2048, one shared expert, int4 group 128).
Default T=64: the decode-shaped configuration the headline metric is quoted on.  Prints ONE
JSON line.  With N>1 (launched by torch.distributed.run, one rank per GPU) every rank runs
its own replica of the layer on its own T tokens: the path shards over independent tokens
with no data-path collective, so scaling is "weak" and the value is all ranks' tokens over
the slowest rank's time.

`--impl reference` times the reference's own CPU float32 MoE (GLM52Model::moe_mlp built from
the reference sources into oracle/_ref, else the C restatement in oracle/) on a bounded
token sample of the same workload, on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GLM = dict(H=6144, E=256, topk=8, I=2048, Is=2048, group=128)
W_EXPERT_BYTES = 3 * GLM["H"] * GLM["I"] // 2 + 3 * GLM["H"] * GLM["I"] // GLM["group"] * 2  # 19,464,192


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [c.strip() for c in r.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            try:
                pw.append(float(f[3]))
            except ValueError:
                pass
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_min_mhz=min(sm) if sm else None,
                    sm_max_mhz=max(mx) if mx else None, power_w_max=max(pw) if pw else None,
                    reasons=sorted(reasons), samples=len(sm))


def algorithmic_bytes(ids_np, T: int) -> dict:
    """Bytes the layer must move at least once: each distinct expert's weights once, router
    weight, activations in and out."""
    import numpy as np
    distinct = int(np.unique(ids_np).size)
    wbytes = (distinct + 1) * W_EXPERT_BYTES
    total = wbytes + GLM["E"] * GLM["H"] * 2 + T * GLM["H"] * 2 + T * GLM["H"] * 4
    gate_up = (distinct + 1) * (2 * GLM["H"] * GLM["I"] // 2 + 2 * GLM["H"] * GLM["I"] // GLM["group"] * 2)
    # what the split-K kernels actually stream: an expert once per group of 8 of its tokens, the shared expert
    # once per group of 8 tokens of the batch
    cnt = np.bincount(ids_np.ravel(), minlength=GLM["E"])
    passes = int(((cnt + 7) // 8).sum() + (T + 7) // 8)
    return dict(distinct_experts=distinct, layer_bytes=total, gate_up_bytes=gate_up,
                down_bytes=wbytes - gate_up, passes=passes)


def cpu_port_baseline(Lnp, x_np, sample_tokens: int) -> dict:
    import oracle
    xs = x_np[:sample_tokens]
    nthreads = oracle.max_threads()
    t0 = time.perf_counter()
    oracle.moe_layer_w4(xs, Lnp, nthreads=nthreads)
    dt = time.perf_counter() - t0
    return dict(value=sample_tokens / dt, unit="tokens/s", cores=nthreads, kind="port",
                sample=f"first {sample_tokens} tokens of the batch, {dt:.1f} s, C restatement of moe_mlp "
                       f"(expert-major, int4 rows dequantised on the fly) on {nthreads} threads")


def layer_flops(T: int) -> dict:
    routed = 2 * T * GLM["topk"] * 3 * GLM["H"] * GLM["I"]
    shared = 2 * T * 3 * GLM["H"] * GLM["Is"]
    router = 2 * T * GLM["H"] * GLM["E"]
    gate_up = 2 * (T * GLM["topk"] * 2 * GLM["H"] * GLM["I"] + T * 2 * GLM["H"] * GLM["Is"])
    return dict(layer=routed + shared + router, gate_up=gate_up, down=gate_up // 2)


def time_layer(layer, x, out, path, steps, warmup, barrier, ops, batches=10):
    """Device time of `steps` forwards (CUDA events on the launching stream, barrier + synchronise on both
    sides), taken `batches` times back to back: the median batch is reported and all of them are returned, so a
    number does not rest on one burst of a few milliseconds.  Plus the stage times from the library's stage
    marks, in a pass of their own."""
    import torch
    for _ in range(max(warmup, 3)):
        layer.forward(x, out=out, path=path)
    assert layer.status() == 0, "device-side wait timed out during warm-up"

    def stage_pass():
        # stage marks in a pass of their own: an event recorded between two kernels keeps the second from
        # being scheduled under the first one's tail (programmatic dependent launch), which the timed
        # steps are allowed to do
        ops.profile_enable(layer, steps)
        for _ in range(steps):
            layer.forward(x, out=out, path=path)
        st = ops.profile_read(layer)
        ops.profile_enable(layer, 0)
        return {k: v for k, v in st.items() if k != "forwards"}

    # the first tens of milliseconds of load run at the full SM clock; after that the software power cap
    # lowers it and the split-K kernels, which need most of the SM's issue slots to keep up with HBM, slow
    # down with it: stage times are taken in both regimes
    stages_burst = stage_pass()
    per_step = []
    for _ in range(batches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            layer.forward(x, out=out, path=path)
        e1.record()
        barrier()
        per_step.append(e0.elapsed_time(e1) / steps)
    ms = sorted(per_step)[len(per_step) // 2]
    stages = stage_pass()
    assert layer.status() == 0, "device-side wait timed out"
    return ms, stages, per_step, stages_burst


def copy_same_schedule(dev, steps, batches, barrier):
    """A plain device copy (read + write bytes, like the measured HBM peak) timed under the schedule of the
    headline: `batches` back-to-back batches of `steps` copies of 2 GiB.  A memory-bound kernel that runs for
    a good fraction of a second no longer sees the burst bandwidth; this is what the memory system gives a
    copy under the same load pattern."""
    import torch
    a = torch.empty(1 << 30, dtype=torch.bfloat16, device=dev)
    b = torch.empty_like(a)
    for _ in range(3):
        b.copy_(a)
    gbs = []
    for _ in range(batches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier(); e0.record()
        for _ in range(steps):
            b.copy_(a)
        e1.record(); barrier()
        gbs.append(2 * a.numel() * 2 / (e0.elapsed_time(e1) / steps * 1e-3) / 1e9)
    del a, b
    torch.cuda.empty_cache()
    return gbs


def reference_stage_names(stages: dict, allreduce_ms=None) -> dict:
    """The library's stage marks grouped under the names the reference's StageProf prints
    (src/model_gpu.cpp:1451-1499): moe.router = router GEMM + top-k + dispatch; moe.experts = the grouped
    gate/up, down and combine launches; the shared expert has no stage of its own here (it is the last
    segment of the same grouped launches, so moe.shared is part of moe.experts); ar.mlp = the all-reduce after
    a tensor-parallel layer."""
    d = {"moe.router": stages["moe.router"] + stages["moe.dispatch"],
         "moe.experts": stages["moe.gate_up"] + stages["moe.down"] + stages["moe.combine"],
         "moe.shared": 0.0}
    if allreduce_ms is not None:
        d["ar.mlp"] = allreduce_ms
    return d


def measured_traffic(key: str):
    """DRAM bytes of the dominant kernel per unit of work (one distinct expert for the decode kernel), from
    the single-kernel ncu capture of a small case summarised in profiles/traffic.json; the caller scales it
    by the units one launch of the full workload processes.  None when the file has no entry."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return None
    with open(p) as f:
        return json.load(f).get(key)


def run_ours(args) -> None:
    import numpy as np
    import torch

    from glmserve_b200 import ops
    from glmserve_b200.synth import layer_to_np, make_layer_torch, make_x_torch, zipf_bias

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    T = args.tokens
    prefill = T >= 256 if args.path == "auto" else args.path == "prefill"
    path = ops.PATH_PREFILL if prefill else ops.PATH_DECODE

    Lt = make_layer_torch(GLM, seed=1, device=dev)
    if prefill:  # configuration 3: Zipf(1.1)-ranked router bias, loads from ~0 to ~8x the mean
        Lt["e_bias"] = (Lt["e_bias"] + torch.from_numpy(zipf_bias(GLM["E"], np.random.default_rng(1), 0.04)).to(dev)).contiguous()
    layer = ops.MoELayer(Lt, keep_raw=False)
    x = make_x_torch(T, GLM["H"], seed=100 + rank, device=dev)
    out = torch.empty((T, GLM["H"]), dtype=torch.float32, device=dev)
    x_host = x.cpu().pin_memory()
    out_host = torch.empty((T, GLM["H"]), dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    _, _, ids, _ = layer.forward(x, out=out, path=path, return_routing=True)
    ids_np = ids.cpu().numpy()
    alg = algorithmic_bytes(ids_np, T)
    loads = np.bincount(ids_np.ravel(), minlength=GLM["E"])

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_step, stages, batches_ms, stages_burst = time_layer(layer, x, out, path, args.steps, args.warmup, barrier, ops, batches=args.batches)

    copy_gbs = copy_same_schedule(dev, args.steps, args.batches, barrier) if (world == 1 and not args.no_extra) else None

    # end to end through the host-buffer call: H2D of the step's tokens, D2H of its output
    for _ in range(3):
        layer.forward_host(x_host, out_host, path=path)
    # the same schedule as the device-timed number: back-to-back batches, the median batch (a single batch after
    # a pause would run at the clocks of the first milliseconds of load and come out faster than `value`)
    e2e_batches = []
    for _ in range(args.batches):
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            layer.forward_host(x_host, out_host, path=path)
        barrier()
        e2e_batches.append((time.perf_counter() - t0) * 1e3 / args.steps)
    e2e_ms = sorted(e2e_batches)[len(e2e_batches) // 2]
    clocks = sampler.stop() if rank == 0 else None

    # the other shapes of the headline metric, on the same resident weights (N=1 only)
    extra = {}
    if world == 1 and not args.no_extra and not prefill and T == 64 and GLM["E"] == 256:
        for t2 in (1, 8):
            x2 = make_x_torch(t2, GLM["H"], seed=100 + t2, device=dev)
            o2 = torch.empty((t2, GLM["H"]), dtype=torch.float32, device=dev)
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
            _, _, i2, _ = layer.forward(x2, out=o2, path=ops.PATH_DECODE, return_routing=True)
            a2 = algorithmic_bytes(i2.cpu().numpy(), t2)
            ts = []
            for _ in range(10):  # small working sets: flush L2 (write 256 MiB) before every timed call
                flush.fill_(1)
                ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ea.record(); layer.forward(x2, out=o2, path=ops.PATH_DECODE); eb.record()
                torch.cuda.synchronize()
                ts.append(ea.elapsed_time(eb))
            m2 = sorted(ts)[len(ts) // 2]
            extra[f"decode_T{t2}"] = {"us_per_layer": m2 * 1e3, "layer_gbs": a2["layer_bytes"] / (m2 * 1e-3) / 1e9,
                                      "distinct_experts": a2["distinct_experts"], "l2": "flushed before each call"}
            del flush
        Tp = 8192
        Ls = dict(Lt)
        Ls["e_bias"] = (Lt["e_bias"] + torch.from_numpy(zipf_bias(GLM["E"], np.random.default_rng(1), 0.04)).to(dev)).contiguous()
        layer_p = ops.MoELayer(Ls, share_from=layer)
        xp = make_x_torch(Tp, GLM["H"], seed=200, device=dev)
        op_ = torch.empty((Tp, GLM["H"]), dtype=torch.float32, device=dev)
        _, _, ip, _ = layer_p.forward(xp, out=op_, path=ops.PATH_PREFILL, return_routing=True)
        lp = np.bincount(ip.cpu().numpy().ravel(), minlength=GLM["E"])
        msp, stp, _, _ = time_layer(layer_p, xp, op_, ops.PATH_PREFILL, 5, 3, barrier, ops, batches=5)
        fl = layer_flops(Tp)
        pk = peaks()
        extra["prefill_T8192"] = {"tokens_per_s": Tp / (msp * 1e-3), "ms_per_layer": msp,
                                  "tflops": fl["layer"] / (msp * 1e-3) / 1e12,
                                  "frac_of_measured_bf16_peak": fl["layer"] / (msp * 1e-3) / 1e12 / pk["bf16_tflops"],
                                  # the layer is timed inside a long loop, under the power cap: the cuBLAS figure
                                  # measured the same way (seconds-long loop) is the like-for-like denominator
                                  "frac_of_measured_sustained_bf16_peak": fl["layer"] / (msp * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
                                  "gate_up_kernel_tflops": fl["gate_up"] / (stp["moe.gate_up"] * 1e-3) / 1e12,
                                  "gate_up_kernel_frac": fl["gate_up"] / (stp["moe.gate_up"] * 1e-3) / 1e12 / pk["bf16_tflops"],
                                  "down_kernel_tflops": fl["down"] / (stp["moe.down"] * 1e-3) / 1e12,
                                  "down_kernel_frac": fl["down"] / (stp["moe.down"] * 1e-3) / 1e12 / pk["bf16_tflops"],
                                  "stage_ms": stp, "load_max_over_mean": float(lp.max() / lp.mean()),
                                  "load_min_over_mean": float(lp.min() / lp.mean()),
                                  "routing": "Zipf(1.1)-ranked router bias, amplitude 0.04"}

    # expert-parallel baseline: the T=4096 uniform-routing layer on one GPU with all experts
    if world == 1 and not args.no_extra and not prefill and T == 64 and GLM["E"] == 256:
        Te = 4096
        xe = make_x_torch(Te, GLM["H"], seed=300, device=dev)
        oe = torch.empty((Te, GLM["H"]), dtype=torch.float32, device=dev)
        mse, ste, _, _ = time_layer(layer, xe, oe, ops.PATH_PREFILL, 5, 3, barrier, ops, batches=3)
        extra["ep_base_T4096"] = {"tokens_per_s": Te / (mse * 1e-3), "ms_per_layer": mse, "stage_ms": ste,
                                  "tflops": layer_flops(Te)["layer"] / (mse * 1e-3) / 1e12,
                                  "note": "one GPU holding all 256 experts, uniform routing; denominator of the "
                                          "expert-parallel scaling efficiency tps(G) / (G * tps(1))"}
        del xe, oe

    # speculative-verify block: 8 consecutive layers (pre-RMSNorm + MoE + residual), 64 x 4 = 256 tokens
    if world == 1 and not args.no_extra and not prefill and T == 64 and GLM["E"] == 256:
        from glmserve_b200.synth import make_layer_torch as mk
        nl, Tv = 8, 256
        layers = [layer] + [ops.MoELayer(mk(GLM, seed=10 + i, device=dev), keep_raw=False) for i in range(1, nl)]
        norms = [(1.0 + 0.02 * torch.randn(GLM["H"], device=dev)).float().contiguous() for _ in range(nl)]
        h0 = make_x_torch(Tv, GLM["H"], seed=400, device=dev).float()
        res = {}
        for pname, pth in (("decode_kernels", ops.PATH_DECODE), ("tcgen05_kernels", ops.PATH_PREFILL)):
            h = h0.clone()
            for _ in range(2):
                for L_, nw in zip(layers, norms):
                    L_.block_forward(h, nw, 1e-5, path=pth)
            ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            h = h0.clone()
            torch.cuda.synchronize(); ea.record()
            for _ in range(3):
                for L_, nw in zip(layers, norms):
                    L_.block_forward(h, nw, 1e-5, path=pth)
            eb.record(); torch.cuda.synchronize()
            res[pname] = ea.elapsed_time(eb) / 3 * 1e3
        best = min(res, key=res.get)
        extra["spec_verify_block_8_layers_T256"] = {"us_per_block": res[best], "us_per_layer": res[best] / nl,
                                                    "kernels": best, "all_us_per_block": res,
                                                    "hbm_floor_us_per_layer_at_measured_peak": 257 * W_EXPERT_BYTES / peaks()["hbm_gbs"] / 1e3}
        del layers[1:]
        torch.cuda.empty_cache()

    # the same experts through the reference's own operator signature (raw layout, fp32 activations and scales,
    # ids and weights from the caller): the direct-layout kernel, and the tile-stream kernels behind the
    # operator cache (weights repacked once, keyed on their pointers)
    if world == 1 and not args.no_extra and not prefill and T == 64 and GLM["E"] == 256:
        n8 = 8
        x8 = x[:n8].contiguous()
        _, _, i8, w8 = layer.forward(x8, path=ops.PATH_DECODE, return_routing=True)
        raw = [Lt["gate_q"], Lt["gate_sc"].float(), Lt["up_q"], Lt["up_sc"].float(), Lt["down_q"], Lt["down_sc"].float()]
        xf = x8.float().contiguous()

        def op_call():
            return ops.moe_expert_ffn_w4a16(xf, i8.contiguous(), w8.contiguous(), *raw, GLM["group"])
        res = {}
        for name, cache in (("direct_layout_kernel", 0), ("operator_cache", 8 << 30)):
            ops.operator_cache_enable(cache)
            for _ in range(3):
                op_call()
            ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); ea.record()
            for _ in range(10):
                op_call()
            eb.record(); torch.cuda.synchronize()
            res[name] = ea.elapsed_time(eb) / 10 * 1e3
        ops.operator_cache_enable(0)
        extra["operator_surface_moe_expert_ffn_w4a16_T8"] = {
            "us_per_call": res, "note": "routed experts only (no router, no shared expert), 8 tokens, "
                                        "the call src/model_gpu.cpp makes; includes the output allocation of the wrapper"}
        del raw
        torch.cuda.empty_cache()

    # N > 1: the two ways the layer is partitioned over the box, on top of the replica headline
    if world > 1 and not args.no_extra and GLM["E"] % world == 0:
        from glmserve_b200.dist import Comm, shard_layer_ep, shard_layer_tp_torch
        from glmserve_b200.synth import make_layer_torch as mk
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def timed(fn, reps, warm=3):
            for _ in range(warm):
                fn()
            barrier(); ea.record()
            for _ in range(reps):
                fn()
            eb.record(); barrier()
            return ea.elapsed_time(eb) / reps

        def max_over_ranks(vals):
            tt = torch.tensor([float(v) for v in vals], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return [float(v) for v in tt]

        Te = 4096
        recv_cap = 2 * Te * GLM["topk"]
        layer_ep = ops.MoELayer(shard_layer_ep(Lt, rank, world), keep_raw=False)
        ar_max = 256 * GLM["H"]
        heap = layer_ep.ep_heap_bytes(Te, recv_cap) + Comm.reserve_bytes(world, ar_max) + (1 << 20)
        comm = Comm(heap_bytes=heap, allreduce_max_count=ar_max)
        xe = make_x_torch(Te, GLM["H"], seed=300 + rank, device=dev)
        oe = torch.empty((Te, GLM["H"]), dtype=torch.float32, device=dev)
        # parity inside the run: the expert-parallel output of this rank's tokens against the single-GPU layer
        # (all experts resident) on the same tokens - the same bits, on every rank
        want = layer.forward(xe, path=ops.PATH_PREFILL).clone()
        got = layer_ep.forward_ep(comm, xe, out=oe, recv_cap=recv_cap, path=ops.PATH_PREFILL)
        torch.cuda.synchronize()
        st_ep = comm.status()
        eq = torch.tensor([1 if torch.equal(got, want) else 0], device=dev)
        dist.all_reduce(eq, op=dist.ReduceOp.MIN)
        del want
        ms_ep = timed(lambda: layer_ep.forward_ep(comm, xe, out=oe, recv_cap=recv_cap, path=ops.PATH_PREFILL), 5)
        st_ep = st_ep or comm.status()
        # where the time goes: the library's stage marks on the caller's stream (a second pass)
        ops.profile_enable(layer_ep, 5)
        for _ in range(5):
            layer_ep.forward_ep(comm, xe, out=oe, recv_cap=recv_cap, path=ops.PATH_PREFILL)
        ph = ops.profile_read(layer_ep, ops.EP_STAGES)
        ops.profile_enable(layer_ep, 0)
        ph_names = [k for k in ph if k != "forwards"]
        ph_max = dict(zip(ph_names, max_over_ranks([ph[k] for k in ph_names])))
        # the denominator of the expert-parallel efficiency, measured in this run: all 256 experts on one GPU
        ms_base = timed(lambda: layer.forward(xe, out=oe, path=ops.PATH_PREFILL), 5)

        # speculative-verify block on the box, expert parallel: 8 consecutive layers (pre-RMSNorm + MoE + residual),
        # 256 tokens in all = 256 / N per GPU, every layer with its own weights (rank r holds its experts of each)
        nl, Tv = 8, 256
        nv = Tv // world
        layers_ep = [layer_ep] + [ops.MoELayer(shard_layer_ep(mk(GLM, seed=10 + i, device=dev), rank, world), keep_raw=False)
                                  for i in range(1, nl)]
        torch.cuda.empty_cache()
        norms = [(1.0 + 0.02 * torch.randn(GLM["H"], device=dev)).float().contiguous() for _ in range(nl)]
        hv = make_x_torch(nv, GLM["H"], seed=400 + rank, device=dev).float()
        cap_v = 2 * nv * GLM["topk"]

        def verify_block_ep():
            for L_, nw in zip(layers_ep, norms):
                L_.block_forward_ep(comm, hv, nw, 1e-5, recv_cap=cap_v, path=ops.PATH_DECODE)
        us_blk_ep = timed(verify_block_ep, 3, warm=2) * 1e3
        st_ep = st_ep or comm.status()
        ops.profile_enable(layer_ep, 4)
        for _ in range(4):
            layer_ep.block_forward_ep(comm, hv, norms[0], 1e-5, recv_cap=cap_v, path=ops.PATH_DECODE)
        phv = ops.profile_read(layer_ep, ops.EP_STAGES)
        ops.profile_enable(layer_ep, 0)
        phv_names = [k for k in phv if k != "forwards"]
        phv_max = dict(zip(phv_names, max_over_ranks([phv[k] * 1e3 for k in phv_names])))
        del layers_ep[1:]
        torch.cuda.empty_cache()

        # the all-reduce alone, both algorithms, against NCCL as the baseline; the faster one is then
        # set for the tensor-parallel layer (the choice changes no bit of the result)
        us_alg_all = {}
        # Device time of the collective: n calls from ONE host call (gsb_comm_allreduce_sum_n) for ours, one
        # CUDA-graph replay of n calls for NCCL - launched call by call from Python both are bound by the host
        # (~10-20 us per call) below about 20 us.
        nrep = 50

        def ours_n(buf):
            comm.allreduce_sum_n(buf, 5)
            barrier(); ea.record()
            comm.allreduce_sum_n(buf, nrep)
            eb.record(); barrier()
            return ea.elapsed_time(eb) / nrep * 1e3

        def nccl_n(buf):
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(3):
                        dist.all_reduce(buf)
                torch.cuda.current_stream().wait_stream(side)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for _ in range(nrep):
                        dist.all_reduce(buf)
                g.replay()
                barrier(); ea.record()
                g.replay()
                eb.record(); barrier()
                return ea.elapsed_time(eb) / nrep * 1e3, "cuda graph replay"
            except Exception:          # capture of the collective refused: per-call launches from the host
                torch.cuda.synchronize()
                return timed(lambda: dist.all_reduce(buf), nrep, warm=5) * 1e3, "host-launched calls"
        nccl_how = ""
        for nfl in (GLM["H"], T * GLM["H"]):
            buf = torch.zeros(nfl, device=dev)
            us_alg = {}
            comm.allreduce_ll_limit(1)                      # the flag-in-data form off: time the two flag forms
            for name, limit in (("one_shot", 1 << 40), ("two_shot", 1)):
                comm.allreduce_one_shot_limit(limit)
                us_alg[name] = ours_n(buf)
            comm.allreduce_ll_limit(0)
            if nfl <= 65536:                                # decode-sized: the form the library picks by default
                us_alg["flag_in_data"] = ours_n(buf)
            us_alg["nccl"], nccl_how = nccl_n(buf)
            keys = list(us_alg)
            us_alg_all[nfl] = dict(zip(keys, max_over_ranks([us_alg[k] for k in keys])))
        us_alg = us_alg_all[T * GLM["H"]]
        comm.allreduce_one_shot_limit((1 << 40) if us_alg["one_shot"] <= us_alg["two_shot"] else 1)
        us_ar, us_nccl = min(us_alg["one_shot"], us_alg["two_shot"]), us_alg["nccl"]
        # tensor parallel: decode batch, gate/up column split, down row split, NVLink all-reduce
        Ltp = shard_layer_tp_torch(Lt, rank, world)
        layer_tp = ops.MoELayer(Ltp, keep_raw=False)
        xt = make_x_torch(T, GLM["H"], seed=100, device=dev)
        ot = torch.empty((T, GLM["H"]), dtype=torch.float32, device=dev)

        def tp_layer():
            layer_tp.forward(xt, out=ot, path=ops.PATH_DECODE)
            comm.allreduce_sum(ot.view(-1))
        ms_tp = timed(tp_layer, args.steps)
        # speculative-verify block under tensor parallelism: 8 x (RMSNorm -> sharded layer -> all-reduce ->
        # residual), 256 tokens.  The eight layers share one set of sharded weights (a shard is far larger
        # than L2, so every layer still streams it from HBM): timing only.
        norm_w = torch.ones(GLM["H"], device=dev)
        hv2 = make_x_torch(Tv, GLM["H"], seed=400, device=dev).float()
        ov2 = torch.empty((Tv, GLM["H"]), dtype=torch.float32, device=dev)

        def verify_block_tp():
            for _ in range(nl):
                xn = ops.rmsnorm(hv2, norm_w, 1e-5).to(torch.bfloat16)
                layer_tp.forward(xn, out=ov2, path=ops.PATH_DECODE)
                comm.allreduce_sum(ov2.view(-1))
                hv2.add_(ov2)
        us_blk = timed(verify_block_tp, 3, warm=2) * 1e3
        st_tp = comm.status()
        ms_ep, ms_tp, ms_base, us_blk, us_blk_ep, st_ep, st_tp = max_over_ranks(
            [ms_ep, ms_tp, ms_base, us_blk, us_blk_ep, float(st_ep), float(st_tp)])
        flops_ep = layer_flops(Te)["layer"]
        extra["expert_parallel_T4096_per_gpu"] = {
            "tokens_per_s": world * Te / (ms_ep * 1e-3), "ms_per_layer": ms_ep, "experts_per_gpu": GLM["E"] // world,
            "tflops_per_gpu": flops_ep / (ms_ep * 1e-3) / 1e12,
            "frac_of_measured_bf16_peak_per_gpu": flops_ep / (ms_ep * 1e-3) / 1e12 / peaks()["bf16_tflops"],
            "single_gpu_all_experts_ms_per_layer": ms_base,
            "ep_efficiency": ms_base / ms_ep,
            "ep_bitwise_equal_single_gpu": bool(int(eq)),
            "phase_ms_max_over_ranks": ph_max, "recv_cap_rows": recv_cap, "status": int(st_ep),
            "exchange": "in-kernel NVLink stores: dispatch push on a side stream under the shared expert, combine "
                        "from the down-GEMM epilogue"}
        extra[f"tensor_parallel_T{T}"] = {"us_per_layer": ms_tp * 1e3, "tp": world, "allreduce_us": us_ar,
                                          "stage_us_reference_names": {"ar.mlp": us_ar, "layer_without_ar": ms_tp * 1e3 - us_ar},
                                          "allreduce_us_by_algorithm": {k: v for k, v in us_alg.items() if k != "nccl"},
                                          "nccl_allreduce_us": us_nccl, "allreduce_floats": T * GLM["H"],
                                          "allreduce_one_row_us": us_alg_all[GLM["H"]],
                                          "allreduce_timing": "device time per call: 50 calls from one host call (ours), " + nccl_how + " (NCCL)",
                                          "status": int(st_tp)}
        extra[f"spec_verify_block_8_layers_T256_tp{world}"] = {
            "us_per_block": us_blk, "us_per_layer": us_blk / nl,
            "note": "RMSNorm -> tensor-parallel layer (split-K kernels) -> NVLink all-reduce -> residual, "
                    "x 8; the layers share one set of sharded weights"}
        extra[f"spec_verify_block_8_layers_T256_ep{world}"] = {
            "us_per_block": us_blk_ep, "us_per_layer": us_blk_ep / nl, "tokens_per_gpu": nv,
            "phase_us_max_over_ranks": phv_max,
            "note": "expert-parallel block entry (pre-norm in the router-logits launch, split-K kernels, NVLink "
                    "dispatch and return, residual in the combine) x 8; eight different layers, 256 tokens over the box"}
        comm.close()

    if world > 1:
        t = torch.tensor([ms_step, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        pk = peaks()
        gu_ms = stages["moe.gate_up"]
        shape = "prefill" if prefill else "decode"
        if prefill:
            fl = layer_flops(T)
            achieved = fl["gate_up"] / (gu_ms * 1e-3) / 1e12 if gu_ms > 0 else 0.0
            roof = {"bound": "tensor", "kernel": "prefill_gemm_kernel<gate_up>", "achieved": achieved,
                    "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / pk["bf16_tflops"],
                    "peak_source": pk["source"], "algorithmic_flops": fl["gate_up"], "kernel_ms": gu_ms,
                    "traffic": None}
            whole = {"layer_tflops": fl["layer"] / (ms_step * 1e-3) / 1e12,
                     "layer_frac_of_measured_bf16_peak": fl["layer"] / (ms_step * 1e-3) / 1e12 / pk["bf16_tflops"],
                     "load_max_over_mean": float(loads.max() / loads.mean()),
                     "load_min_over_mean": float(loads.min() / loads.mean())}
            l2 = "inputs larger than L2: 5 GB of expert weights and 0.9 GB of gathered activations per step"
        else:
            achieved = alg["gate_up_bytes"] / (gu_ms * 1e-3) / 1e9 if gu_ms > 0 else 0.0
            roof = {"bound": "hbm", "kernel": "decode_reg_kernel<gate_up>", "achieved": achieved,
                    "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                    "peak_source": pk["source"], "algorithmic_bytes": alg["gate_up_bytes"], "kernel_ms": gu_ms,
                    "traffic": None}
            gb = stages_burst["moe.gate_up"]
            roof["burst"] = {"kernel_ms": gb, "achieved": alg["gate_up_bytes"] / (gb * 1e-3) / 1e9,
                             "frac": alg["gate_up_bytes"] / (gb * 1e-3) / 1e9 / pk["hbm_gbs"],
                             "note": "the same kernel in the first tens of milliseconds of load, before the software "
                                     "power cap lowers the SM clock"}
            layer_gbs = alg["layer_bytes"] / (ms_step * 1e-3) / 1e9
            whole = {"layer_gbs": layer_gbs, "layer_frac_of_measured_hbm": layer_gbs / pk["hbm_gbs"],
                     "layer_frac_of_8tbs": layer_gbs / 8000.0}
            l2 = ("inputs larger than L2: every step streams the touched experts' "
                  f"{alg['layer_bytes'] / 1e9:.2f} GB of weights, far beyond the 126 MB L2")
        line = {
            "metric": f"w4a16_moe_layer_{shape}_T{T}_tokens_per_s",
            "value": world * T / (ms_step * 1e-3),
            "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "us_per_layer": ms_step * 1e3, "timing": f"median of {len(batches_ms)} back-to-back batches of {args.steps} steps",
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "w4a16 (int4 weights, fp16 tensor-core math, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": f"GLM-scale {shape} MoE layer, T={T} tokens per GPU: hidden 6144, {GLM['E']} routed "
                                   "experts top-8, expert intermediate 2048, 1 shared expert, W4A16 group 128, "
                                   "fp16 scales, bf16 activations" + (", Zipf(1.1)-skewed routing" if prefill else ""),
                       "multi_gpu": "independent replicas (tokens shard, no collective)" if world > 1 else "single GPU",
                       "l2": l2, "distinct_experts": alg["distinct_experts"], "expert_passes": alg["passes"]},
            **whole,
            "stage_ms": stages,
            "stage_ms_reference_names": reference_stage_names(stages),
            "timed_batches_ms_per_step": batches_ms, "burst_ms_per_step": min(batches_ms),
            "roofline": roof,
            "e2e": {"value": world * T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": T * GLM["H"] * 2, "d2h_bytes_per_step": T * GLM["H"] * 4,
                    "timing": f"host clock, median of {args.batches} back-to-back batches of {args.steps} calls with pinned host buffers"},
            # decode-sized batches: logits (+ activation conversion), fused routing, gate/up, down, combine;
            # above 128 tokens top-k, dispatch and the work lists are launches of their own; the tcgen05 path:
            # logits, top-k, 3 dispatch launches, gather, tile list, gate/up, down, combine.  All timed batches.
            "gpu_launches": (10 if prefill else (5 if T <= 128 else 8)) * args.steps * len(batches_ms),
            "clocks": clocks,
        }
        line.update(extra)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_port_baseline(layer_to_np(Lt), x.float().cpu().numpy(),
                                                     min(T, args.cpu_tokens))
        if copy_gbs:
            med = sorted(copy_gbs)[len(copy_gbs) // 2]
            line["roofline"]["copy_same_schedule_gbs"] = {"median": med, "batches": copy_gbs}
            if not prefill:
                line["roofline"]["frac_of_copy_same_schedule"] = line["roofline"]["achieved"] / med
        tr = measured_traffic(f"{shape}_gate_up")
        if tr:   # scaled from a small-case capture by the units one launch processes
            units = alg["passes"] if not prefill else 1
            line["roofline"]["traffic"] = tr["bytes_per_unit"] * units
            line["roofline"]["traffic_units"] = units
            line["roofline"]["traffic_source"] = tr["source"]
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_reference(args) -> None:
    """The reference's own CPU float32 MoE on a bounded token sample (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import numpy as np
    import torch

    import oracle
    from glmserve_b200.synth import layer_to_np, make_layer_torch, make_x_torch

    T = args.tokens
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
    sample = max(1, min(T, args.ref_tokens))
    Lt = make_layer_torch(GLM, seed=1, device=dev)
    x_np = make_x_torch(T, GLM["H"], seed=100, device=dev).float().cpu().numpy()[:sample]
    Lnp = layer_to_np(Lt)
    del Lt
    logits = oracle.linear(Lnp["router_w"], x_np)
    ids, _, _ = oracle.router(logits, Lnp["e_bias"], GLM["topk"], True, 2.5)
    use_ref = oracle.ref_available()
    times = []
    if use_ref:
        active = np.zeros(GLM["E"], np.uint8)
        active[np.unique(ids)] = 1
        ref_layer = oracle.RefLayer(Lnp, active=active)
        for i in range(args.warmup + args.steps):
            _, secs = ref_layer.run(x_np)
            if i >= args.warmup:
                times.append(secs)
        ref_layer.close()
        cores, kind = 1, "reference"
        what = (f"GLM52Model::moe_mlp built from the reference sources, first {sample} tokens of the batch, "
                "1 thread (the reference runs its token loop single-threaded below 256 tokens), weights "
                "dequantised to fp32 beforehand as the reference does at load")
    else:
        cores, kind = oracle.max_threads(), "port"
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            oracle.moe_layer_w4(x_np, Lnp, nthreads=cores)
            if i >= args.warmup:
                times.append(time.perf_counter() - t0)
        what = f"C restatement of moe_mlp, first {sample} tokens of the batch, {cores} threads"
    sec = sum(times) / len(times)
    val = sample / sec
    print(json.dumps({
        "impl": "reference", "metric": f"w4a16_moe_layer_decode_T{T}_tokens_per_s", "value": val,
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"GLM-scale decode MoE layer, T={T}: bounded sample of {sample} tokens on the host CPU"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": what},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-tokens", type=int, default=16, help="token sample of the CPU baseline leg")
    ap.add_argument("--ref-tokens", type=int, default=4, help="token sample of --impl reference")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--batches", type=int, default=10, help="timed batches of --steps forwards (the median is reported)")
    ap.add_argument("--no-extra", action="store_true", help="skip the T=1, T=8 and T=8192 legs")
    ap.add_argument("--path", default="auto", choices=["auto", "decode", "prefill"],
                    help="auto: tcgen05 grouped GEMM from 256 tokens, split-K decode kernels below")
    ap.add_argument("--experts", type=int, default=256,
                    help="routed experts (256 = the benchmark layer; fewer = a small case for profiler captures)")
    args = ap.parse_args()
    GLM["E"] = args.experts
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
