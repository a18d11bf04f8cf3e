#!/usr/bin/env python
"""Benchmark of the quantized GEMV hot path: the Q4_K projection sweep over Qwen3-8B
layer shapes at M = 1 (batch-1 decode), all 36 layers' distinct weights streamed once
per step, so every step reads 3.9 GB of weights -- far larger than L2.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl nnq|reference]

One JSON line on stdout (rank 0). `value` is algorithmic GB/s of the whole job with
inputs resident in HBM; `e2e` is the same metric through the host entry point of the
C ABI (host activations in, host outputs out, copies inside the timed region);
`cpu_baseline` is the CPU oracle (a port of the reference's CPU path) on a bounded
sample; `--impl reference` times that CPU path alone with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "quant_gemv_hbm_gbs"
UNIT = "GB/s"
WORKLOAD = "q4_k_projection_sweep_qwen3_8b_m1"

# dram bytes (read + write) per algorithmic byte of the dominant kernel, from its ncu capture on the
# two-layer case (27.18 MB moved for 27.17 MB of tiles, activations and outputs per launch; the
# per-launch traffic does not depend on the layer count)
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 27.18 / 27.17


def workload_config(m: int, layers: int) -> dict:
    """The workload both arms report: identical keys and values for the same flags."""
    return {"workload": WORKLOAD, "m": m, "layers": layers, "format": "Q4_K", "activations": "bf16",
            "outputs": "bf16", "accumulate": "f32"}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    BAD = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown"}
    NOTE = {0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in {**self.BAD, **self.NOTE}.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.004)

    def __enter__(self):
        if self._nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------- #
# CPU baseline / reference arm
# --------------------------------------------------------------------------- #

def cpu_sample(threads: int, reps: int, seed: int = 0x5EED):
    """One decoder layer's seven Q4_K projections at M = 1 through the CPU oracle
    (dequantize the whole weight, then the nn-cpu row dot): returns (GB/s, seconds/rep)."""
    import numpy as np
    from nn_b200 import formats as F
    from nn_b200 import workload as W
    from oracle import cpu as orc
    orc.build()
    ws, xs, scratch = [], {}, None
    for i, (name, n, k) in enumerate(W.PROJECTIONS):
        ws.append((n, k, W.gen_q4_k_host(seed + i, n, k)))
        if k not in xs:
            xs[k] = F.gen_activations(seed + 100 + k, 1, k, bf16=True)
    scratch = np.empty(max(n * k for n, k, _ in ws), np.float32)
    algo = W.layer_bytes(1).algorithmic
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        for n, k, w in ws:
            orc.cpu_forward(F.QuantFormat.Q4_K, w, xs[k], None, 1, n, k, threads=threads, scratch=scratch)
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    return algo / best / 1e9, best


def run_reference(args, rank):
    """Reference arm: the reference's CPU implementation of the path (restated in C, since
    the Rust workspace cannot be built here), all host threads, one layer per step."""
    if rank != 0:
        return
    import numpy as np
    from nn_b200 import formats as F
    from nn_b200 import workload as W
    from oracle import cpu as orc
    orc.build()
    threads = os.cpu_count() or 1
    seed = 0x5EED
    ws, xs = [], {}
    for i, (name, n, k) in enumerate(W.PROJECTIONS):
        ws.append((n, k, W.gen_q4_k_host(seed + i, n, k)))
        if k not in xs:
            xs[k] = F.gen_activations(seed + 100 + k, 1, k, bf16=True)
    scratch = np.empty(max(n * k for n, k, _ in ws), np.float32)
    algo = W.layer_bytes(1).algorithmic

    def step():
        for n, k, w in ws:
            orc.cpu_forward(F.QuantFormat.Q4_K, w, xs[k], None, 1, n, k, threads=threads, scratch=scratch)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = algo / dt / 1e9
    sample = ("one layer of the 36 (7 projections, 108.5 MB of Q4_K) per step: dequantize whole weight + nn-cpu row dot, "
              "all host threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.m, args.layers),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# --------------------------------------------------------------------------- #
# GPU arm
# --------------------------------------------------------------------------- #

def run_nnq(args, rank, world, local_rank):
    import ctypes

    import torch
    import torch.distributed as dist

    from nn_b200 import api, comm
    from nn_b200 import workload as W
    from nn_b200.formats import QuantFormat

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    backend = api.Backend(local_rank)
    api.register_gpu_backend(backend)
    lib, ctx = backend._lib, backend._ctx
    m = args.m
    # row-parallel partial outputs are summed by the library's one-shot all-reduce over peer memory
    # slots: 8 bytes per output row of the fused exchange + the record of the distributed argmax
    # (and the [rows, hidden] f32 partial sums of the prompt pass, 256 rows at a time)
    peer = comm.PeerComm(backend, rank, world, max_bytes=256 * W.HIDDEN * 4 + 256) if world > 1 else None
    gen = torch.Generator(device=dev)
    gen.manual_seed(0x5EED)  # same weights on every rank, each keeps its shard

    # ---- weights: `layers` distinct layers, tensor-parallel shards when world > 1 ----
    # With N > 1 every rank also keeps the unsharded weights the parity check multiplies: layer 0's
    # row-parallel projections everywhere, and on rank 0 all layers (the single-GPU decoder the
    # tensor-parallel tokens are compared with).
    layers, full_layers = [], []
    keep_all_full = world > 1 and rank == 0 and m == 1 and args.layers == W.LAYERS and not args.no_others
    for li in range(args.layers):
        lw, fw = {}, {}
        for name, n, k in W.PROJECTIONS:
            raw = W.gen_q4_k_device(torch, gen, n, k)
            shard = (W.TP_AXIS[name], rank, world) if world > 1 else None
            lw[name] = api.DeviceWeight.from_device(backend, QuantFormat.Q4_K, raw, n, k, shard=shard)
            if world > 1 and (keep_all_full or (li == 0 and W.TP_AXIS[name] == 1)):
                fw[name] = api.DeviceWeight.from_device(backend, QuantFormat.Q4_K, raw, n, k)
            del raw
        layers.append(lw)
        full_layers.append(fw)
    torch.cuda.synchronize()

    # ---- activations / outputs (bf16), one set per layer ----
    def shard_k(name, k):
        return k // world if W.TP_AXIS[name] == 1 else k

    xs, ys = [], []
    for li in range(args.layers):
        xg, yg = {}, {}
        for group in W.GROUPS:
            k = shard_k(group[0], dict((p[0], p[2]) for p in W.PROJECTIONS)[group[0]])
            x = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
            for name in group:
                xg[name] = x
                yg[name] = torch.empty(m, layers[li][name].shape[0], dtype=torch.bfloat16, device=dev)
        xs.append(xg)
        ys.append(yg)

    VP = ctypes.c_void_p
    calls = []  # prebuilt ctypes argument packs: one nnq_linear_batch call per group
    for li in range(args.layers):
        for group in W.GROUPS:
            cnt = len(group)
            wh = (VP * cnt)(*[layers[li][n_].handle().value for n_ in group])
            xp = (VP * cnt)(*[xs[li][n_].data_ptr() for n_ in group])
            yp = (VP * cnt)(*[ys[li][n_].data_ptr() for n_ in group])
            reduce_out = ys[li][group[0]] if (world > 1 and W.TP_AXIS[group[0]] == 1) else None
            calls.append((cnt, wh, xp, yp, reduce_out))
    launches_per_step = len(calls)

    def step(stream_ptr):
        for cnt, wh, xp, yp, reduce_out in calls:
            if reduce_out is not None and not args.no_fused:
                # row-parallel projection (o_proj, down_proj): product and all-reduce in one call
                # (one kernel at M = 1: partial sums are pushed to the peers as row tiles finish)
                st = peer.linear_raw(wh[0], xp[0], api.BF16, m, None, yp[0], api.BF16, stream_ptr)
                if st != 0:
                    backend.check(st)
                continue
            st = lib.nnq_linear_batch(ctx, cnt, wh, xp, api.BF16, m, None, yp, api.BF16, stream_ptr)
            if st != 0:
                backend.check(st)
            if reduce_out is not None:   # separate all-reduce of the partial sums
                st = peer.all_reduce_raw(reduce_out.data_ptr(), api.BF16, reduce_out.numel(), stream_ptr)
                if st != 0:
                    backend.check(st)

    stream = torch.cuda.Stream(device=dev)
    graph = None
    parity = None
    with torch.cuda.stream(stream):
        sp = VP(stream.cuda_stream)
        for _ in range(2):
            step(sp)
        stream.synchronize()
        backend.device_status(stream)
        parity = None
        if world > 1:
            parity = check_tp_products(torch, dist, backend, full_layers[0], xs[0], ys[0], m, world, stream)
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step(VP(torch.cuda.current_stream().cuda_stream))

        def run_step():
            if graph is not None:
                graph.replay()
            else:
                step(sp)

        def fence():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()

        for _ in range(args.warmup):
            run_step()
        fence()
        launches_before = backend.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            e0.record(stream)
            for _ in range(args.steps):
                run_step()
            e1.record(stream)
            fence()
        ms = e0.elapsed_time(e1)
    backend.device_status(stream)
    launched = backend.launch_count() - launches_before
    if graph is not None:
        n_reduce = 0 if (not args.no_fused and m == 1) else sum(1 for c_ in calls if c_[4] is not None)
        launched = (launches_per_step + n_reduce) * args.steps  # replays re-issue the captured kernels
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps

    per_layer = W.layer_bytes(m)
    algo_step = per_layer.algorithmic * args.layers          # whole job, all ranks
    value = algo_step / (ms_per_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel ----
    # At one token the step mixes two kernels: launches of more than 2 x SMs row tiles (q/k/v, gate/up)
    # run skinny_q4k_m1_kernel, the 256-tile o / down launches the token-column kernel. The dominant
    # one (by time and by bytes) is timed on its own launches: the same calls without the others,
    # captured and replayed the same way, CUDA events on the launching stream.
    peak, peak_kind = _peaks()
    from nn_b200.formats import algorithmic_bytes
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    group_rows = [sum(layers[0][n_].shape[0] for n_ in g) for g in W.GROUPS]
    dominant = [gi for gi, rows in enumerate(group_rows) if (rows + 15) // 16 > 2 * sms]
    roofline = None
    if world == 1 and m == 1 and dominant and len(dominant) < len(W.GROUPS):
        dom_calls = [c for ci, c in enumerate(calls) if ci % len(W.GROUPS) in dominant]

        def dom_step(stream_ptr):
            for cnt, wh, xp, yp, _ in dom_calls:
                st = lib.nnq_linear_batch(ctx, cnt, wh, xp, api.BF16, m, None, yp, api.BF16, stream_ptr)
                if st != 0:
                    backend.check(st)

        with torch.cuda.stream(stream):
            dom_step(sp)
            stream.synchronize()
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=stream):
                dom_step(VP(torch.cuda.current_stream().cuda_stream))
            for _ in range(args.warmup):
                g2.replay()
            stream.synchronize()
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            d0.record(stream)
            for _ in range(args.steps):
                g2.replay()
            d1.record(stream)
            stream.synchronize()
        dom_ms = d0.elapsed_time(d1) / args.steps
        proj = {p[0]: p for p in W.PROJECTIONS}
        dom_bytes = sum(algorithmic_bytes(QuantFormat.Q4_K, m, proj[n_][1], proj[n_][2], 2, 2)
                        for gi in dominant for n_ in W.GROUPS[gi]) * args.layers
        bytes_per_launch = dom_bytes / len(dom_calls)
        per_launch_s = dom_ms * 1e-3 / len(dom_calls)
        achieved = bytes_per_launch / per_launch_s / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "peak_source": f"of {peak_kind}", "frac_of_nominal_8000": achieved / 8000.0,
                    "traffic": bytes_per_launch * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                    "traffic_source": "ncu capture of the two-layer case, scaled by the bytes per launch",
                    "kernel": "skinny_q4k_m1_kernel", "launches_per_step": len(dom_calls),
                    "share_of_step_bytes": dom_bytes / algo_step, "share_of_step_time": dom_ms / ms_per_step,
                    "bytes_per_launch": bytes_per_launch, "us_per_launch": per_launch_s * 1e6,
                    "other_kernel": "skinny_mn_kernel (o_proj, down_proj: 256 row tiles each)",
                    "whole_step_frac": value / peak}
    if roofline is None:
        per_gpu_bytes_per_launch = algo_step / world / launches_per_step
        per_launch_s = ms_per_step * 1e-3 / launches_per_step
        achieved = per_gpu_bytes_per_launch / per_launch_s / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "peak_source": f"of {peak_kind}", "frac_of_nominal_8000": achieved / 8000.0, "traffic": None,
                    "kernel": "skinny_q4k_m1_kernel (+ skinny_mn_kernel)" if m == 1 else "skinny_mn_kernel / gemm_tc_kernel",
                    "bytes_per_launch": per_gpu_bytes_per_launch, "us_per_launch": per_launch_s * 1e6}

    # ---- the other configurations of the path, timed briefly (not the headline) ----
    others = None
    if world == 1 and m == 1 and not args.no_others:
        others = other_configs(torch, backend, layers, gen, dev)
    elif world > 1 and m == 1 and not args.no_others:
        # tensor-parallel decode: the same shards, o / down exchanged inside the product kernel
        peak_hbm, _ = _peaks()
        dec = decode_tokens_per_s(torch, backend, layers, gen, dev, peak_hbm, tp=(rank, world), peer=peer,
                                  full_layers=full_layers if keep_all_full else None, dist=dist)
        if dec is not None:
            if parity is not None and dec.get("parity") is not None:
                parity["decode"] = dec.pop("parity")
                parity["ok"] = bool(parity["ok"] and parity["decode"]["ok"])
            t = torch.tensor([dec["ms_per_token"]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dec["ms_per_token"] = float(t.item())
            dec["tokens_per_s"] = 1e3 / dec["ms_per_token"]
        others = {"qwen3_8b_decode_ctx2048": dec}
        try:
            others["q4_k_projection_sweep_m1_plan_tp"] = sweep_plan_tp(torch, dist, backend, layers, xs, ys, peer, dev, algo_step)
        except Exception as e:   # a side measurement must not take the headline down
            others["q4_k_projection_sweep_m1_plan_tp"] = {"error": str(e)[:300]}
        try:
            others["qwen3_32b_prefill_m4096_tp"] = prefill_32b_tp(torch, dist, backend, gen, dev, rank, world)
        except Exception as e:   # a side measurement must not take the headline down
            others["qwen3_32b_prefill_m4096_tp"] = {"error": str(e)[:300]}
        try:
            others["gptoss_20b_moe_block_ep"] = moe_block_ep(torch, dist, backend, dev, rank, world)
        except Exception as e:
            others["gptoss_20b_moe_block_ep"] = {"error": str(e)[:300]}

    # ---- end to end through the host entry point of the C ABI ----
    e2e = None
    if world == 1 and not args.no_e2e:
        proj = {p[0]: p for p in W.PROJECTIONS}
        hx = {k: torch.randn(m, k).to(torch.bfloat16).pin_memory() for k in (W.HIDDEN, W.FFN)}
        hy = {n: torch.empty(m, n, dtype=torch.bfloat16).pin_memory() for n in (W.HIDDEN, W.KV_DIM, W.FFN)}
        h2d = d2h = 0

        VPh = ctypes.c_void_p
        host_calls = []   # one nnq_linear_batch_host call per launch group of a layer
        for li in range(args.layers):
            for group in W.GROUPS:
                cnt = len(group)
                k = proj[group[0]][2]
                wh = (VPh * cnt)(*[layers[li][n_].handle().value for n_ in group])
                xp = (VPh * cnt)(*[hx[k].data_ptr()] * cnt)
                houts = [torch.empty(m, proj[n_][1], dtype=torch.bfloat16).pin_memory() for n_ in group] if li == 0 else host_calls[len(host_calls) - len(W.GROUPS)][4]
                yp = (VPh * cnt)(*[t.data_ptr() for t in houts])
                host_calls.append((cnt, wh, xp, yp, houts, m * k * 2, sum(m * proj[n_][1] * 2 for n_ in group)))

        def host_step():
            nonlocal h2d, d2h
            h2d = d2h = 0
            for cnt, wh, xp, yp, _, bi, bo in host_calls:
                st = lib.nnq_linear_batch_host(ctx, cnt, wh, xp, api.BF16, m, None, yp, api.BF16)
                if st != 0:
                    backend.check(st)
                h2d += bi
                d2h += bo

        host_step()
        e_steps = max(1, min(args.steps, 5))
        t0 = time.perf_counter()
        for _ in range(e_steps):
            host_step()
        dt = (time.perf_counter() - t0) / e_steps
        e2e = {"value": algo_step / dt / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": dt * 1e3, "calls_per_step": len(host_calls),
               "api": "nnq_linear_batch_host (host activations in, host outputs out, one synchronous call per group "
                      "of projections that share their input: 4 per layer)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v1, s1 = cpu_sample(1, 2)
        cores = os.cpu_count() or 1
        vN, sN = cpu_sample(cores, 3)
        cpu = {"value": v1, "unit": UNIT, "cores": 1, "kind": "port",
               "sample": "one layer (7 Q4_K projections, 108.5 MB) at M=1: dequantize whole weight + nn-cpu row "
                         "dot, best of 2; the reference path is single-threaded",
               "seconds_per_layer": s1,
               "all_cores": {"value": vN, "cores": cores, "seconds_per_layer": sN}}

    if parity is not None and not parity["ok"]:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "error": "tensor-parallel parity check failed", "parity": parity}), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        raise SystemExit(3)
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": workload_config(m, args.layers),
            "run": {"parallelism": f"tp{world}" if world > 1 else "single",
                    "weight_bytes_per_step": per_layer.weights * args.layers,
                    "l2_policy": "inputs larger than L2 (every step streams all layers' distinct weights)",
                    "cuda_graph": graph is not None,
                    "tokens_per_s_equiv": 1e3 / ms_per_step * (36 / args.layers)},
            "parity": parity,
            "roofline": roofline, "clocks": clocks.summary(), "gpu_launches": int(launched),
            "e2e": e2e, "cpu_baseline": cpu, "other_configs": others,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def sweep_plan_tp(torch, dist, backend, layers, xs, ys, peer, dev, algo_step):
    """The tensor-parallel M = 1 step as ONE persistent launch per rank (the compiled plan): the
    column-parallel groups as plain groups, o_proj / down_proj with their exchange inside the kernel,
    every group waiting for the one before it. Outputs are compared with what the separate launches
    of the headline step left in the same buffers (2e-3 + one bf16 rounding), before anything is timed."""
    from nn_b200 import plan
    from nn_b200 import workload as W
    want = [{k: v.clone() for k, v in yl.items()} for yl in ys]
    pl = plan.ProductPlan(backend, torch.bfloat16, torch.bfloat16)
    for li, lw in enumerate(layers):
        for group in W.GROUPS:
            if W.TP_AXIS[group[0]] == 1:
                pl.add_reduced(peer, lw[group[0]], xs[li][group[0]], ys[li][group[0]])
            else:
                pl.add([lw[n_] for n_ in group], xs[li][group[0]], [ys[li][n_] for n_ in group])
    pl.finalize()
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for yl in ys:
            for v in yl.values():
                v.zero_()
        pl.run(stream)
        stream.synchronize()
        backend.device_status(stream)
        err = 0.0
        for li in range(len(layers)):
            for k in ys[li]:
                a, b_ = ys[li][k].float(), want[li][k].float()
                err = max(err, float((a - b_).abs().max() / b_.abs().max()))
        t = torch.tensor([err], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tol = 2e-3 + 2.0 ** -7
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            pl.run(torch.cuda.current_stream())
        for _ in range(3):
            g.replay()
        stream.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        reps = 10
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    backend.device_status(stream)
    tt = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt.item())
    out = {"ms_per_step": ms, "gbs": algo_step / ms / 1e6, "launches_per_step_per_rank": 1,
           "parity_max_rel_err_vs_separate_launches": float(t.item()), "tolerance": tol, "ok": bool(t.item() <= tol),
           "info": pl.info()}
    pl.release()
    return out


def sweep_variants(torch, backend, layers, gen, dev, peak_hbm):
    import ctypes

    from nn_b200 import api, plan
    from nn_b200 import workload as W
    lib, ctx = backend._lib, backend._ctx
    VP = ctypes.c_void_p
    algo = W.layer_bytes(1).algorithmic * len(layers)
    proj = {p_[0]: p_ for p_ in W.PROJECTIONS}
    groups = []
    for lw in layers:
        for group in W.GROUPS:
            x = torch.randn(proj[group[0]][2], device=dev, generator=gen).to(torch.bfloat16)
            ys = [torch.empty(proj[n_][1], dtype=torch.bfloat16, device=dev) for n_ in group]
            groups.append(([lw[n_] for n_ in group], x, ys))
    out = {}

    def time_graph(g, reps=10):
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        return {"ms_per_step": ms, "gbs": algo / ms / 1e6, "frac": algo / ms / 1e6 / peak_hbm}

    # (a) four streams
    calls = []
    for ws, x, ys in groups:
        cnt = len(ws)
        calls.append((cnt, (VP * cnt)(*[w.handle().value for w in ws]), (VP * cnt)(*[x.data_ptr()] * cnt),
                      (VP * cnt)(*[y.data_ptr() for y in ys])))
    main = torch.cuda.Stream(device=dev)
    side = [torch.cuda.Stream(device=dev) for _ in range(3)]
    with torch.cuda.stream(main):
        for cnt, wh, xp, yp in calls[:8]:
            backend.check(lib.nnq_linear_batch(ctx, cnt, wh, xp, api.BF16, 1, None, yp, api.BF16, VP(main.cuda_stream)))
        main.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=main):
            cur = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(cur)
            lanes = [cur] + side
            for s_ in side:
                s_.wait_event(fork)
            for i, (cnt, wh, xp, yp) in enumerate(calls):
                backend.check(lib.nnq_linear_batch(ctx, cnt, wh, xp, api.BF16, 1, None, yp, api.BF16,
                                                   VP(lanes[i % 4].cuda_stream)))
            for s_ in side:
                join = torch.cuda.Event()
                join.record(s_)
                cur.wait_event(join)
        row = time_graph(g)
        row["how"] = "the 144 launches of the headline step dealt over 4 streams of one graph (independent products)"
        out["separate_launches_4_streams"] = row
    backend.device_status()

    # (b) the compiled plan
    for name, analyze in (("plan_kernel_ordered", False), ("plan_kernel_dependency_analysed", True)):
        pl = plan.ProductPlan(backend, torch.bfloat16, torch.bfloat16, analyze_deps=analyze)
        for ws, x, ys in groups:
            pl.add(ws, x, ys)
        pl.finalize()
        with torch.cuda.stream(main):
            pl.run(main)
            main.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=main):
                pl.run(torch.cuda.current_stream())
            row = time_graph(g)
        row["launches_per_step"] = 1
        row["info"] = pl.info()
        out[name] = row
        backend.device_status()
        pl.release()
    return out


def prefill_32b(torch, backend, gen, dev, peak_tf, timed):
    """The Qwen3-32B prefill configuration on one GPU: the seven projections of a Qwen3-32B layer (hidden 5120,
    64 query / 8 key-value heads x 128, FFN 25600) at 4096 tokens of bf16 activations, Q4_K and Q6_K
    weights, on the tensor-core path; per shape the time, TFLOP/s and the fraction of the measured
    bf16 peak, and the whole layer."""
    from nn_b200 import api
    from nn_b200 import workload as W
    from nn_b200.formats import QuantFormat
    lib, ctx = backend._lib, backend._ctx
    m = 4096
    shapes = (("q_proj", 8192, 5120), ("k_proj", 1024, 5120), ("v_proj", 1024, 5120), ("o_proj", 5120, 8192),
              ("gate_proj", 25600, 5120), ("up_proj", 25600, 5120), ("down_proj", 5120, 25600))
    out = {}
    for fmt, genfn, tag in ((QuantFormat.Q4_K, W.gen_q4_k_device, "q4_k"), (QuantFormat.Q6_K, W.gen_q6_k_device, "q6_k")):
        rows, total_s, total_f = {}, 0.0, 0.0
        for name, n, k in shapes:
            raw = genfn(torch, gen, n, k)
            w = api.DeviceWeight.from_device(backend, fmt, raw, n, k)
            del raw
            x = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
            y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)

            def one():
                st = lib.nnq_linear(ctx, w.handle(), x.data_ptr(), api.BF16, m, None, y.data_ptr(), api.BF16, None)
                if st != 0:
                    backend.check(st)

            sec = timed(one, 3)
            flops = 2.0 * m * n * k
            rows[name] = {"n": n, "k": k, "ms": sec * 1e3, "tflops": flops / sec / 1e12, "frac": flops / sec / 1e12 / peak_tf}
            total_s += sec
            total_f += flops
            w.release()
            del x, y
        rows["layer"] = {"ms": total_s * 1e3, "tflops": total_f / total_s / 1e12, "frac": total_f / total_s / 1e12 / peak_tf,
                         "tflop": total_f / 1e12}
        out[tag] = rows
    out["bound"] = "tensor"
    out["tokens"] = m
    backend.device_status()
    return out


def moe_block(torch, backend, gen, dev, peak_hbm, peak_tf, timed):
    """The gpt-oss-20b configuration on one GPU: one gpt-oss-20b MoE block (32 experts, top-4, hidden =
    inter = 2880, MXFP4 experts in the [N, K/2] + [N, K/32] layout) at 64 tokens (one decode token of 64
    sequences: bound by the expert weights, 423 MB) and 4096 tokens (prefill: bound by the tensor
    cores, 2 * 16384 routed rows * 3 * 2880 * 2880 flop)."""
    import numpy as np

    from nn_b200 import moe
    from nn_b200.formats import QuantFormat
    E, H, I, k = 32, 2880, 2880, 4
    rng = np.random.default_rng(20)
    rw = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    rb = np.zeros(E, np.float32)

    def payload(n, kk):
        return (rng.integers(0, 256, size=n * (kk // 2), dtype=np.uint8), rng.integers(119, 128, size=n * (kk // 32), dtype=np.uint8))

    gu, gus = payload(E * 2 * I, H)
    dn, dns = payload(E * H, I)
    blk = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, moe.LAYOUT_NK, QuantFormat.MXFP4_SPLIT, gu, gus, np.zeros((E, 2 * I), np.float32),
                       dn, dns, np.zeros((E, H), np.float32), backend=backend)
    weight_bytes = gu.size + gus.size + dn.size + dns.size
    out = {"experts": E, "top_k": k, "hidden": H, "inter": I, "format": "MXFP4 [N,K/2]+[N,K/32]", "weight_bytes": int(weight_bytes)}
    for tokens in (64, 4096):
        x = (torch.randn(tokens, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        sec = timed(lambda: blk(x), 5 if tokens == 64 else 3)
        flops = 2.0 * tokens * k * 3 * H * I
        row = {"us": sec * 1e6, "gbs_over_expert_weights": weight_bytes / sec / 1e9, "tflops": flops / sec / 1e12}
        if tokens == 64:
            row["bound"], row["frac"] = "hbm", weight_bytes / sec / 1e9 / peak_hbm
        else:
            row["bound"], row["frac"] = "tensor", flops / sec / 1e12 / peak_tf
        out[f"tokens_{tokens}"] = row
    backend.device_status()
    blk.release()
    # the same block with the experts stored as nn-gptoss stores them: [E, K, N] tensors, blocks along N
    try:
        blk = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, moe.LAYOUT_KN_GPTOSS, QuantFormat.MXFP4_GPTOSS, gu, gus, np.zeros((E, 2 * I), np.float32),
                           dn, dns, np.zeros((E, H), np.float32), backend=backend)
        kn = {"format": "MXFP4 nn-gptoss [E,K,N/2]+[E,K,N/32]"}
        for tokens in (64, 4096):
            x = (torch.randn(tokens, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
            sec = timed(lambda: blk(x), 5 if tokens == 64 else 3)
            flops = 2.0 * tokens * k * 3 * H * I
            kn[f"tokens_{tokens}"] = {"us": sec * 1e6, "gbs_over_expert_weights": weight_bytes / sec / 1e9, "tflops": flops / sec / 1e12}
        backend.device_status()
        blk.release()
        out["experts_stored_kn"] = kn
    except Exception as e:  # noqa: BLE001 -- a side measurement must not take the line down
        out["experts_stored_kn"] = {"error": str(e)[:200]}
    return out


def _peak_tf():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f).get("bf16_tflops", 0.0)) or 1590.0, "measured"
    except OSError:
        return 1590.0, "fallback"


def prefill_32b_tp(torch, dist, backend, gen, dev, rank, world):
    """The Qwen3-32B prefill configuration over N GPUs: one Qwen3-32B layer's projections at 4096 tokens, Q4_K,
    Megatron split -- q / k / v / gate / up by rows (no exchange), o / down along K (13 / 12
    super-blocks per rank for down_proj at 8 ranks) with the [4096, 5120] bf16 partial outputs summed
    by NCCL's all-reduce, issued eagerly on the timing stream (never captured in a graph). Device
    time with the all-reduces inside, maximum over the ranks; the o_proj result of a sample of
    token rows is compared with the single-GPU product of the unsharded weight first."""
    from nn_b200 import api, tp
    from nn_b200 import workload as W
    from nn_b200.formats import QuantFormat
    lib, ctx = backend._lib, backend._ctx
    m, fmt = 4096, QuantFormat.Q4_K
    peak_tf, peak_kind = _peak_tf()
    shapes = (("q_proj", 8192, 5120, 0), ("k_proj", 1024, 5120, 0), ("v_proj", 1024, 5120, 0), ("o_proj", 5120, 8192, 1),
              ("gate_proj", 25600, 5120, 0), ("up_proj", 25600, 5120, 0), ("down_proj", 5120, 25600, 1))
    out = {"tokens": m, "format": "Q4_K", "parallelism": f"tp{world}", "exchange": "ncclAllReduce (eager, bf16 partial sums)"}
    rows, total_ms, total_f = {}, 0.0, 0.0
    parity = None
    for name, n, k, axis in shapes:
        raw = W.gen_q4_k_device(torch, gen, n, k)          # same bytes on every rank
        w = api.DeviceWeight.from_device(backend, fmt, raw, n, k, shard=(axis, rank, world))
        x_full = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
        x = x_full[:, tp.input_slice(k, axis, rank, world, fmt)].contiguous() if axis == 1 else x_full
        y = torch.empty(m, w.shape[0], dtype=torch.bfloat16, device=dev)

        def one():
            st = lib.nnq_linear(ctx, w.handle(), x.data_ptr(), api.BF16, m, None, y.data_ptr(), api.BF16, None)
            if st != 0:
                backend.check(st)
            if axis == 1:
                dist.all_reduce(y)

        for _ in range(2):
            one()
        torch.cuda.synchronize()
        if name == "o_proj":
            full = api.DeviceWeight.from_device(backend, fmt, raw, n, k)
            sample = torch.arange(0, m, 331, device=dev)
            want = api.quantized_linear(x_full[sample].contiguous(), full, None, out_dtype=torch.float32)
            err = float((y[sample].float() - want).abs().max() / want.abs().max())
            t = torch.tensor([err], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            parity = {"product": "o_proj", "sampled_rows": int(sample.numel()), "max_rel_err_over_ranks": float(t.item()),
                      "tolerance": 1e-2, "ok": bool(t.item() <= 1e-2)}
            full.release()
        del raw
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            one()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        flops = 2.0 * m * n * k
        rows[name] = {"n": n, "k": k, "split": "rows" if axis == 0 else "K", "ms": ms, "tflops": flops / ms / 1e9,
                      "frac_of_n_gpus": flops / ms / 1e9 / (peak_tf * world)}
        total_ms += ms
        total_f += flops
        w.release()
        del x, x_full, y
    rows["layer"] = {"ms": total_ms, "tflops": total_f / total_ms / 1e9, "frac_of_n_gpus": total_f / total_ms / 1e9 / (peak_tf * world),
                     "tflop": total_f / 1e12}
    out["shapes"] = rows
    out["parity"] = parity
    out["peak_source"] = f"of {peak_kind}"
    backend.device_status()
    return out


def moe_block_ep(torch, dist, backend, dev, rank, world):
    """The gpt-oss-20b configuration over N GPUs: one gpt-oss-20b MoE block (32 experts, top-4, hidden =
    inter = 2880, MXFP4) with the experts split over the ranks and the tokens sharded: each rank
    routes its own tokens, rows travel to the experts' owners and back by all-to-all (NCCL), the
    library's kernels gather, run the experts and combine. 64 tokens and 4096 tokens in all; device
    time, maximum over the ranks. Parity first: rank 0 also holds the whole block and compares its
    own tokens' outputs with it."""
    import numpy as np

    from nn_b200 import moe
    from nn_b200.formats import QuantFormat
    E, H, I, k = 32, 2880, 2880, 4
    if E % world:
        return {"skipped": f"{E} experts do not split over {world} ranks"}
    rng = np.random.default_rng(20)        # same bytes on every rank
    rw = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    rb = np.zeros(E, np.float32)

    def payload(n, kk):
        return (rng.integers(0, 256, size=n * (kk // 2), dtype=np.uint8).reshape(E, -1),
                rng.integers(119, 128, size=n * (kk // 32), dtype=np.uint8).reshape(E, -1))

    gu, gus = payload(E * 2 * I, H)
    dn, dns = payload(E * H, I)
    bgu, bd = np.zeros((E, 2 * I), np.float32), np.zeros((E, H), np.float32)
    ec = E // world
    sl = slice(rank * ec, (rank + 1) * ec)
    fmt, layout = QuantFormat.MXFP4_SPLIT, moe.LAYOUT_NK
    shard = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu[sl], gus[sl], bgu[sl], dn[sl], dns[sl], bd[sl], backend=backend,
                         expert_range=(rank * ec, ec))
    ep = moe.ExpertParallelMoe(shard, rank, world)
    full = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu, gus, bgu, dn, dns, bd, backend=backend) if rank == 0 else None
    out = {"experts": E, "top_k": k, "hidden": H, "inter": I, "parallelism": f"ep{world}", "exchange": "all-to-all (NCCL), rows bf16 out / f32 back"}
    g = torch.Generator(device=dev)
    g.manual_seed(77)
    for tokens in (64, 4096):
        tl = tokens // world
        x_all = (torch.randn(tokens, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)   # same on every rank
        x = x_all[rank * tl:(rank + 1) * tl].contiguous()
        y = ep(x)
        torch.cuda.synchronize()
        err = 0.0
        if full is not None:
            want = full(x)
            err = float((y - want).abs().max() / want.abs().max())
        t = torch.tensor([err], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tol = 1e-2 if tokens > 64 else 2e-3
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        e0.record()
        for _ in range(reps):
            ep(x)
        e1.record()
        torch.cuda.synchronize()
        tt = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
        flops = 2.0 * tokens * k * 3 * H * I
        out[f"tokens_{tokens}"] = {"ms": ms, "tokens_per_s": tokens / ms * 1e3, "tflops": flops / ms / 1e9,
                                   "parity_max_rel_err_rank0": float(t.item()), "tolerance": tol, "ok": bool(t.item() <= tol)}
    backend.device_status()
    shard.release()
    if full is not None:
        full.release()
    return out


def check_tp_products(torch, dist, backend, full0, xs0, ys0, m, world, stream):
    """Before anything is timed at N > 1: the fused row-parallel products of layer 0 (o_proj,
    down_proj: product + exchange in one kernel), as the warm-up steps left them in the bench's own
    output buffers, against the library's single-GPU product of the unsharded weight with the
    concatenated activations. Every rank checks its own copy (the exchange promises the same bits
    everywhere); the verdict is the minimum over the ranks. bf16 outputs: 2e-3 + one bf16 rounding."""
    from nn_b200 import api
    tol = 2e-3 + 2.0 ** -8
    out = {"ok": True, "tolerance": tol, "products": {}}
    from nn_b200 import workload as W
    for name, wfull in full0.items():
        if W.TP_AXIS[name] != 1:
            continue   # column-parallel products involve no exchange
        x_full = torch.cat([xs0[name]] * world, dim=1).contiguous()   # every rank drew the same shard values
        want = api.quantized_linear(x_full, wfull, None, out_dtype=torch.float32)
        stream.synchronize()
        torch.cuda.synchronize()
        got = ys0[name].float()
        err = float((got - want).abs().max() / want.abs().max())
        t = torch.tensor([err], device=got.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # identical bits on every rank: compare a checksum of the raw outputs
        cs = ys0[name].view(torch.int16).to(torch.int64).sum().reshape(1)
        lo, hi = cs.clone(), cs.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool(lo.item() == hi.item())
        out["products"][name] = {"max_rel_err_over_ranks": float(t.item()), "same_bits_on_all_ranks": same}
        out["ok"] = bool(out["ok"] and float(t.item()) <= tol and same)
    backend.device_status(stream)
    return out


def other_configs(torch, backend, layers, gen, dev):
    """Short device-timed runs of the path's other configurations (inputs resident in HBM, more
    weight bytes per pass than L2 holds): the Q4_K sweep at 16 / 128 / 512 tokens over the same
    36 layers, the Q8_0 4096 x 4096 GEMV with f32 activations, a Q6_K vocabulary-sized GEMV and the same shape with
    INT8 per-channel weights."""
    import ctypes

    from nn_b200 import api
    from nn_b200 import workload as W
    from nn_b200.formats import QuantFormat, algorithmic_bytes

    lib, ctx = backend._lib, backend._ctx
    peak_hbm, _ = _peaks()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak_tf = float(json.load(f).get("bf16_tflops", 0.0)) or 1590.0
    except OSError:
        peak_tf = 1590.0   # fallback figure
    out = {}

    def timed(fn, reps):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3

    side = torch.cuda.Stream(device=dev)

    def timed_graph(issue, reps):
        """`issue(stream_ptr)` launches one pass on the given stream; the pass is captured once and
        replayed (as the headline step is), so that a Python loop does not bound 5-20 us kernels.
        Seconds per pass."""
        with torch.cuda.stream(side):
            issue(side.cuda_stream)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                issue(torch.cuda.current_stream().cuda_stream)
            for _ in range(2):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(reps):
                g.replay()
            e1.record(side)
            side.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3

    # Q4_K projection sweep at larger token counts (bf16 in / out), one pass over all layers
    for mm in (16, 128, 512):
        xs = {k: torch.randn(mm, k, device=dev, generator=gen).to(torch.bfloat16) for k in (W.HIDDEN, W.FFN)}
        ys = {n: torch.empty(mm, n, dtype=torch.bfloat16, device=dev) for n in (W.HIDDEN, W.KV_DIM, W.FFN)}

        def sweep(stream_ptr):
            for lw in layers:
                for name, n, k in W.PROJECTIONS:
                    st = lib.nnq_linear(ctx, lw[name].handle(), xs[k].data_ptr(), api.BF16, mm, None,
                                        ys[n].data_ptr(), api.BF16, stream_ptr)
                    if st != 0:
                        backend.check(st)

        sec = timed_graph(sweep, 2)
        algo = W.layer_bytes(mm).algorithmic * len(layers)
        flops = 2.0 * mm * sum(n * k for _, n, k in W.PROJECTIONS) * len(layers)
        row = {"ms_per_pass": sec * 1e3, "gbs": algo / sec / 1e9, "tflops": flops / sec / 1e12}
        if mm <= 16:
            row["bound"], row["frac"] = "hbm", algo / sec / 1e9 / peak_hbm
        else:
            row["bound"], row["frac"] = "tensor", flops / sec / 1e12 / peak_tf
        out[f"q4_k_projection_sweep_m{mm}"] = row

    def gemv(fmt, gen_fn, n, k, copies, x_f32, reps):
        ws = []
        for _ in range(copies):
            raw = gen_fn(torch, gen, n, k)
            ws.append(api.DeviceWeight.from_device(backend, fmt, raw, n, k))
            del raw
        x = torch.randn(1, k, device=dev, generator=gen)
        if not x_f32:
            x = x.to(torch.bfloat16)
        y = torch.empty(1, n, dtype=torch.float32, device=dev)
        xdt = api.F32 if x_f32 else api.BF16

        def one_pass(stream_ptr):
            for w in ws:
                st = lib.nnq_linear(ctx, w.handle(), x.data_ptr(), xdt, 1, None, y.data_ptr(), api.F32, stream_ptr)
                if st != 0:
                    backend.check(st)

        sec = timed_graph(one_pass, reps) / copies
        algo = algorithmic_bytes(fmt, 1, n, k, 4 if x_f32 else 2, 4)
        for w in ws:
            w.release()
        return {"us": sec * 1e6, "gbs": algo / sec / 1e9, "bound": "hbm", "frac": algo / sec / 1e9 / peak_hbm,
                "weights_rotated": copies}

    # ---- the M = 1 sweep issued other ways (same weights, same products) ----
    # (a) the products are independent (distinct input and output buffers), so they may run
    #     concurrently: the same 144 launches dealt over four streams of one captured graph;
    # (b) the compiled plan: all 252 products in one persistent kernel, every group waiting for the
    #     one before it (the chain a decoder imposes), and with the waits the buffer analysis allows
    #     it to drop (none are needed here).
    try:
        out["q4_k_projection_sweep_m1_variants"] = sweep_variants(torch, backend, layers, gen, dev, peak_hbm)
    except Exception as e:   # a side measurement must not take the headline down
        out["q4_k_projection_sweep_m1_variants"] = {"error": str(e)[:200]}

    # ---- large prefill, Qwen3-32B layer shapes, 4096 tokens (tensor-core path) ----
    try:
        out["qwen3_32b_prefill_m4096"] = prefill_32b(torch, backend, gen, dev, peak_tf, timed)
    except Exception as e:
        out["qwen3_32b_prefill_m4096"] = {"error": str(e)[:200]}

    # ---- gpt-oss-20b MoE block, MXFP4 experts: 64-token decode batch and 4096-token prefill ----
    try:
        out["gptoss_20b_moe_block"] = moe_block(torch, backend, gen, dev, peak_hbm, peak_tf, timed)
    except Exception as e:
        out["gptoss_20b_moe_block"] = {"error": str(e)[:200]}

    out["qwen3_8b_decode_ctx2048"] = decode_tokens_per_s(torch, backend, layers, gen, dev, peak_hbm)
    out["q8_0_gemv_4096x4096_f32_m1"] = gemv(QuantFormat.Q8_0, W.gen_q8_0_device, 4096, 4096, 10, True, 40)
    out["q6_k_gemv_151936x4096_bf16_m1"] = gemv(QuantFormat.Q6_K, W.gen_q6_k_device, 151936, 4096, 1, False, 10)

    def int8_gemv(n, k, reps):
        q = torch.randint(0, 256, (n, k), dtype=torch.uint8, device=dev, generator=gen)
        scale = torch.rand(n, device=dev, generator=gen) * 1e-3
        zp = torch.randint(-20, 20, (n,), dtype=torch.int32, device=dev, generator=gen)
        x = torch.randn(1, k, device=dev, generator=gen)
        y = torch.empty(1, n, dtype=torch.float32, device=dev)

        def one(stream_ptr):
            st = lib.nnq_int8_linear(ctx, q.data_ptr(), scale.data_ptr(), zp.data_ptr(), n, k, x.data_ptr(), api.F32, 1, None,
                                     y.data_ptr(), api.F32, stream_ptr)
            if st != 0:
                backend.check(st)

        sec = timed_graph(one, reps)
        algo = n * k + n * 8 + k * 4 + n * 4   # one byte per weight, scale + zero point per row, x and y once
        return {"us": sec * 1e6, "gbs": algo / sec / 1e9, "bound": "hbm", "frac": algo / sec / 1e9 / peak_hbm,
                "weights_rotated": 1}

    try:   # a side measurement must not take the headline down
        out["int8_w8a16_gemv_151936x4096_f32_m1"] = int8_gemv(151936, 4096, 10)
    except Exception as e:
        out["int8_w8a16_gemv_151936x4096_f32_m1"] = {"error": str(e)[:200]}
    def group_gemv(bits, n, k, g, reps, gptq_form=False):
        """One-token product over INT4 / INT8 per-group codes (or a GPTQ-packed weight), bf16 activations;
        `copies` weights are rotated so that a pass reads more than L2 holds."""
        import ctypes as ct
        from nn_b200 import gptq as G
        from nn_b200 import weight_quant as wq
        copies = max(1, int(300e6 // (n * k * bits // 8)) + 1)
        ws = []
        for _ in range(copies):
            if gptq_form:
                qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8, n), dtype=torch.int32, device=dev, generator=gen)
                qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // g, n // 8), dtype=torch.int32, device=dev, generator=gen)
                sc = torch.rand(k // g, n, device=dev, generator=gen) * 1e-2
                ws.append(G.load_gptq_linear(qw, sc, qz, None, g, backend)._packed)
            else:
                q = torch.randint(0, 256, (n * k * bits // 8,), dtype=torch.uint8, device=dev, generator=gen)
                sc = torch.rand(n * (k // g), device=dev, generator=gen) * 1e-2
                zp = torch.randint(-4, 4, (n * (k // g),), dtype=torch.int32, device=dev, generator=gen)
                cfgq = wq.QuantizationConfig(wq.QuantDtype.Int4 if bits == 4 else wq.QuantDtype.Int8, g, False)
                ws.append(wq.QuantizedTensor(q, sc, zp, cfgq, [n, k], backend).device_weight())
        x = torch.randn(1, k, device=dev, generator=gen).to(torch.bfloat16)
        y = torch.empty(1, n, dtype=torch.float32, device=dev)

        def one_pass(stream_ptr):
            for w in ws:
                st = lib.nnq_gq_linear(w._handle, x.data_ptr(), api.BF16, 1, None, y.data_ptr(), api.F32, stream_ptr)
                if st != 0:
                    backend.check(st)

        sec = timed_graph(one_pass, reps) / copies
        algo = n * k * bits // 8 + n * (k // g) * 8 + k * 2 + n * 4   # codes, scale + zero point per group, x and y once
        for w in ws:
            w.release()
        return {"us": sec * 1e6, "gbs": algo / sec / 1e9, "bound": "hbm", "frac": algo / sec / 1e9 / peak_hbm,
                "weights_rotated": copies, "group_size": g}

    for key, args_ in (("int4_per_group_gemv_12288x4096_g128_bf16_m1", (4, 12288, 4096, 128, 40)),
                       ("int8_per_group_gemv_12288x4096_g128_bf16_m1", (8, 12288, 4096, 128, 40)),
                       ("gptq_int4_gemv_12288x4096_g128_bf16_m1", (4, 12288, 4096, 128, 40, True)),
                       ("int4_per_group_gemv_151936x4096_g128_bf16_m1", (4, 151936, 4096, 128, 10))):
        try:
            out[key] = group_gemv(*args_)
        except Exception as e:
            out[key] = {"error": str(e)[:200]}
    backend.device_status()
    return out


def decode_tokens_per_s(torch, backend, layers, gen, dev, peak_hbm, prompt=2048, new_tokens=256, tp=(0, 1), peer=None,
                        full_layers=None, dist=None):
    """Batch-1 greedy decode of a Qwen3-8B-shaped model (the bench's 36 Q4_K layers, a Q6_K
    vocabulary projection, bf16 embedding, unit norms): a prompt of 2048 random ids through the prompt
    pass, then 256 greedy tokens timed from position 2048.
    With tensor parallelism the vocabulary projection is split by rows over the ranks and the greedy
    token is agreed on through the communicator; before the timed run, 8 tokens of the
    tensor-parallel decoder are compared with the single-GPU decoder over the unsharded weights
    (rank 0 holds them: `full_layers`)."""
    from nn_b200 import api, decoder
    from nn_b200 import workload as W
    from nn_b200.formats import QuantFormat
    if len(layers) != W.LAYERS:
        return None
    rank, world = tp
    cfg = decoder.DecoderConfig(max_seq=prompt + new_tokens + 8, act_dtype=api.BF16, tp_rank=rank, tp_world=world)
    dec = decoder.Decoder(backend, cfg)
    if peer is not None:
        dec.set_comm(peer)
    ones_h = torch.ones(cfg.hidden, device=dev)
    ones_d = torch.ones(cfg.head_dim, device=dev)

    def set_layers(d, lws):
        for li, lw in enumerate(lws):
            d.set_layer(li, lw["q_proj"], lw["k_proj"], lw["v_proj"], lw["o_proj"], lw["gate_proj"], lw["up_proj"],
                        lw["down_proj"], ones_h, ones_h, ones_d, ones_d)

    set_layers(dec, layers)
    raw = W.gen_q6_k_device(torch, gen, cfg.vocab, cfg.hidden)
    vocab_parallel = world > 1 and cfg.vocab % world == 0
    head = api.DeviceWeight.from_device(backend, QuantFormat.Q6_K, raw, cfg.vocab, cfg.hidden,
                                        shard=(0, rank, world) if vocab_parallel else None)
    head_full = None
    if full_layers is not None:
        head_full = api.DeviceWeight.from_device(backend, QuantFormat.Q6_K, raw, cfg.vocab, cfg.hidden)
    del raw
    embed = torch.randn(cfg.vocab, cfg.hidden, device=dev, generator=gen).to(torch.bfloat16)
    dec.set_head(embed, ones_h, head)
    kc, vc, logits, toks = dec.buffers()
    stream = torch.cuda.Stream(device=dev)
    # ---- the prompt: 2048 random ids through the decoder (M > 1 products, causal attention) ----
    import numpy as np
    ids = np.random.default_rng(2048).integers(0, cfg.vocab, size=prompt).tolist()   # same ids on every rank
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    dec.prefill(ids, 0, stream)
    prompt_s = time.perf_counter() - t0
    first_token, _, _ = dec.state(stream)

    # ---- parity of the tensor-parallel decoder (N > 1), before anything is timed ----
    parity = None
    if world > 1 and dist is not None:
        check_tokens = 8
        with torch.cuda.stream(stream):
            for _ in range(check_tokens):
                dec.step(stream)
            stream.synchronize()
        backend.device_status(stream)
        mine = [first_token] + toks[prompt:prompt + check_tokens].cpu().tolist()
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        same = all(g_ == gathered[0] for g_ in gathered)
        verdict = {"prompt_tokens": prompt, "decode_tokens": check_tokens, "same_tokens_on_all_ranks": bool(same)}
        if full_layers is not None:
            cfg1 = decoder.DecoderConfig(max_seq=cfg.max_seq, act_dtype=api.BF16)
            dec1 = decoder.Decoder(backend, cfg1)
            set_layers(dec1, full_layers)
            dec1.set_head(embed, ones_h, head_full)
            _, _, logits1, toks1 = dec1.buffers()
            dec1.prefill(ids, 0, stream)
            first1, _, _ = dec1.state(stream)
            with torch.cuda.stream(stream):
                for _ in range(check_tokens):
                    dec1.step(stream)
                stream.synchronize()
            backend.device_status(stream)
            want = [first1] + toks1[prompt:prompt + check_tokens].cpu().tolist()
            rows = slice(rank * cfg.vocab // world, (rank + 1) * cfg.vocab // world) if vocab_parallel else slice(0, cfg.vocab)
            err = float((logits[rows] - logits1[rows]).abs().max() / logits1.abs().max())
            # the prompt pass runs on the tensor cores (bf16 operands), where the split along K changes
            # the rounding of partial sums: the 1e-2 class, not the 2e-3 of the f32-accumulating decode
            verdict.update({"tokens_equal_single_gpu": bool(mine == want), "last_logits_max_rel_err": err,
                            "logits_tolerance": 1e-2})
            dec1.release()
            head_full.release()
        flag = [verdict if rank == 0 else None]
        dist.broadcast_object_list(flag, src=0)
        verdict = flag[0]
        verdict["same_tokens_on_all_ranks"] = bool(same)
        verdict["ok"] = bool(same and verdict.get("last_logits_max_rel_err", 0.0) <= 1e-2)
        parity = verdict

    with torch.cuda.stream(stream):
        dec.reset(1, prompt, stream)
        dec.step(stream)
        stream.synchronize()
        dec.reset(1, prompt, stream)
        launches0 = backend.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            dec.step(torch.cuda.current_stream())
        per_token = backend.launch_count() - launches0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(new_tokens):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    backend.device_status(stream)
    sec = e0.elapsed_time(e1) * 1e-3 / new_tokens
    _, pos, steps = dec.state()
    ctx_mid = prompt + new_tokens // 2
    # per GPU: its shard of the layers, of the caches and of the vocabulary projection
    head_bytes = cfg.vocab * (cfg.hidden // 256) * 210 // (world if vocab_parallel else 1)
    weights = W.layer_bytes(1).weights * W.LAYERS // world + head_bytes
    kv = 2 * cfg.n_layers * (cfg.n_kv_heads // world) * cfg.head_dim * 4 * ctx_mid
    out = {"tokens_per_s": 1.0 / sec, "tp": world, "ms_per_token": sec * 1e3, "new_tokens": new_tokens, "prompt_positions": prompt,
           "kernels_per_token": int(per_token), "end_position": pos, "steps": steps,
           "hbm_bytes_per_token_per_gpu": weights + kv, "gbs_per_gpu": (weights + kv) / sec / 1e9, "bound": "hbm",
           "frac": (weights + kv) / sec / 1e9 / peak_hbm, "kv_cache": "f32", "product_inputs": "bf16",
           "vocabulary_projection": "split by rows over the ranks, distributed argmax" if vocab_parallel else "whole on this GPU",
           "prompt": "2048 random ids through nnq_decoder_prefill (tensor-core products, causal attention)",
           "prompt_pass_s": prompt_s, "prompt_tokens_per_s": prompt / prompt_s,
           "parity": parity}
    dec.release()
    head.release()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="nnq", choices=["nnq", "reference"])
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-others", action="store_true")
    ap.add_argument("--no-fused", action="store_true", help="N > 1: separate all-reduce kernel after the row-parallel products")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    run_nnq(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
