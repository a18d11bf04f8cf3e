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
    sample = "one layer (7 projections, 108.5 MB of Q4_K) per step: dequantize whole weight + nn-cpu row dot"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": 1, "layers_per_step": 1, "format": "Q4_K"},
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
    peer = comm.PeerComm(backend, rank, world, max_bytes=max(m, 2) * W.HIDDEN * 4) if world > 1 else None
    gen = torch.Generator(device=dev)
    gen.manual_seed(0x5EED)  # same weights on every rank, each keeps its shard

    # ---- weights: `layers` distinct layers, tensor-parallel shards when world > 1 ----
    layers = []
    for li in range(args.layers):
        lw = {}
        for name, n, k in W.PROJECTIONS:
            raw = W.gen_q4_k_device(torch, gen, n, k)
            shard = (W.TP_AXIS[name], rank, world) if world > 1 else None
            lw[name] = api.DeviceWeight.from_device(backend, QuantFormat.Q4_K, raw, n, k, shard=shard)
            del raw
        layers.append(lw)
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
    with torch.cuda.stream(stream):
        sp = VP(stream.cuda_stream)
        for _ in range(2):
            step(sp)
        stream.synchronize()
        backend.device_status(stream)
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
                    # dram__bytes_read+write per launch from the ncu capture summarised in profiles/ (2-layer
                    # case; per-launch traffic does not depend on the layer count): equal to the algorithmic
                    # bytes within 0.1 %
                    "traffic": bytes_per_launch * (27.18 / 27.17),
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
        dec = decode_tokens_per_s(torch, backend, layers, gen, dev, peak_hbm, tp=(rank, world), peer=peer)
        if dec is not None:
            t = torch.tensor([dec["ms_per_token"]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dec["ms_per_token"] = float(t.item())
            dec["tokens_per_s"] = 1e3 / dec["ms_per_token"]
        others = {"qwen3_8b_decode_ctx2048": dec}

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

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "m": m, "layers": args.layers, "format": "Q4_K",
                       "activations": "bf16", "outputs": "bf16", "accumulate": "f32",
                       "parallelism": f"tp{world}" if world > 1 else "single",
                       "weight_bytes_per_step": per_layer.weights * args.layers * world // world,
                       "l2_policy": "inputs larger than L2 (every step streams all layers' distinct weights)",
                       "cuda_graph": graph is not None,
                       "tokens_per_s_equiv": 1e3 / ms_per_step * (36 / args.layers)},
            "roofline": roofline, "clocks": clocks.summary(), "gpu_launches": int(launched),
            "e2e": e2e, "cpu_baseline": cpu, "other_configs": others,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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

    # Q4_K projection sweep at larger token counts (bf16 in / out), one pass over all layers
    for mm in (16, 128, 512):
        xs = {k: torch.randn(mm, k, device=dev, generator=gen).to(torch.bfloat16) for k in (W.HIDDEN, W.FFN)}
        ys = {n: torch.empty(mm, n, dtype=torch.bfloat16, device=dev) for n in (W.HIDDEN, W.KV_DIM, W.FFN)}

        def sweep():
            for lw in layers:
                for name, n, k in W.PROJECTIONS:
                    st = lib.nnq_linear(ctx, lw[name].handle(), xs[k].data_ptr(), api.BF16, mm, None,
                                        ys[n].data_ptr(), api.BF16, None)
                    if st != 0:
                        backend.check(st)

        sec = timed(sweep, 2)
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
        i = [0]

        def one():
            st = lib.nnq_linear(ctx, ws[i[0] % copies].handle(), x.data_ptr(), xdt, 1, None, y.data_ptr(), api.F32, None)
            i[0] += 1
            if st != 0:
                backend.check(st)

        sec = timed(one, reps)
        algo = algorithmic_bytes(fmt, 1, n, k, 4 if x_f32 else 2, 4)
        for w in ws:
            w.release()
        return {"us": sec * 1e6, "gbs": algo / sec / 1e9, "bound": "hbm", "frac": algo / sec / 1e9 / peak_hbm,
                "weights_rotated": copies}

    out["qwen3_8b_decode_ctx2048"] = decode_tokens_per_s(torch, backend, layers, gen, dev, peak_hbm)
    out["q8_0_gemv_4096x4096_f32_m1"] = gemv(QuantFormat.Q8_0, W.gen_q8_0_device, 4096, 4096, 10, True, 40)
    out["q6_k_gemv_151936x4096_bf16_m1"] = gemv(QuantFormat.Q6_K, W.gen_q6_k_device, 151936, 4096, 1, False, 10)

    def int8_gemv(n, k, reps):
        q = torch.randint(0, 256, (n, k), dtype=torch.uint8, device=dev, generator=gen)
        scale = torch.rand(n, device=dev, generator=gen) * 1e-3
        zp = torch.randint(-20, 20, (n,), dtype=torch.int32, device=dev, generator=gen)
        x = torch.randn(1, k, device=dev, generator=gen)
        y = torch.empty(1, n, dtype=torch.float32, device=dev)

        def one():
            st = lib.nnq_int8_linear(ctx, q.data_ptr(), scale.data_ptr(), zp.data_ptr(), n, k, x.data_ptr(), api.F32, 1, None,
                                     y.data_ptr(), api.F32, None)
            if st != 0:
                backend.check(st)

        sec = timed(one, reps)
        algo = n * k + n * 8 + k * 4 + n * 4   # one byte per weight, scale + zero point per row, x and y once
        return {"us": sec * 1e6, "gbs": algo / sec / 1e9, "bound": "hbm", "frac": algo / sec / 1e9 / peak_hbm,
                "weights_rotated": 1}

    try:   # a side measurement must not take the headline down
        out["int8_w8a16_gemv_151936x4096_f32_m1"] = int8_gemv(151936, 4096, 10)
    except Exception as e:
        out["int8_w8a16_gemv_151936x4096_f32_m1"] = {"error": str(e)[:200]}
    backend.device_status()
    return out


def decode_tokens_per_s(torch, backend, layers, gen, dev, peak_hbm, prompt=2048, new_tokens=256, tp=(0, 1), peer=None):
    """Batch-1 greedy decode of a Qwen3-8B-shaped model (the bench's 36 Q4_K layers, a Q6_K
    vocabulary projection, bf16 embedding, unit norms): 256 tokens from position 2048. The key /
    value caches of the 2048 earlier positions are filled with seeded random values, which stands
    in for the prompt pass: the cost of a decode step depends on the context length only."""
    from nn_b200 import api, decoder
    from nn_b200 import workload as W
    from nn_b200.formats import QuantFormat
    if len(layers) != W.LAYERS:
        return None
    cfg = decoder.DecoderConfig(max_seq=prompt + new_tokens + 8, act_dtype=api.BF16, tp_rank=tp[0], tp_world=tp[1])
    dec = decoder.Decoder(backend, cfg)
    if peer is not None:
        dec.set_comm(peer)
    ones_h = torch.ones(cfg.hidden, device=dev)
    ones_d = torch.ones(cfg.head_dim, device=dev)
    for li, lw in enumerate(layers):
        dec.set_layer(li, lw["q_proj"], lw["k_proj"], lw["v_proj"], lw["o_proj"], lw["gate_proj"], lw["up_proj"],
                      lw["down_proj"], ones_h, ones_h, ones_d, ones_d)
    raw = W.gen_q6_k_device(torch, gen, cfg.vocab, cfg.hidden)
    head = api.DeviceWeight.from_device(backend, QuantFormat.Q6_K, raw, cfg.vocab, cfg.hidden)
    del raw
    embed = torch.randn(cfg.vocab, cfg.hidden, device=dev, generator=gen).to(torch.bfloat16)
    dec.set_head(embed, ones_h, head)
    kc, vc, _, toks = dec.buffers()
    kc[:, :, :prompt].normal_(generator=gen)
    vc[:, :, :prompt].normal_(generator=gen)
    stream = torch.cuda.Stream(device=dev)
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
    # per GPU: its shard of the layers and of the caches, and the whole (replicated) vocabulary projection
    weights = W.layer_bytes(1).weights * W.LAYERS // tp[1] + cfg.vocab * (cfg.hidden // 256) * 210
    kv = 2 * cfg.n_layers * (cfg.n_kv_heads // tp[1]) * cfg.head_dim * 4 * ctx_mid
    out = {"tokens_per_s": 1.0 / sec, "tp": tp[1], "ms_per_token": sec * 1e3, "new_tokens": new_tokens, "prompt_positions": prompt,
           "kernels_per_token": int(per_token), "end_position": pos, "steps": steps,
           "hbm_bytes_per_token_per_gpu": weights + kv, "gbs_per_gpu": (weights + kv) / sec / 1e9, "bound": "hbm",
           "frac": (weights + kv) / sec / 1e9 / peak_hbm, "kv_cache": "f32", "product_inputs": "bf16",
           "prompt": "key/value caches of the first 2048 positions filled with seeded random values"}
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
