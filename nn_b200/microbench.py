"""Device-timed runs of single products of the library (weights drawn on the device).

  python -m nn_b200.microbench linear --fmt q4_k --n 12288 --k 4096 --m 16 [--x f32] [--path tensor]
  python -m nn_b200.microbench moe --layout nk --tokens 64
  python -m nn_b200.microbench codec --fmt q4_k_ggml --elements 268435456
  python -m nn_b200.microbench int8 --n 12288 --k 4096 --m 1
  python -m nn_b200.microbench groupq --bits 4 --n 12288 --k 4096 --group 128 --m 1 [--gptq]
  python -m nn_b200.microbench decoder --layers 4 --pos 2048 [--eager]

`linear` rotates `--copies` distinct weights so that every call streams its weight from HBM
(more bytes in rotation than L2 holds unless --copies says otherwise); `moe` times one
mixture-of-experts block of the gpt-oss expert geometry. `codec` times the block
encoder (where the reference has one) and the decoder over one flat tensor larger than L2.
`groupq` times the product over INT4 / INT8 per-group codes (or a GPTQ-packed weight), replayed
from a CUDA graph so that the host loop does not bound 20 us kernels. `decoder` builds a
Qwen3-8B-shaped decoder of `--layers` Q4_K layers (no vocabulary head worth timing: a 1024-row Q6_K
one), places it at `--pos` and replays one captured step; `--eager` issues the launches one by one
instead (the form a profiler can list).
CUDA events around `--reps` calls after 3 warm-up calls; one line per run.
"""
from __future__ import annotations

import argparse
import ctypes


def _formats():
    from .formats import QuantFormat as Q
    return {"q8_0": Q.Q8_0, "q4_k": Q.Q4_K, "q6_k": Q.Q6_K, "mxfp4": Q.MXFP4_SPLIT, "q4_0": Q.Q4_0, "q4_1": Q.Q4_1}


def _draw(torch, gen, fmt, n, k):
    """Raw blocks with uniform code bytes and small finite scales; (data, scales or None)."""
    from . import workload as W
    from .formats import QuantFormat as Q
    dev = gen.device
    if fmt == Q.Q4_K:
        return W.gen_q4_k_device(torch, gen, n, k), None
    if fmt == Q.Q8_0:
        return W.gen_q8_0_device(torch, gen, n, k), None
    if fmt == Q.Q6_K:
        return W.gen_q6_k_device(torch, gen, n, k), None
    if fmt == Q.MXFP4_SPLIT:
        data = torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device=dev, generator=gen)
        scales = torch.randint(119, 128, (n * k // 32,), dtype=torch.uint8, device=dev, generator=gen)
        return data, scales
    nb, bs = n * k // 32, (18 if fmt == Q.Q4_0 else 20)
    out = torch.randint(0, 256, (nb, bs), dtype=torch.uint8, device=dev, generator=gen)
    out[:, 1] = 0x20   # high byte of the fp16 scale: a small finite value
    if fmt == Q.Q4_1:
        out[:, 3] = 0x20
    return out.reshape(-1), None


def _timed(torch, fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e-3


def run_linear(a):
    import torch

    from . import api
    from .formats import algorithmic_bytes
    fmt = _formats()[a.fmt]
    b = api.gpu_backend()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1)
    ws = []
    for _ in range(a.copies):
        data, scales = _draw(torch, gen, fmt, a.n, a.k)
        ws.append(api.DeviceWeight.from_device(b, fmt, data, a.n, a.k, scales=scales))
        del data, scales
    x = torch.randn(a.m, a.k, device=dev, generator=gen)
    xdt = api.F32
    if a.x == "bf16":
        x, xdt = x.to(torch.bfloat16), api.BF16
    y = torch.empty(a.m, a.n, dtype=torch.float32, device=dev)
    b.set_path({"auto": api.PATH_AUTO, "generic": api.PATH_GENERIC, "skinny": api.PATH_SKINNY, "tensor": api.PATH_TENSOR}[a.path])
    i = [0]

    def one():
        b.check(b._lib.nnq_linear(b._ctx, ws[i[0] % a.copies].handle(), x.data_ptr(), xdt, a.m, None, y.data_ptr(), api.F32, None))
        i[0] += 1

    sec = _timed(torch, one, a.reps)
    b.set_path(api.PATH_AUTO)
    b.device_status()
    algo = algorithmic_bytes(fmt, a.m, a.n, a.k, 4 if a.x == "f32" else 2, 4)
    print(f"linear {a.fmt} N={a.n} K={a.k} M={a.m} x={a.x} path={a.path}: {sec * 1e6:.1f} us, "
          f"{algo / sec / 1e9:.0f} GB/s algorithmic, {2.0 * a.m * a.n * a.k / sec / 1e12:.1f} TFLOP/s", flush=True)
    for w in ws:
        w.release()


def run_moe(a):
    import torch

    from . import api
    b = api.gpu_backend()
    lib, ctx = b._lib, b._ctx
    dev = torch.device("cuda", 0)
    E, H, I, k = a.experts, a.hidden, a.inter, a.top_k
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)

    def u8(n, lo=0, hi=256):
        return torch.randint(lo, hi, (n,), dtype=torch.uint8, device=dev, generator=gen)

    rw = (torch.randn(E, H, device=dev, generator=gen) * 0.5).float()
    rb = torch.zeros(E, device=dev)
    bgu, bd = torch.zeros(E, 2 * I, device=dev), torch.zeros(E, H, device=dev)
    layout, fmt = (0, 8) if a.layout == "kn" else (1, 7)   # [E,K,N] nn-gptoss | per-expert [N,K] split MXFP4
    if a.format == "mxfp4":
        gu, gus = u8(E * H * 2 * I // 2), u8(E * H * 2 * I // 32, 119, 128)
        dn, dns = u8(E * I * H // 2), u8(E * I * H // 32, 119, 128)
    else:
        # [N, K] experts in a GGUF block format: random codes, every f16 scale field a small finite number
        if a.layout != "nk":
            raise SystemExit("--format other than mxfp4 needs --layout nk")
        fmt, elems, nbytes, f16_at = {"q8_0": (2, 32, 34, (0,)), "q4_k": (3, 256, 144, (0, 2))}[a.format]
        if H % elems or I % elems:
            raise SystemExit(f"--hidden and --inter must be multiples of {elems} for {a.format}")

        def blocks(n):
            t = u8(n // elems * nbytes).view(-1, nbytes)
            for o in f16_at:
                t[:, o + 1] = 0x1C + (t[:, o + 1] & 3)   # f16 high byte: exponent 7..8 of 15 -> about 2^-8
            return t.reshape(-1)

        gu, dn = blocks(E * H * 2 * I), blocks(E * I * H)
        gus = dns = torch.empty(0, dtype=torch.uint8, device=dev)
    h = ctypes.c_void_p()
    b.check(lib.nnq_moe_create(ctx, E, H, I, k, ctypes.c_float(7.0), rw.data_ptr(), rb.data_ptr(), layout, fmt,
                               gu.data_ptr(), gu.numel(), gus.data_ptr() if gus.numel() else None, gus.numel(), bgu.data_ptr(),
                               dn.data_ptr(), dn.numel(), dns.data_ptr() if dns.numel() else None, dns.numel(), bd.data_ptr(),
                               ctypes.byref(h)))
    T = a.tokens
    x = torch.randn(T, H, device=dev, generator=gen).to(torch.bfloat16)
    y = torch.empty(T, H, device=dev)
    sec = _timed(torch, lambda: b.check(lib.nnq_moe_forward(ctx, h, x.data_ptr(), api.BF16, T, y.data_ptr(), None)), a.reps)
    b.device_status()
    wbytes = gu.numel() + gus.numel() + dn.numel() + dns.numel()
    touched = wbytes * min(1.0, T * k / E)
    print(f"moe layout={a.layout} {a.format} E={E} hidden={H} inter={I} top{k} tokens={T}: {sec * 1e6:.0f} us, "
          f"about {touched / 1e6:.0f} MB of expert weights touched -> {touched / sec / 1e9:.0f} GB/s", flush=True)
    lib.nnq_moe_destroy(h)


def run_codec(a):
    import torch

    from . import api
    from .formats import GEOMETRY, QuantFormat as Q
    names = dict(_formats(), q4_k_ggml=Q.Q4_K_GGML, mxfp4_core=Q.MXFP4_CORE, mxfp4_gptoss=Q.MXFP4_GPTOSS, q5_0=Q.Q5_0,
                 q5_1=Q.Q5_1, q2_k=Q.Q2_K, q3_k=Q.Q3_K, q5_k=Q.Q5_K)
    fmt = names[a.fmt]
    b = api.gpu_backend()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    g = GEOMETRY[fmt]
    n = a.elements // g.elems * g.elems
    nb = n // g.elems
    src = torch.randn(n, device=dev, generator=gen) * 0.05
    out = torch.empty(n, device=dev)
    if fmt in (Q.Q4_K_GGML, Q.MXFP4_CORE, Q.MXFP4_GPTOSS):
        sec = _timed(torch, lambda: api.quantize(src, fmt, b), a.reps)
        blocks, scales = api.quantize(src, fmt, b)
        moved = n * 4 + nb * (g.bytes + g.scale_bytes)
        print(f"encode {a.fmt} {n} weights: {sec * 1e3:.2f} ms, {moved / sec / 1e9:.0f} GB/s "
              f"({n * 4 / 1e6:.0f} MB read, {nb * (g.bytes + g.scale_bytes) / 1e6:.0f} MB written)", flush=True)
    else:
        blocks = torch.randint(0, 256, (nb, g.bytes), dtype=torch.uint8, device=dev, generator=gen)
        blocks[:, 1] = 0x20   # keeps most f16 scale fields small and finite
        blocks, scales = blocks.reshape(-1), None
    decoded = ctypes.c_int64()
    sp, sn = (scales.data_ptr(), scales.numel()) if scales is not None else (None, 0)

    def dec():
        b.check(b._lib.nnq_dequantize_raw(b._ctx, int(fmt), blocks.data_ptr(), blocks.numel(), sp, sn, n, out.data_ptr(),
                                          ctypes.byref(decoded), None))

    sec = _timed(torch, dec, a.reps)
    b.device_status()
    moved = n * 4 + nb * (g.bytes + g.scale_bytes)
    print(f"decode {a.fmt} {n} weights: {sec * 1e3:.2f} ms, {moved / sec / 1e9:.0f} GB/s "
          f"({nb * (g.bytes + g.scale_bytes) / 1e6:.0f} MB read, {n * 4 / 1e6:.0f} MB written)", flush=True)


def run_int8(a):
    import torch

    from . import api, int8
    b = api.gpu_backend()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    layers = []
    for _ in range(a.copies):
        q = torch.randint(0, 256, (a.n, a.k), dtype=torch.uint8, device=dev, generator=gen)
        p = int8.Int8QuantParams(torch.rand(a.n, device=dev, generator=gen) * 1e-3,
                                 torch.randint(-20, 20, (a.n,), dtype=torch.int32, device=dev, generator=gen))
        layers.append(int8.Int8Linear(q, p, None, b))
    x = torch.randn(a.m, a.k, device=dev, generator=gen)
    if a.x == "bf16":
        x = x.to(torch.bfloat16)
    i = [0]

    def one():
        layers[i[0] % a.copies].forward(x, check_finite=False)
        i[0] += 1

    sec = _timed(torch, one, a.reps)
    algo = a.n * a.k + a.n * 8 + a.m * a.k * (4 if a.x == "f32" else 2) + a.m * a.n * 4
    print(f"int8 linear N={a.n} K={a.k} M={a.m} x={a.x}: {sec * 1e6:.1f} us, {algo / sec / 1e9:.0f} GB/s algorithmic, "
          f"{2.0 * a.m * a.n * a.k / sec / 1e12:.2f} TFLOP/s", flush=True)


def run_groupq(a):
    import torch

    from . import api, gptq
    from . import weight_quant as wq
    b = api.gpu_backend()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    n, k, g, bits = a.n, a.k, a.group, a.bits
    copies = max(1, int(300e6 // (n * k * bits // 8)) + 1)
    ws = []
    for _ in range(copies):
        if a.gptq:
            qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 8, n), dtype=torch.int32, device=dev, generator=gen)
            qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // g, n // 8), dtype=torch.int32, device=dev, generator=gen)
            sc = torch.rand(k // g, n, device=dev, generator=gen) * 1e-2
            ws.append(gptq.load_gptq_linear(qw, sc, qz, None, g, b)._packed)
        else:
            q = torch.randint(0, 256, (n * k * bits // 8,), dtype=torch.uint8, device=dev, generator=gen)
            sc = torch.rand(n * (k // g), device=dev, generator=gen) * 1e-2
            zp = torch.randint(-4, 4, (n * (k // g),), dtype=torch.int32, device=dev, generator=gen)
            cfg = wq.QuantizationConfig(wq.QuantDtype.Int4 if bits == 4 else wq.QuantDtype.Int8, g, False)
            ws.append(wq.QuantizedTensor(q, sc, zp, cfg, [n, k], b).device_weight())
    x = torch.randn(a.m, k, device=dev, generator=gen).to(torch.bfloat16)
    y = torch.empty(a.m, n, dtype=torch.float32, device=dev)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        def pass_over_copies():
            for w in ws:
                b.check(b._lib.nnq_gq_linear(w._handle, x.data_ptr(), api.BF16, a.m, None, y.data_ptr(), api.F32, st.cuda_stream))
        pass_over_copies()
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            pass_over_copies()
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(a.reps):
            graph.replay()
        e1.record(st)
        st.synchronize()
    b.device_status()
    sec = e0.elapsed_time(e1) * 1e-3 / a.reps / copies
    algo = n * k * bits // 8 + n * (k // g) * 8 + a.m * k * 2 + a.m * n * 4
    print(f"groupq {'gptq ' if a.gptq else ''}int{bits} N={n} K={k} group={g} M={a.m}: {sec * 1e6:.1f} us, "
          f"{algo / sec / 1e9:.0f} GB/s algorithmic ({copies} weights in rotation)", flush=True)
    for w in ws:
        w.release()


def run_decoder(a):
    import torch

    from . import api, decoder
    from . import workload as W
    from .formats import QuantFormat as Q
    b = api.gpu_backend()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    cfg = decoder.DecoderConfig(n_layers=a.layers, vocab=1024, max_seq=a.pos + 64, act_dtype=api.BF16)
    dec = decoder.Decoder(b, cfg)
    oh, od = torch.ones(cfg.hidden, device=dev), torch.ones(cfg.head_dim, device=dev)
    keep = []
    for li in range(a.layers):
        lw = {}
        for name, n, k in W.PROJECTIONS:
            raw = W.gen_q4_k_device(torch, gen, n, k)
            lw[name] = api.DeviceWeight.from_device(b, Q.Q4_K, raw, n, k)
            del raw
        keep.append(lw)
        dec.set_layer(li, lw["q_proj"], lw["k_proj"], lw["v_proj"], lw["o_proj"], lw["gate_proj"], lw["up_proj"],
                      lw["down_proj"], oh, oh, od, od)
    head = api.DeviceWeight.from_device(b, Q.Q6_K, W.gen_q6_k_device(torch, gen, cfg.vocab, cfg.hidden), cfg.vocab, cfg.hidden)
    embed = torch.randn(cfg.vocab, cfg.hidden, device=dev, generator=gen).to(torch.bfloat16)
    dec.set_head(embed, oh, head)
    kc, vc, _, _ = dec.buffers()
    kc.normal_(generator=gen)
    vc.normal_(generator=gen)
    st = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(st):
        dec.reset(1, a.pos, st)
        dec.step(st)
        st.synchronize()
        if a.eager:
            def one():
                dec.reset(1, a.pos, st)
                dec.step(st)
        else:
            dec.reset(1, a.pos, st)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                dec.step(torch.cuda.current_stream())
            def one():
                graph.replay()
        for _ in range(3):
            one()
        dec.reset(1, a.pos, st)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(a.reps):
            one()
        e1.record(st)
        st.synchronize()
    b.device_status(st)
    ms = e0.elapsed_time(e1) / a.reps
    print(f"decoder step, {a.layers} layers, context {a.pos}.., {'eager' if a.eager else 'graph'}: {ms * 1e3:.1f} us per token, "
          f"{ms * 1e3 / a.layers:.1f} us per layer", flush=True)
    dec.release()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("linear")
    p.add_argument("--fmt", default="q4_k", choices=sorted(_formats()))
    p.add_argument("--n", type=int, default=4096)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--m", type=int, default=1)
    p.add_argument("--x", default="bf16", choices=["bf16", "f32"])
    p.add_argument("--path", default="auto", choices=["auto", "generic", "skinny", "tensor"])
    p.add_argument("--copies", type=int, default=8)
    p.add_argument("--reps", type=int, default=40)
    p = sub.add_parser("moe")
    p.add_argument("--layout", default="nk", choices=["nk", "kn"])
    p.add_argument("--format", default="mxfp4", choices=["mxfp4", "q8_0", "q4_k"])
    p.add_argument("--tokens", type=int, default=64)
    p.add_argument("--experts", type=int, default=32)
    p.add_argument("--hidden", type=int, default=2880)
    p.add_argument("--inter", type=int, default=2880)
    p.add_argument("--top-k", type=int, default=4)
    p.add_argument("--reps", type=int, default=10)
    p = sub.add_parser("codec")
    p.add_argument("--fmt", default="q4_k_ggml")
    p.add_argument("--elements", type=int, default=1 << 28)
    p.add_argument("--reps", type=int, default=5)
    p = sub.add_parser("int8")
    p.add_argument("--n", type=int, default=12288)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--m", type=int, default=1)
    p.add_argument("--x", default="f32", choices=["bf16", "f32"])
    p.add_argument("--copies", type=int, default=8)
    p.add_argument("--reps", type=int, default=40)
    p = sub.add_parser("groupq")
    p.add_argument("--bits", type=int, default=4, choices=[4, 8])
    p.add_argument("--n", type=int, default=12288)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--group", type=int, default=128)
    p.add_argument("--m", type=int, default=1)
    p.add_argument("--gptq", action="store_true")
    p.add_argument("--reps", type=int, default=20)
    p = sub.add_parser("decoder")
    p.add_argument("--layers", type=int, default=4)
    p.add_argument("--pos", type=int, default=2048)
    p.add_argument("--eager", action="store_true")
    p.add_argument("--reps", type=int, default=20)
    a = ap.parse_args()
    {"linear": run_linear, "moe": run_moe, "codec": run_codec, "int8": run_int8, "groupq": run_groupq,
     "decoder": run_decoder}[a.cmd](a)


if __name__ == "__main__":
    main()
