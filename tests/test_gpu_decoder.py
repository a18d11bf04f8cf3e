"""Device decode step (Qwen3-shaped, batch 1) against the numpy restatement of the reference's
decoder (oracle/qwen3_ref.py), through the C ABI: logits per step with f32 and bf16 product
inputs, the device-side token / position loop, and graph replay."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api, decoder
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc
from oracle import qwen3_ref as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _build(act_dtype, seed=11, backend=None, tp=(0, 1), comm=None, vocab_parallel=False, max_seq=48):
    """Decoder + dequantized model; with tp = (rank, world) the decoder holds that rank's shards."""
    rank, world = tp
    cfg = decoder.DecoderConfig(hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, n_layers=2, vocab=1024,
                                max_seq=max_seq, rms_eps=1e-6, rope_theta=1e6, act_dtype=act_dtype, tp_rank=rank, tp_world=world)
    s = F.Stream(seed)
    qdim, kvdim = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim

    b = backend or api.gpu_backend()
    dev = f"cuda:{b.device}"
    axis = {"q": 0, "k": 0, "v": 0, "gate": 0, "up": 0, "o": 1, "down": 1}

    def qw(fmt, n, k, sd, name=None):
        raw, sc = F.gen_weight(fmt, sd, n, k)
        t = api.QuantizedTensor(raw, fmt, [n, k], sc, b)
        if world > 1 and name in axis:
            t = t.shard(axis[name], rank, world)
        return t, orc.dequantize(fmt, raw, n * k, sc).reshape(n, k)

    def norm(n):
        return (1.0 + 0.1 * s.normal(n)).astype(np.float32)

    dec = decoder.Decoder(b, cfg)
    if comm is not None:
        dec.set_comm(comm)
    model = {"cfg": dict(n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, rms_eps=cfg.rms_eps),
             "rope": ref.rope_tables(cfg.head_dim, cfg.max_seq, cfg.rope_theta), "layers": []}
    keep = []
    for li in range(cfg.n_layers):
        shapes = [("q", qdim, cfg.hidden), ("k", kvdim, cfg.hidden), ("v", kvdim, cfg.hidden), ("o", cfg.hidden, qdim),
                  ("gate", cfg.ffn, cfg.hidden), ("up", cfg.ffn, cfg.hidden), ("down", cfg.hidden, cfg.ffn)]
        L, ws = {}, []
        for i, (name, n, k) in enumerate(shapes):
            w, wf = qw(Q.Q4_K, n, k, seed + 10 * li + i, name)
            # scale the synthetic weights to keep the residual stream of order one
            ws.append(w)
            L[name] = wf
        for name, n in (("in_norm", cfg.hidden), ("post_norm", cfg.hidden), ("q_norm", cfg.head_dim), ("k_norm", cfg.head_dim)):
            L[name] = norm(n)
        dec.set_layer(li, *ws, L["in_norm"], L["post_norm"], L["q_norm"], L["k_norm"])
        model["layers"].append(L)
        keep.append(ws)
    embed = (s.normal(cfg.vocab * cfg.hidden) * 0.5).astype(np.float32).reshape(cfg.vocab, cfg.hidden)
    embed_bf16 = torch.from_numpy(embed).to(dev).to(torch.bfloat16)
    model["embed"] = embed_bf16.float().cpu().numpy()
    model["final_norm"] = norm(cfg.hidden)
    head, head_f = qw(Q.Q6_K, cfg.vocab, cfg.hidden, seed + 99)
    if vocab_parallel and world > 1:
        head = head.shard(0, rank, world)     # this rank's rows of the vocabulary projection
    model["lm_head"] = head_f
    dec.set_head(embed_bf16, model["final_norm"], head)
    return cfg, dec, model, (keep, head, embed_bf16)


@pytest.mark.parametrize("act_dtype,tol", [(api.F32, 2e-3), (api.BF16, 1e-2)])
def test_decode_steps_match_reference_restatement(act_dtype, tol):
    """f32 product inputs: the reference's arithmetic, 2e-3. bf16 product inputs: 1e-2 against the
    restatement with the same rounding points (the normed states, the attention output and
    silu(gate) * up rounded to bf16 before their products), and a looser 3e-2 against the all-f32
    restatement -- input rounding of 2^-9 per element and product grows with depth, which is a
    property of feeding bf16 activations, not of the kernels."""
    cfg, dec, model, keep = _build(act_dtype)
    kc = np.zeros((cfg.n_layers, cfg.n_kv_heads, cfg.max_seq, cfg.head_dim), np.float32)
    vc = np.zeros_like(kc)
    kc32, vc32 = np.zeros_like(kc), np.zeros_like(kc)
    dec.reset(3, 0)
    token = 3
    _, _, logits_dev, tokens_dev = dec.buffers()
    agree = 0
    for pos in range(10):
        dec.step()
        nxt, npos, steps = dec.state()
        assert (npos, steps) == (pos + 1, pos + 1)
        got = logits_dev.cpu().numpy()
        # teacher-forced with the device's tokens
        want, want_tok = ref.step(model, token, pos, kc, vc, act_bf16=(act_dtype == api.BF16))
        assert np.all(np.isfinite(got))
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err <= tol, (pos, err)
        if act_dtype == api.BF16:
            want32, _ = ref.step(model, token, pos, kc32, vc32)
            assert np.max(np.abs(got - want32)) / np.max(np.abs(want32)) <= 3e-2
        assert nxt == ref.argmax_last(got)          # the device argmax is the argmax of the device logits
        top2 = np.sort(want)[-2:]
        if top2[1] - top2[0] > 4 * tol * np.max(np.abs(want)):
            assert nxt == want_tok
            agree += 1
        assert int(tokens_dev[pos].item()) == nxt
        token = nxt
    assert agree >= 1
    dec.backend.device_status()
    k_dev, v_dev, _, _ = dec.buffers()
    assert np.max(np.abs(k_dev[:, :, :10].cpu().numpy() - kc[:, :, :10])) <= (5e-3 if act_dtype == api.F32 else 5e-2)
    dec.release()


def test_context_full_is_reported_not_overwritten():
    """max_seq positions and no more: the host refuses the step past the end, and a captured graph
    replayed past the end raises the device status word instead of reusing the last slot."""
    b = api.gpu_backend()
    cfg, dec, model, keep = _build(api.BF16, seed=51)
    dec.reset(3, cfg.max_seq - 3)
    for _ in range(3):
        dec.step()
    tok, pos, steps = dec.state()
    assert (pos, steps) == (cfg.max_seq - 1, 3)
    b.device_status()
    with pytest.raises(api.Unsupported):
        dec.step()
    toks_before = dec.buffers()[3].clone()
    # graph replay: the host does not see the steps
    stream = torch.cuda.Stream(device=DEV)
    dec.reset(3, cfg.max_seq - 2, stream)
    with torch.cuda.stream(stream):
        dec.step(stream)
        stream.synchronize()
        dec.reset(3, cfg.max_seq - 2, stream)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            dec.step(torch.cuda.current_stream())
        g.replay()
        g.replay()
        stream.synchronize()
        b.device_status(stream)          # two steps fit
        tok2, pos2, steps2 = dec.state(stream)
        assert (pos2, steps2) == (cfg.max_seq - 1, 2)
        last = dec.buffers()[3][cfg.max_seq - 1].item()
        g.replay()                        # no position left
        stream.synchronize()
        with pytest.raises(api.Unsupported):
            b.device_status(stream)
        b.device_status(stream)           # reported once, then clear
        assert dec.state(stream) == (tok2, pos2, steps2)
        assert dec.buffers()[3][cfg.max_seq - 1].item() == last
    dec.reset(1, 0)
    dec.step()                            # usable again after a reset
    b.device_status()
    dec.release()


@pytest.mark.parametrize("act_dtype,tol", [(api.F32, 2e-3), (api.BF16, 1e-2)])
def test_qwen3_8b_width_steps_at_long_context(act_dtype, tol):
    """The benchmark's widths (hidden 4096, 32 query / 8 key-value heads, FFN 12288, vocabulary
    151936, Q4_K projections, Q6_K vocabulary projection), two layers, three tokens from position
    2048 over caches filled with seeded values. Weights are drawn on the device (the SplitMix64
    host stream would take minutes at this size) and dequantized by the oracle for the restatement."""
    from nn_b200 import workload as W
    b = api.gpu_backend()
    n_layers, start = 2, 2048
    cfg = decoder.DecoderConfig(n_layers=n_layers, max_seq=start + 8, act_dtype=act_dtype)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(808)
    rng = np.random.default_rng(809)

    def qw(fmt, genfn, n, k, scale):
        raw = genfn(torch, gen, n, k, scale)
        w = api.DeviceWeight.from_device(b, fmt, raw, n, k)
        return w, orc.dequantize(fmt, raw.cpu().numpy(), n * k).reshape(n, k)

    dec = decoder.Decoder(b, cfg)
    model = {"cfg": dict(n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, rms_eps=cfg.rms_eps),
             "rope": ref.rope_tables(cfg.head_dim, cfg.max_seq, cfg.rope_theta), "layers": []}
    keep = []
    qdim, kvdim = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    shapes = [("q", qdim, cfg.hidden), ("k", kvdim, cfg.hidden), ("v", kvdim, cfg.hidden), ("o", cfg.hidden, qdim),
              ("gate", cfg.ffn, cfg.hidden), ("up", cfg.ffn, cfg.hidden), ("down", cfg.hidden, cfg.ffn)]
    for li in range(n_layers):
        L, ws = {}, []
        for name, n, k in shapes:
            # block scales small enough that the residual stream stays of order one
            w, wf = qw(Q.Q4_K, W.gen_q4_k_device, n, k, 2e-5)
            ws.append(w)
            L[name] = wf
        for name, n in (("in_norm", cfg.hidden), ("post_norm", cfg.hidden), ("q_norm", cfg.head_dim), ("k_norm", cfg.head_dim)):
            L[name] = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        dec.set_layer(li, *ws, L["in_norm"], L["post_norm"], L["q_norm"], L["k_norm"])
        model["layers"].append(L)
        keep.append(ws)
    embed_bf16 = (torch.randn(cfg.vocab, cfg.hidden, device=DEV, generator=gen) * 0.5).to(torch.bfloat16)
    model["embed"] = embed_bf16.float().cpu().numpy()
    model["final_norm"] = (1.0 + 0.1 * rng.standard_normal(cfg.hidden)).astype(np.float32)
    head, head_f = qw(Q.Q6_K, W.gen_q6_k_device, cfg.vocab, cfg.hidden, 1e-3)
    model["lm_head"] = head_f
    dec.set_head(embed_bf16, model["final_norm"], head)
    kdev, vdev, logits_dev, _ = dec.buffers()
    kdev[:, :, :start].normal_(generator=gen)
    vdev[:, :, :start].normal_(generator=gen)
    kc, vc = kdev.cpu().numpy().copy(), vdev.cpu().numpy().copy()
    token = 1234
    dec.reset(token, start)
    for i in range(3):
        dec.step()
        nxt, npos, _ = dec.state()
        assert npos == start + i + 1
        got = logits_dev.cpu().numpy()
        want, _ = ref.step(model, token, start + i, kc, vc, act_bf16=(act_dtype == api.BF16))
        assert np.all(np.isfinite(got))
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err <= tol, (i, err)
        assert nxt == ref.argmax_last(got)
        token = nxt
    b.device_status()
    dec.release()
    head.release()
    for ws in keep:
        for w in ws:
            w.release()


@pytest.mark.parametrize("act_dtype", [api.F32, api.BF16])
@pytest.mark.parametrize("count", [9, 300])
def test_prompt_pass_matches_token_by_token(act_dtype, count):
    """A prompt of random ids through nnq_decoder_prefill (M > 1 products, causal mask; 300 tokens
    take two blocks of rows) against the restatement stepped token by token, then three greedy
    steps. The prompt products run on the tensor cores with bf16 operands: the 1e-2 class per
    product, 3e-2 on the logits after two layers (measured well below)."""
    cfg, dec, model, keep = _build(act_dtype, seed=61, max_seq=count + 8)
    rng = np.random.default_rng(62)
    prompt = rng.integers(0, cfg.vocab, size=count).tolist()
    kc = np.zeros((cfg.n_layers, cfg.n_kv_heads, cfg.max_seq, cfg.head_dim), np.float32)
    vc = np.zeros_like(kc)
    bf = act_dtype == api.BF16
    want = None
    for i, t in enumerate(prompt):
        want, want_tok = ref.step(model, t, i, kc, vc, act_bf16=bf)
    dec.prefill(prompt, 0)
    nxt, pos, steps = dec.state()
    assert (pos, steps) == (count, 1)
    k_dev, v_dev, logits_dev, tokens_dev = dec.buffers()
    got = logits_dev.cpu().numpy()
    assert np.all(np.isfinite(got))
    err = np.max(np.abs(got - want)) / np.max(np.abs(want))
    assert err <= 3e-2, err
    assert nxt == ref.argmax_last(got) and int(tokens_dev[count - 1].item()) == nxt
    # caches: every entry against the restatement's, relative to the largest entry
    assert np.max(np.abs(k_dev[:, :, :count].cpu().numpy() - kc[:, :, :count])) <= 5e-2 * np.max(np.abs(kc))
    assert np.max(np.abs(v_dev[:, :, :count].cpu().numpy() - vc[:, :, :count])) <= 5e-2 * np.max(np.abs(vc))
    # the decode loop continues from the prompt's caches (teacher-forced restatement)
    token = nxt
    for i in range(3):
        dec.step()
        want, _ = ref.step(model, token, count + i, kc, vc, act_bf16=bf)
        got = logits_dev.cpu().numpy()
        assert np.max(np.abs(got - want)) / np.max(np.abs(want)) <= 3e-2
        token, p2, _ = dec.state()
        assert p2 == count + i + 1
    dec.backend.device_status()
    with pytest.raises(api.Unsupported):
        dec.prefill(prompt, 9)           # does not fit max_seq
    with pytest.raises(api.InvalidArgument):
        dec.prefill([cfg.vocab], 0)      # token out of range
    dec.release()


def test_generate_graph_replay_equals_stepwise():
    cfg, dec, model, keep = _build(api.BF16, seed=23)
    a = dec.generate(5, 0, 12, use_graph=False)
    b = dec.generate(5, 0, 12, use_graph=True)
    assert a == b and len(a) == 12
    assert all(0 <= t < cfg.vocab for t in a)
    dec.release()


def test_exchange_path_on_one_rank_matches_plain_decoder():
    """world = 1 with a communicator: the o / down products run the fused product + exchange kernel."""
    from nn_b200 import comm
    b = api.gpu_backend()
    c = comm.PeerComm(b, 0, 1, max_bytes=512 * 8)
    cfg, dec, model, keep = _build(api.BF16, seed=31)
    cfg2, dec2, model2, keep2 = _build(api.BF16, seed=31, comm=c)
    a = dec.generate(7, 0, 8, use_graph=False)
    la = dec.buffers()[2].clone()
    b2 = dec2.generate(7, 0, 8, use_graph=True)
    lb = dec2.buffers()[2].clone()
    assert a == b2
    assert float((la - lb).abs().max()) <= 1e-4 * float(la.abs().max())
    dec.release()
    dec2.release()
    c.release()


def _tp_worker(rank, world, port, out):
    import os

    import torch.distributed as dist

    from nn_b200 import comm
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b = api.Backend(rank)
        c = comm.PeerComm(b, rank, world, max_bytes=512 * 8 + 256)
        cfg1, dec1, model1, keep1 = _build(api.BF16, seed=41, backend=b)      # the single-GPU decoder, on every rank
        want = dec1.generate(9, 0, 8, use_graph=False)
        l1 = dec1.buffers()[2].cpu().numpy()
        ok = True
        for vocab_parallel in (False, True):
            cfg, dec, model, keep = _build(api.BF16, seed=41, backend=b, tp=(rank, world), comm=c, vocab_parallel=vocab_parallel)
            toks = dec.generate(9, 0, 8, use_graph=True)
            logits = dec.buffers()[2].cpu().numpy()
            rows = slice(rank * cfg.vocab // world, (rank + 1) * cfg.vocab // world) if vocab_parallel else slice(0, cfg.vocab)
            ok = ok and toks == want
            ok = ok and float(np.max(np.abs(logits[rows] - l1[rows]))) <= 2e-3 * float(np.max(np.abs(l1)))
            gathered = [None] * world
            dist.all_gather_object(gathered, toks)
            ok = ok and all(g == gathered[0] for g in gathered)     # every rank produced the same tokens
            b.device_status()
            dec.release()
        dec1.release()
        oks = [None] * world
        dist.all_gather_object(oks, bool(ok))                       # every rank's verdict counts
        if rank == 0:
            np.save(out, np.array([1 if all(oks) else 0]))
        dist.barrier()
        c.release()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_decoder_matches_single_gpu(tmp_path):
    import socket

    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "ok.npy")
    mp.spawn(_tp_worker, args=(2, port, out), nprocs=2, join=True)
    assert int(np.load(out)[0]) == 1


def test_decoder_argument_errors():
    b = api.gpu_backend()
    with pytest.raises(api.Unsupported):
        decoder.Decoder(b, decoder.DecoderConfig(hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, n_layers=1,
                                                 vocab=256, max_seq=8))
    dec = decoder.Decoder(b, decoder.DecoderConfig(hidden=256, n_heads=2, n_kv_heads=1, head_dim=128, ffn=256, n_layers=1,
                                                   vocab=256, max_seq=8))
    with pytest.raises(api.TensorError):
        dec.step()          # nothing set yet
    with pytest.raises(api.TensorError):
        dec.reset(999, 0)   # token out of range
    dec.release()
