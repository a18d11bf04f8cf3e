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


def _build(act_dtype, seed=11, backend=None, tp=(0, 1), comm=None):
    """Decoder + dequantized model; with tp = (rank, world) the decoder holds that rank's shards."""
    rank, world = tp
    cfg = decoder.DecoderConfig(hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, n_layers=2, vocab=1024,
                                max_seq=48, rms_eps=1e-6, rope_theta=1e6, act_dtype=act_dtype, tp_rank=rank, tp_world=world)
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
    model["lm_head"] = head_f
    dec.set_head(embed_bf16, model["final_norm"], head)
    return cfg, dec, model, (keep, head, embed_bf16)


@pytest.mark.parametrize("act_dtype,tol", [(api.F32, 2e-3), (api.BF16, 3e-2)])
def test_decode_steps_match_reference_restatement(act_dtype, tol):
    cfg, dec, model, keep = _build(act_dtype)
    kc = np.zeros((cfg.n_layers, cfg.n_kv_heads, cfg.max_seq, cfg.head_dim), np.float32)
    vc = np.zeros_like(kc)
    dec.reset(3, 0)
    token = 3
    _, _, logits_dev, tokens_dev = dec.buffers()
    agree = 0
    for pos in range(10):
        dec.step()
        nxt, npos, steps = dec.state()
        assert (npos, steps) == (pos + 1, pos + 1)
        got = logits_dev.cpu().numpy()
        want, want_tok = ref.step(model, token, pos, kc, vc)   # teacher-forced with the device's tokens
        assert np.all(np.isfinite(got))
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err <= tol, (pos, err)
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
    assert np.max(np.abs(k_dev[:, :, :10].cpu().numpy() - kc[:, :, :10])) <= (5e-3 if act_dtype == api.F32 else 1e-1)
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
        c = comm.PeerComm(b, rank, world, max_bytes=512 * 8)
        cfg, dec, model, keep = _build(api.BF16, seed=41, backend=b, tp=(rank, world), comm=c)
        toks = dec.generate(9, 0, 8, use_graph=True)
        logits = dec.buffers()[2].cpu().numpy()
        ok = True
        if rank == 0:
            cfg1, dec1, model1, keep1 = _build(api.BF16, seed=41, backend=b)
            want = dec1.generate(9, 0, 8, use_graph=False)
            l1 = dec1.buffers()[2].cpu().numpy()
            ok = toks == want and float(np.max(np.abs(logits - l1))) <= 2e-3 * float(np.max(np.abs(l1)))
            dec1.release()
        gathered = [None] * world
        dist.all_gather_object(gathered, toks)
        ok = ok and all(g == gathered[0] for g in gathered)     # every rank produced the same tokens
        b.device_status()
        if rank == 0:
            np.save(out, np.array([1 if ok else 0]))
        dist.barrier()
        dec.release()
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
