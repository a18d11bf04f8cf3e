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


def _build(act_dtype, seed=11):
    cfg = decoder.DecoderConfig(hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, n_layers=2, vocab=1024,
                                max_seq=48, rms_eps=1e-6, rope_theta=1e6, act_dtype=act_dtype)
    s = F.Stream(seed)
    qdim, kvdim = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim

    def qw(fmt, n, k, sd):
        raw, sc = F.gen_weight(fmt, sd, n, k)
        return api.from_quantized(raw, fmt, [n, k], sc), orc.dequantize(fmt, raw, n * k, sc).reshape(n, k)

    def norm(n):
        return (1.0 + 0.1 * s.normal(n)).astype(np.float32)

    b = api.gpu_backend()
    dec = decoder.Decoder(b, cfg)
    model = {"cfg": dict(n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, rms_eps=cfg.rms_eps),
             "rope": ref.rope_tables(cfg.head_dim, cfg.max_seq, cfg.rope_theta), "layers": []}
    keep = []
    for li in range(cfg.n_layers):
        shapes = [("q", qdim, cfg.hidden), ("k", kvdim, cfg.hidden), ("v", kvdim, cfg.hidden), ("o", cfg.hidden, qdim),
                  ("gate", cfg.ffn, cfg.hidden), ("up", cfg.ffn, cfg.hidden), ("down", cfg.hidden, cfg.ffn)]
        L, ws = {}, []
        for i, (name, n, k) in enumerate(shapes):
            w, wf = qw(Q.Q4_K, n, k, seed + 10 * li + i)
            # scale the synthetic weights to keep the residual stream of order one
            ws.append(w)
            L[name] = wf
        for name, n in (("in_norm", cfg.hidden), ("post_norm", cfg.hidden), ("q_norm", cfg.head_dim), ("k_norm", cfg.head_dim)):
            L[name] = norm(n)
        dec.set_layer(li, *ws, L["in_norm"], L["post_norm"], L["q_norm"], L["k_norm"])
        model["layers"].append(L)
        keep.append(ws)
    embed = (s.normal(cfg.vocab * cfg.hidden) * 0.5).astype(np.float32).reshape(cfg.vocab, cfg.hidden)
    embed_bf16 = torch.from_numpy(embed).to(DEV).to(torch.bfloat16)
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
