"""A Qwen3-shaped GGUF file written to disk, opened through nn_b200.gguf and loaded into the device
decoder with its projections kept in their quantized blocks: logits per step against the numpy
restatement of the reference's decoder (oracle/qwen3_ref.py) fed the oracle's dequantized weights."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api
from nn_b200 import formats as F
from nn_b200 import gguf as G
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc
from oracle import qwen3_ref as ref

pytestmark = pytest.mark.gpu

HID, HEADS, KV, HD, FFN, LAYERS, VOCAB, SEQ = 512, 4, 2, 128, 1024, 2, 1024, 32
GG = {v: k for k, v in G.QUANT_OF.items()}


def _write(path, tied, seed=5):
    s = F.Stream(seed)
    md = {"general.architecture": "qwen3", "qwen3.embedding_length": HID, "qwen3.block_count": LAYERS,
          "qwen3.attention.head_count": HEADS, "qwen3.attention.head_count_kv": KV, "qwen3.feed_forward_length": FFN,
          "qwen3.attention.layer_norm_rms_epsilon": 1e-6, "qwen3.rope.freq_base": 1e6, "qwen3.context_length": 4096}
    tensors, model = [], {"cfg": dict(n_heads=HEADS, n_kv_heads=KV, head_dim=HD, rms_eps=float(np.float32(1e-6))),
                          "rope": ref.rope_tables(HD, SEQ, 1e6), "layers": []}

    def qw(name, fmt, n, k, sd):
        raw, _ = F.gen_weight(fmt, sd, n, k)
        tensors.append((name, [n, k], GG[fmt], raw))
        return orc.dequantize(fmt, raw, n * k, None).reshape(n, k)

    def dense(name, kind, n, k, sd):
        v = (F.Stream(sd).normal(n * k) * 0.05).astype(np.float32)
        if kind == "F16":
            stored = v.astype("<f2")
            w = stored.astype(np.float32)
        elif kind == "BF16":
            stored = F.to_bf16_bits(v).astype("<u2")
            w = F.bf16_bits_to_f32(stored)
        else:
            stored, w = v, v
        tensors.append((name, [n, k], kind, stored))
        return np.asarray(w, np.float32).reshape(n, k)

    def norm(name, n):
        v = (1.0 + 0.1 * s.normal(n)).astype(np.float32)
        tensors.append((name, [n], "F32", v))
        return v

    # every GGUF format the library multiplies with appears in some projection
    # (and, in the second layer, the unquantized tensor types a file may carry for a projection)
    fmts = [{"q": Q.Q4_K, "k": Q.Q8_0, "v": Q.Q6_K, "o": Q.Q4_K, "gate": Q.Q4_0, "up": Q.Q4_1, "down": Q.Q4_K},
            {"q": Q.Q5_K, "k": "F16", "v": "BF16", "o": Q.Q3_K, "gate": Q.Q2_K, "up": "F32", "down": Q.Q5_0}]
    gname = {"q": "attn_q", "k": "attn_k", "v": "attn_v", "o": "attn_output", "gate": "ffn_gate", "up": "ffn_up", "down": "ffn_down"}
    for li in range(LAYERS):
        shapes = [("q", HEADS * HD, HID), ("k", KV * HD, HID), ("v", KV * HD, HID), ("o", HID, HEADS * HD),
                  ("gate", FFN, HID), ("up", FFN, HID), ("down", HID, FFN)]
        L = {}
        for i, (nm, n, k) in enumerate(shapes):
            kind = fmts[li % 2][nm]
            make = dense if isinstance(kind, str) else qw
            L[nm] = make(f"blk.{li}.{gname[nm]}.weight", kind, n, k, seed + 10 * li + i)
        L["in_norm"] = norm(f"blk.{li}.attn_norm.weight", HID)
        L["post_norm"] = norm(f"blk.{li}.ffn_norm.weight", HID)
        L["q_norm"] = norm(f"blk.{li}.attn_q_norm.weight", HD)
        L["k_norm"] = norm(f"blk.{li}.attn_k_norm.weight", HD)
        model["layers"].append(L)
    model["final_norm"] = norm("output_norm.weight", HID)
    if tied:
        emb = qw("token_embd.weight", Q.Q6_K, VOCAB, HID, seed + 77)
        model["lm_head"] = emb
    else:
        emb16 = (s.normal(VOCAB * HID) * 0.5).astype(np.float32).astype("<f2")
        tensors.append(("token_embd.weight", [VOCAB, HID], "F16", emb16))
        emb = emb16.astype(np.float32).reshape(VOCAB, HID)
        model["lm_head"] = qw("output.weight", Q.Q6_K, VOCAB, HID, seed + 99)
    model["embed"] = torch.from_numpy(emb).to(torch.bfloat16).float().numpy()   # the decoder's table is bf16
    tensors.append(("tokenizer.unused", [4], "I32", np.arange(4, dtype="<i4")))
    G.write_gguf(path, md, tensors)
    return model


@pytest.mark.parametrize("tied", [False, True])
def test_decoder_loaded_from_gguf_matches_reference_restatement(tmp_path, tied):
    path = tmp_path / "tiny.gguf"
    model = _write(path, tied)
    f = G.GgufFile.open(path)
    dec, cfg = G.load_qwen3_decoder(f, max_seq=SEQ, act_dtype=api.F32)
    assert (cfg.vocab_size, cfg.head_dim, cfg.num_key_value_heads) == (VOCAB, HD, KV)
    kc = np.zeros((LAYERS, KV, SEQ, HD), np.float32)
    vc = np.zeros_like(kc)
    dec.reset(3, 0)
    token = 3
    logits_dev = dec.buffers()[2]
    for pos in range(6):
        dec.step()
        nxt, npos, _ = dec.state()
        got = logits_dev.cpu().numpy()
        want, _ = ref.step(model, token, pos, kc, vc)
        assert np.all(np.isfinite(got)) and npos == pos + 1
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err <= 2e-3, (pos, err)
        token = nxt
    dec.backend.device_status()
    toks = dec.generate(3, 0, 8)
    assert len(toks) == 8 and all(0 <= t < VOCAB for t in toks)
    dec.release()
    f.close()


def test_missing_tensor_is_reported(tmp_path):
    path = tmp_path / "broken.gguf"
    _write(path, False)
    f = G.GgufFile.open(path)
    del f.tensors["blk.1.ffn_down.weight"]
    with pytest.raises(G.TensorNotFound):
        G.load_qwen3_decoder(f, max_seq=SEQ)
    f.close()
