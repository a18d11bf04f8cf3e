"""The numpy restatement of the reference's decoder parts (oracle/qwen3_ref.py) against the
known answers the reference's own unit tests assert, read from its sources:
RMSNorm  crates/nn-core/src/layers/rms_norm.rs (test_rms_norm_basic, test_rms_norm_with_weight),
RoPE     crates/nn-core/src/layers/attention/rope_tests.rs (identity at position 0, known values at
         position 1 for one frequency pair, norm preservation),
argmax   crates/nn-core/src/layers/generation/autoregressive_tests.rs and the documented rule of
         autoregressive_sampling.rs:14-21 (Iterator::max_by keeps the last of equal maxima)."""
import numpy as np

from oracle import qwen3_ref as ref


def test_rms_norm_known_answers():
    y = ref.rms_norm(np.array([1, 2, 3, 4], np.float32), np.ones(4, np.float32), 1e-5)
    assert abs(y[0] - 0.3651) < 0.01 and abs(y[3] - 1.4606) < 0.01
    y = ref.rms_norm(np.array([3, 4], np.float32), np.array([2.0, 0.5], np.float32), 1e-5)
    assert abs(y[0] - 1.6971) < 0.01 and abs(y[1] - 0.5657) < 0.01


def test_rope_known_values_identity_and_norm():
    cos, sin = ref.rope_tables(2, 4, 10000.0)      # one frequency pair: inv_freq = 1
    y = ref.rotate(np.array([1.0, 0.0], np.float32), cos[1], sin[1])
    assert abs(y[0] - np.cos(np.float32(1.0))) < 1e-5 and abs(y[1] - np.sin(np.float32(1.0))) < 1e-5
    cos, sin = ref.rope_tables(128, 64, 1e6)
    x = np.random.default_rng(0).standard_normal(128).astype(np.float32)
    assert np.array_equal(ref.rotate(x, cos[0], sin[0]), x)            # position 0 is the identity
    for pos in (1, 7, 63):
        assert abs(np.linalg.norm(ref.rotate(x, cos[pos], sin[pos])) - np.linalg.norm(x)) < 1e-4
    # inv_freq is rounded to f32 before the angle is formed in f64 and rounded to f32
    inv = np.float32(1.0 / 1e6 ** (2 * 5 / 128))
    assert cos[9, 5] == np.cos(np.float32(np.float64(9) * np.float64(inv)))


def test_argmax_rules():
    assert ref.argmax_last([1.0]) == 0
    assert ref.argmax_last([-np.inf, -np.inf]) < 2
    assert ref.argmax_last([1.0, 3.0, 3.0, 2.0]) == 2   # the last of equal maxima


def test_step_shapes_and_cache_update():
    rng = np.random.default_rng(1)
    cfg = dict(n_heads=2, n_kv_heads=1, head_dim=4, rms_eps=1e-6)
    hid, ffn, vocab = 8, 16, 10

    def w(n, k):
        return (rng.standard_normal((n, k)) * 0.3).astype(np.float32)

    layer = dict(q=w(8, hid), k=w(4, hid), v=w(4, hid), o=w(hid, 8), gate=w(ffn, hid), up=w(ffn, hid), down=w(hid, ffn),
                 in_norm=np.ones(hid, np.float32), post_norm=np.ones(hid, np.float32), q_norm=np.ones(4, np.float32),
                 k_norm=np.ones(4, np.float32))
    model = dict(cfg=cfg, rope=ref.rope_tables(4, 8, 1e4), layers=[layer], embed=w(vocab, hid),
                 final_norm=np.ones(hid, np.float32), lm_head=w(vocab, hid))
    kc = np.zeros((1, 1, 8, 4), np.float32)
    vc = np.zeros_like(kc)
    logits0, t0 = ref.step(model, 3, 0, kc, vc)
    assert logits0.shape == (vocab,) and t0 == ref.argmax_last(logits0)
    assert np.any(kc[0, 0, 0] != 0) and np.all(kc[0, 0, 1:] == 0)
    # with a single key the softmax weight is 1: the attention output is the value row itself
    x = ref.rms_norm(model["embed"][3], layer["in_norm"], 1e-6)
    assert np.allclose(vc[0, 0, 0], layer["v"] @ x, atol=1e-6)
    logits1, _ = ref.step(model, t0, 1, kc, vc)
    assert np.all(np.isfinite(logits1)) and np.any(kc[0, 0, 1] != 0)
