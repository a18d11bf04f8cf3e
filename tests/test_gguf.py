"""GGUF v3 reader / writer of nn_b200.gguf against the cases of the reference's own tests
(crates/nn-gguf/src/gguf_security_hardening_tests.rs, reader.rs:488-760, arch_qwen3.rs tests):
limits at and one past their bounds, overflow checks, magic / version, metadata types, the
32-byte data alignment, bounds of tensor data, the Qwen3 name map and configuration keys."""
import struct

import numpy as np
import pytest

from nn_b200 import gguf as G
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q

U64 = (1 << 64) - 1


def header(tensors=0, kvs=0, magic=G.GGUF_MAGIC, version=3):
    return struct.pack("<IIQQ", magic, version, tensors, kvs)


def s(b):
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def info(name, dims, dtype=0, offset=0):
    return s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", dtype, offset)


def test_minimal_file():
    f = G.GgufFile.from_bytes(header())
    assert f.version == 3 and not f.tensors and not f.metadata and f.data_offset == 32
    assert f.architecture() is None and f.tensor_names() == []


def test_magic_is_the_reference_constant():
    assert G.GGUF_MAGIC == 0x46475547
    for bad in (0, 0x67676D6C, G.GGUF_MAGIC ^ 1, int.from_bytes(struct.pack(">I", G.GGUF_MAGIC), "little"), 0xFFFFFFFF,
                G.GGUF_MAGIC_STANDARD):
        with pytest.raises(G.InvalidMagic):
            G.GgufFile.from_bytes(header(magic=bad))
    G.GgufFile.from_bytes(header(magic=G.GGUF_MAGIC_STANDARD), accept_standard_magic=True)


@pytest.mark.parametrize("v", [0, 1, 2, 4, 0xFFFFFFFF])
def test_versions_other_than_3_rejected(v):
    with pytest.raises(G.UnsupportedVersion):
        G.GgufFile.from_bytes(header(version=v))


def test_count_limits():
    # at the limit the header is accepted and parsing then runs out of data
    with pytest.raises(G.UnexpectedEof):
        G.GgufFile.from_bytes(header(tensors=G.MAX_TENSOR_COUNT))
    with pytest.raises(G.UnexpectedEof):
        G.GgufFile.from_bytes(header(kvs=G.MAX_METADATA_KV_COUNT))
    for n in (G.MAX_TENSOR_COUNT + 1, U64, U64 - 1):
        with pytest.raises(G.TensorCountExceeded):
            G.GgufFile.from_bytes(header(tensors=n))
    with pytest.raises(G.MetadataCountExceeded):
        G.GgufFile.from_bytes(header(kvs=G.MAX_METADATA_KV_COUNT + 1))
    with pytest.raises(G.TensorCountExceeded):   # tensor count is checked first
        G.GgufFile.from_bytes(header(tensors=U64, kvs=U64))


def test_string_limits():
    bomb = struct.pack("<Q", G.MAX_STRING_LENGTH + 1)
    with pytest.raises(G.StringLengthExceeded):      # key position
        G.GgufFile.from_bytes(header(kvs=1) + bomb)
    with pytest.raises(G.StringLengthExceeded):      # value position
        G.GgufFile.from_bytes(header(kvs=1) + s("k") + struct.pack("<I", 8) + bomb)
    with pytest.raises(G.StringLengthExceeded):      # tensor name
        G.GgufFile.from_bytes(header(tensors=1) + bomb)
    with pytest.raises(G.StringLengthExceeded):      # inside an array of strings
        G.GgufFile.from_bytes(header(kvs=1) + s("a") + struct.pack("<IIQ", 9, 8, 1) + bomb)
    with pytest.raises(G.UnexpectedEof):             # at the limit: accepted, then no data
        G.GgufFile.from_bytes(header(kvs=1) + struct.pack("<Q", G.MAX_STRING_LENGTH))
    with pytest.raises(G.InvalidUtf8):
        G.GgufFile.from_bytes(header(kvs=1) + s(b"\xff\xfe") + struct.pack("<II", 4, 1))


def test_array_limits_and_nesting():
    pre = header(kvs=1) + s("a") + struct.pack("<II", 9, 0)
    for n in (G.MAX_ARRAY_LENGTH + 1, U64):
        with pytest.raises(G.ArrayLengthExceeded):
            G.GgufFile.from_bytes(pre + struct.pack("<Q", n))
    with pytest.raises(G.UnexpectedEof):
        G.GgufFile.from_bytes(pre + struct.pack("<Q", G.MAX_ARRAY_LENGTH))
    nested = header(kvs=1) + s("deep") + struct.pack("<IIQ", 9, 9, 1) + struct.pack("<IQ", 9, 1) + struct.pack("<IQ", 0, 0)
    assert G.GgufFile.from_bytes(nested).metadata["deep"] == [[[]]]
    with pytest.raises(G.UnknownMetadataType):
        G.GgufFile.from_bytes(header(kvs=1) + s("k") + struct.pack("<I", 13))


def test_dimension_limits():
    ok = header(tensors=1) + info("t", [1] * G.MAX_DIMENSIONS)
    f = G.GgufFile.from_bytes(ok + b"\0" * 64)
    assert f.tensors["t"].shape == (1,) * 8
    with pytest.raises(G.DimensionCountExceeded):
        G.GgufFile.from_bytes(header(tensors=1) + s("t") + struct.pack("<I", G.MAX_DIMENSIONS + 1))
    for dims in ([0, 4, 4], [4, 0, 4], [4, 4, 0]):
        with pytest.raises(G.ZeroDimension):
            G.GgufFile.from_bytes(header(tensors=1) + info("z", dims))
    with pytest.raises(G.UnknownMetadataType):   # the reference reports an unknown dtype id with this variant
        G.GgufFile.from_bytes(header(tensors=1) + info("t", [4], dtype=15))


def T(dims, dtype):
    return G.GgufTensorInfo("t", tuple(dims), G.DTYPE_ID[dtype], 0)


def test_checked_sizes():
    for dims in ([U64 // 2 + 1, 3], [2_097_152, 2_097_152, 4_194_304]):
        with pytest.raises((G.ElementCountOverflow, G.ByteSizeOverflow)):
            T(dims, "F32").checked_byte_size()
    with pytest.raises((G.ByteSizeOverflow, G.TensorTooLarge)):
        T([U64 // 4 + 1], "F32").checked_byte_size()
    with pytest.raises((G.ElementCountOverflow, G.ByteSizeOverflow, G.TensorTooLarge)):
        T([min(U64, (U64 // 144 + 1) * 256)], "Q4K").checked_byte_size()
    assert T([], "F32").checked_num_elements() == 1 and T([1], "F32").checked_num_elements() == 1
    assert T([32, 64], "F32").checked_byte_size() == 32 * 64 * 4
    assert T([4, 256], "Q4K").checked_byte_size() == 4 * 144
    assert T([2, 256], "Q6K").checked_byte_size() == 2 * 210 and T([64], "Q8_0").checked_byte_size() == 68
    gib8 = G.MAX_TENSOR_BYTE_SIZE
    for dtype, size in (("F32", 4), ("F16", 2), ("I8", 1), ("F64", 8)):
        assert T([gib8 // size], dtype).checked_byte_size() == gib8
        with pytest.raises(G.TensorTooLarge):
            T([gib8 // size + 1], dtype).checked_byte_size()


def test_dtype_table_matches_reference_ids():
    want = {"F32": (0, 1, 4), "F16": (1, 1, 2), "Q4_0": (2, 32, 18), "Q4_1": (3, 32, 20), "Q5_0": (6, 32, 22),
            "Q5_1": (7, 32, 24), "Q8_0": (8, 32, 34), "Q8_1": (9, 32, 40), "Q2K": (10, 256, 84), "Q3K": (11, 256, 110),
            "Q4K": (12, 256, 144), "Q5K": (13, 256, 176), "Q6K": (14, 256, 210), "BF16": (30, 1, 2), "I32": (26, 1, 4)}
    for name, (tid, bs, ts) in want.items():
        assert G.DTYPES[tid] == (name, bs, ts)
    assert 4 not in G.DTYPES and 5 not in G.DTYPES and 15 not in G.DTYPES


def test_data_offset_is_32_byte_aligned_and_bounds_are_checked():
    x = np.arange(6, dtype="<f4")
    for pad in range(0, 9):
        b = G.write_gguf(None, {"k" + "x" * pad: 1}, [("t", [2, 3], "F32", x)])
        f = G.GgufFile.from_bytes(b)
        assert f.data_offset % 32 == 0 and np.array_equal(f.tensor_f32("t"), x.reshape(2, 3))
        with pytest.raises(G.DataOutOfBounds):
            G.GgufFile.from_bytes(b[:-1])
    with pytest.raises(G.DataOutOfBounds):
        G.GgufFile.from_bytes(header(tensors=1) + info("t", [4], 0, offset=1 << 40))
    with pytest.raises((G.DataOffsetOverflow, G.DataOutOfBounds)):
        G.GgufFile.from_bytes(header(tensors=1) + info("t", [4], 0, offset=U64 - 8))
    with pytest.raises(G.TensorNotFound):
        G.GgufFile.from_bytes(header()).tensor_data("nope")


def test_metadata_values_of_every_type_round_trip():
    md = {"u8": G.Typed(0, 200), "i8": G.Typed(1, -5), "u16": G.Typed(2, 60000), "i16": G.Typed(3, -300), "u32": 7,
          "i32": G.Typed(5, -7), "f32": 0.5, "bool": True, "str": "grüße", "u64": 1 << 40, "i64": -(1 << 40),
          "f64": G.Typed(12, 1e300), "arr": [1, 2, 3], "sarr": ["a", "bc"], "empty": G.Typed(9, (8, []))}
    f = G.GgufFile.from_bytes(G.write_gguf(None, md, []))
    want = {k: (v.value if isinstance(v, G.Typed) else v) for k, v in md.items()}
    want["empty"] = []
    assert f.metadata == want
    assert [f.metadata_types[k] for k in md] == [0, 1, 2, 3, 4, 5, 6, 7, 8, 10, 11, 12, 9, 9, 9]
    assert f.get_u32("u32") == 7 and f.get_u32("u64") is None and f.get_u32("missing") is None
    assert f.get_f32("f32") == 0.5 and f.get_f32("f64") is None


def test_open_maps_the_file_and_returns_raw_blocks(tmp_path):
    n, k = 16, 512
    raws = {"Q4K": F.gen_weight(Q.Q4_K, 1, n, k)[0], "Q6K": F.gen_weight(Q.Q6_K, 2, n, k)[0],
            "Q8_0": F.gen_weight(Q.Q8_0, 3, n, k)[0], "Q4_0": F.gen_weight(Q.Q4_0, 4, n, k)[0],
            "Q4_1": F.gen_weight(Q.Q4_1, 5, n, k)[0]}
    half = np.linspace(-2, 2, 24, dtype=np.float32).astype("<f2")
    bf = (np.linspace(-3, 3, 8, dtype=np.float32).view(np.uint32) >> 16).astype("<u2")
    tensors = [(f"w.{t}", [n, k], t, r) for t, r in raws.items()]
    tensors += [("h", [4, 6], "F16", half), ("b", [8], "BF16", bf), ("i", [3], "I32", np.array([1, -2, 3], "<i4"))]
    path = tmp_path / "m.gguf"
    G.write_gguf(path, {"general.architecture": "qwen3", "general.name": "tiny"}, tensors)
    f = G.GgufFile.open(path)
    assert f.architecture() == "qwen3" and f.model_name() == "tiny" and len(f.tensor_names()) == 8
    for t, r in raws.items():
        info = f.tensors[f"w.{t}"]
        assert info.shape == (n, k) and info.dtype == t and (f.data_offset + info.offset) % 32 == 0
        assert np.array_equal(f.tensor_data(f"w.{t}"), np.frombuffer(r, np.uint8))
        q = f.quantized(f"w.{t}")
        assert q.quant_type == G.QUANT_OF[t] and q.dims() == (n, k) and q.is_quantized()
        with pytest.raises(G.GgufError):
            f.tensor_f32(f"w.{t}")
    assert np.array_equal(f.tensor_f32("h"), half.astype(np.float32).reshape(4, 6))
    assert np.array_equal(f.tensor_f32("b").view(np.uint32) >> 16, bf)
    assert f.tensor_f32("i").tolist() == [1.0, -2.0, 3.0]
    f.close()
    with pytest.raises(FileNotFoundError):
        G.GgufFile.open(tmp_path / "missing.gguf")


def test_quantized_refuses_formats_without_a_product():
    from nn_b200 import api
    b = G.write_gguf(None, {}, [("w", [1, 32], "Q8_1", np.zeros(40, np.uint8)), ("x", [4], "I32", np.zeros(4, "<i4")),
                                ("v", [4], "F32", np.zeros(4, "<f4"))])
    f = G.GgufFile.from_bytes(b)
    for name in ("w", "x"):
        with pytest.raises(api.Unsupported):
            f.quantized(name)
    # an unquantized tensor is a dense weight of the same entry points: whole 32-value units only
    with pytest.raises(api.InvalidShape):
        f.quantized("v")


def test_qwen3_name_map():
    m = G.gguf_to_hf_name
    assert m("token_embd.weight") == "model.embed_tokens.weight"
    assert m("output_norm.weight") == "model.norm.weight" and m("output.weight") == "lm_head.weight"
    pairs = {"attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
             "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm",
             "attn_k_norm": "self_attn.k_norm", "ffn_norm": "post_attention_layernorm", "ffn_gate": "mlp.gate_proj",
             "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}
    for g, h in pairs.items():
        assert m(f"blk.17.{g}.weight") == f"model.layers.17.{h}.weight"
    for other in ("tokenizer.ggml.tokens", "blk.0.attn_q.bias", "blk.3", "blk..weight", "rope_freqs.weight"):
        assert m(other) is None


def _qwen3_md(prefix="qwen3", **over):
    md = {"general.architecture": prefix, f"{prefix}.embedding_length": 512, f"{prefix}.block_count": 2,
          f"{prefix}.attention.head_count": 4, f"{prefix}.attention.head_count_kv": 2, f"{prefix}.feed_forward_length": 1024,
          f"{prefix}.attention.layer_norm_rms_epsilon": 1e-5, f"{prefix}.rope.freq_base": 10000.0,
          f"{prefix}.context_length": 4096, f"{prefix}.vocab_size": 1000}
    md.update(over)
    return {k: v for k, v in md.items() if v is not None}


def test_qwen3_config_keys_defaults_and_errors():
    c = G.qwen3_config_from_gguf(G.GgufFile.from_bytes(G.write_gguf(None, _qwen3_md(), [])))
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (1000, 512, 1024, 2)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.max_position_embeddings) == (4, 2, 128, 4096)
    assert c.rms_norm_eps == np.float32(1e-5) and c.rope_theta == 10000.0
    # qwen2.* keys win when present; defaults for the optional keys; vocabulary from the embedding shape
    md = _qwen3_md("qwen2", **{"qwen2.attention.head_count_kv": None, "qwen2.attention.layer_norm_rms_epsilon": None,
                               "qwen2.rope.freq_base": None, "qwen2.context_length": None, "qwen2.vocab_size": None})
    emb = ("token_embd.weight", [300, 512], "F16", np.zeros(300 * 512, "<f2"))
    c = G.qwen3_config_from_gguf(G.GgufFile.from_bytes(G.write_gguf(None, md, [emb])))
    assert (c.vocab_size, c.num_key_value_heads, c.rms_norm_eps, c.rope_theta, c.max_position_embeddings) == (300, 4, 1e-6, 1e6, 32768)
    with pytest.raises(G.MissingMetadata):
        G.qwen3_config_from_gguf(G.GgufFile.from_bytes(G.write_gguf(None, md, [])))
    with pytest.raises(G.ArchitectureMismatch):
        G.qwen3_config_from_gguf(G.GgufFile.from_bytes(G.write_gguf(None, _qwen3_md(**{"general.architecture": "llama"}), [])))
    with pytest.raises(G.MissingMetadata):
        G.qwen3_config_from_gguf(G.GgufFile.from_bytes(G.write_gguf(None, _qwen3_md(**{"qwen3.block_count": None}), [])))
    # a count stored with another integer type does not satisfy the u32 getter
    with pytest.raises(G.MissingMetadata):
        G.qwen3_config_from_gguf(G.GgufFile.from_bytes(G.write_gguf(None, _qwen3_md(**{"qwen3.block_count": G.Typed(10, 2)}), [])))


def test_gptoss_name_map():
    m = G.gptoss_map_tensor_name
    assert m("token_embd.weight") == "model.embed_tokens.weight" and m("output.weight") == "lm_head.weight"
    assert m("blk.3.attn_q.bias") == "model.layers.3.self_attn.q_proj.bias"
    assert m("blk.0.attn_sinks") == "model.layers.0.self_attn.sinks"
    assert m("blk.23.ffn_router.weight") == "model.layers.23.mlp.router.weight"
    assert m("blk.5.ffn_experts_gate_up") == "model.layers.5.mlp.experts.gate_up_proj"
    assert m("blk.5.ffn_experts_gate_up_bias") == "model.layers.5.mlp.experts.gate_up_proj_bias"
    assert m("blk.5.ffn_experts_down") == "model.layers.5.mlp.experts.down_proj"
    assert m("blk.5.ffn_experts_down_bias") == "model.layers.5.mlp.experts.down_proj_bias"
    assert m("blk.7.ffn_norm.weight") == "model.layers.7.post_attention_layernorm.weight"
    for other in ("blk.x.attn_q.weight", "blk.-1.attn_q.weight", "blk.2.ffn_gate.weight", "blk.2", "foo", "blk.2.attn_q_norm.weight"):
        assert m(other) is None
    assert G.gptoss_layer_index("blk.12.attn_sinks") == 12 and G.gptoss_layer_index("output.weight") is None
