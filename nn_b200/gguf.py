"""GGUF v3 container: reader with the reference's hardening limits, a writer for shards and test
files, the Qwen3 name map / configuration, and loaders that hand the raw quantized blocks to the
library without a detour through f32.

Mirrors, in the reference tree (crates/nn-gguf/src):
  header.rs:12-34,38-75      magic constant 0x46475547 (the reference's value), version 3, count limits, little-endian scalars
  header.rs:107-120          strings: u64 length (<= 16 MiB) + UTF-8 bytes
  metadata.rs:113-201        typed values 0..12, arrays (<= 10 M elements)
  tensor_info.rs:36-120      name, n_dims (<= 8), dims (non-zero), dtype id, offset; checked sizes
  dequant.rs:49-114          dtype ids, block sizes, bytes per block
  reader.rs:68-141           tensor data starts at the next multiple of 32 after the tensor infos;
                             every tensor must lie inside the file
  arch_qwen3.rs:62-135       configuration from qwen2.* / qwen3.* metadata keys
  arch_qwen3.rs:147-184      GGUF tensor name -> model weight name
Shapes are taken as stored (dimension 0 = rows), as the reference's reader does.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .formats import QuantFormat

GGUF_MAGIC = 0x46475547           # header.rs:12; files written by other tools carry 0x46554747
GGUF_MAGIC_STANDARD = 0x46554747  # accepted only when the caller asks for it
MAX_STRING_LENGTH = 16 * 1024 * 1024
MAX_TENSOR_BYTE_SIZE = 8 * 1024 * 1024 * 1024
MAX_TENSOR_COUNT = 100_000
MAX_METADATA_KV_COUNT = 100_000
MAX_ARRAY_LENGTH = 10_000_000
MAX_DIMENSIONS = 8
ALIGNMENT = 32


class GgufError(Exception):
    """Base of the reader's errors; `kind` names the reference's GgufError variant."""
    kind = "Io"

    def __init__(self, message: str = ""):
        super().__init__(f"{self.kind}: {message}" if message else self.kind)


def _err(kind: str):
    return type(kind, (GgufError,), {"kind": kind})


InvalidMagic = _err("InvalidMagic")
UnsupportedVersion = _err("UnsupportedVersion")
TensorCountExceeded = _err("TensorCountExceeded")
MetadataCountExceeded = _err("MetadataCountExceeded")
StringLengthExceeded = _err("StringLengthExceeded")
InvalidUtf8 = _err("InvalidUtf8")
ArrayLengthExceeded = _err("ArrayLengthExceeded")
UnknownMetadataType = _err("UnknownMetadataType")
DimensionCountExceeded = _err("DimensionCountExceeded")
ZeroDimension = _err("ZeroDimension")
ElementCountOverflow = _err("ElementCountOverflow")
ByteSizeOverflow = _err("ByteSizeOverflow")
TensorTooLarge = _err("TensorTooLarge")
DataOffsetOverflow = _err("DataOffsetOverflow")
DataOutOfBounds = _err("DataOutOfBounds")
MissingMetadata = _err("MissingMetadata")
ArchitectureMismatch = _err("ArchitectureMismatch")
UnexpectedEof = _err("UnexpectedEof")
TensorNotFound = _err("TensorNotFound")

# dtype id -> (name, weights per block, bytes per block); 0 bytes = recognised but not decodable
DTYPES: Dict[int, Tuple[str, int, int]] = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 40), 10: ("Q2K", 256, 84), 11: ("Q3K", 256, 110),
    12: ("Q4K", 256, 144), 13: ("Q5K", 256, 176), 14: ("Q6K", 256, 210), 16: ("IQ2XXS", 1, 0), 17: ("IQ2XS", 1, 0),
    18: ("IQ3XXS", 1, 0), 19: ("IQ1S", 1, 0), 20: ("IQ4NL", 1, 0), 21: ("IQ3S", 1, 0), 22: ("IQ2S", 1, 0),
    23: ("IQ4XS", 1, 0), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
    29: ("IQ1M", 1, 0), 30: ("BF16", 1, 2),
}
DTYPE_ID = {v[0]: k for k, v in DTYPES.items()}
# GGUF dtypes the library multiplies with directly (the reference's nn-gguf element orders)
QUANT_OF = {"Q4_0": QuantFormat.Q4_0, "Q4_1": QuantFormat.Q4_1, "Q8_0": QuantFormat.Q8_0, "Q4K": QuantFormat.Q4_K,
            "Q6K": QuantFormat.Q6_K, "Q5_0": QuantFormat.Q5_0, "Q5_1": QuantFormat.Q5_1, "Q2K": QuantFormat.Q2_K,
            "Q3K": QuantFormat.Q3_K, "Q5K": QuantFormat.Q5_K}
U64_MAX = (1 << 64) - 1


class _Cursor:
    def __init__(self, buf, pos: int = 0):
        self.buf, self.pos = buf, pos

    def take(self, n: int) -> bytes:
        if self.pos + n > len(self.buf):
            raise UnexpectedEof(f"need {n} bytes at offset {self.pos}, file has {len(self.buf)}")
        b = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return b

    def scalar(self, fmt: str):
        return struct.unpack("<" + fmt, self.take(struct.calcsize("<" + fmt)))[0]

    def string(self) -> str:
        n = self.scalar("Q")
        if n > MAX_STRING_LENGTH:
            raise StringLengthExceeded(f"{n} > {MAX_STRING_LENGTH}")
        try:
            return self.take(n).decode("utf-8")
        except UnicodeDecodeError:
            raise InvalidUtf8(f"offset {self.pos}") from None


_SCALAR_FMT = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 10: "Q", 11: "q", 12: "d"}


def _read_value(c: _Cursor, type_id: int):
    if type_id in _SCALAR_FMT:
        return c.scalar(_SCALAR_FMT[type_id])
    if type_id == 7:
        return c.scalar("B") != 0
    if type_id == 8:
        return c.string()
    if type_id == 9:
        elem = c.scalar("I")
        count = c.scalar("Q")
        if count > MAX_ARRAY_LENGTH:
            raise ArrayLengthExceeded(f"{count} > {MAX_ARRAY_LENGTH}")
        return [_read_value(c, elem) for _ in range(count)]
    raise UnknownMetadataType(f"type id {type_id}")


@dataclass
class GgufTensorInfo:
    """One tensor-info record (tensor_info.rs:21-34): `offset` is relative to the data section."""
    name: str
    shape: Tuple[int, ...]
    dtype_id: int
    offset: int

    @property
    def dtype(self) -> str:
        return DTYPES[self.dtype_id][0]

    def checked_num_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
            if n > U64_MAX:
                raise ElementCountOverflow(self.name)
        return max(n, 1)

    def checked_byte_size(self) -> int:
        """(elements / block) * bytes per block, with the reference's overflow and 8 GiB checks
        (tensor_info.rs:106-137)."""
        n = self.checked_num_elements()
        _, bs, ts = DTYPES[self.dtype_id]
        size = (n // bs) * ts
        if size > U64_MAX:
            raise ByteSizeOverflow(f"{self.name}: elements={n} type_size={ts} block_size={bs}")
        if size > MAX_TENSOR_BYTE_SIZE:
            raise TensorTooLarge(f"{self.name}: {size} > {MAX_TENSOR_BYTE_SIZE}")
        return size


def _read_tensor_info(c: _Cursor) -> GgufTensorInfo:
    name = c.string()
    n_dims = c.scalar("I")
    if n_dims > MAX_DIMENSIONS:
        raise DimensionCountExceeded(f"{n_dims} > {MAX_DIMENSIONS}")
    shape = []
    for i in range(n_dims):
        d = c.scalar("Q")
        if d == 0:
            raise ZeroDimension(f"{name}: dimension {i}")
        shape.append(d)
    type_id = c.scalar("I")
    if type_id not in DTYPES:
        raise UnknownMetadataType(f"type id {type_id}")   # the reference reuses this variant for dtypes
    return GgufTensorInfo(name, tuple(shape), type_id, c.scalar("Q"))


class GgufFile:
    """Parsed GGUF v3 file over a byte buffer (an mmap when opened from a path).

    `metadata` maps key -> Python value, `metadata_types` key -> GGUF value type id,
    `tensors` name -> GgufTensorInfo, `data_offset` the start of the tensor data section.
    """

    def __init__(self, buf, *, accept_standard_magic: bool = False, _keep=None):
        self._buf, self._keep = buf, _keep
        c = _Cursor(buf)
        magic = c.scalar("I")
        if magic != GGUF_MAGIC and not (accept_standard_magic and magic == GGUF_MAGIC_STANDARD):
            raise InvalidMagic(f"expected {GGUF_MAGIC:#010x}, got {magic:#010x}")
        self.version = c.scalar("I")
        if self.version != 3:
            raise UnsupportedVersion(f"{self.version} (only v3 supported)")
        tensor_count, kv_count = c.scalar("Q"), c.scalar("Q")
        if tensor_count > MAX_TENSOR_COUNT:
            raise TensorCountExceeded(f"{tensor_count} > {MAX_TENSOR_COUNT}")
        if kv_count > MAX_METADATA_KV_COUNT:
            raise MetadataCountExceeded(f"{kv_count} > {MAX_METADATA_KV_COUNT}")
        self.metadata: Dict[str, object] = {}
        self.metadata_types: Dict[str, int] = {}
        for _ in range(kv_count):
            key = c.string()
            t = c.scalar("I")
            self.metadata[key] = _read_value(c, t)
            self.metadata_types[key] = t
        self.tensors: Dict[str, GgufTensorInfo] = {}
        for _ in range(tensor_count):
            info = _read_tensor_info(c)
            self.tensors[info.name] = info
        self.data_offset = -(-c.pos // ALIGNMENT) * ALIGNMENT
        file_len = len(buf)
        for name, info in self.tensors.items():
            size = info.checked_byte_size()
            start = self.data_offset + info.offset
            if start > U64_MAX or start + size > U64_MAX:
                raise DataOffsetOverflow(f"{name}: data_offset={self.data_offset} tensor_offset={info.offset}")
            if start + size > file_len:
                raise DataOutOfBounds(f"{name}: [{start}..{start + size}) beyond {file_len} bytes")

    @classmethod
    def open(cls, path, **kw) -> "GgufFile":
        """Map the file read-only; tensor bytes are views of the mapping (reader.rs:68-141)."""
        f = open(path, "rb")
        try:
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError:   # empty file
            f.close()
            raise UnexpectedEof("empty file") from None
        return cls(mm, _keep=f, **kw)

    @classmethod
    def from_bytes(cls, data: bytes, **kw) -> "GgufFile":
        return cls(data, **kw)

    # -- metadata ------------------------------------------------------------
    def architecture(self) -> Optional[str]:
        v = self.metadata.get("general.architecture")
        return v if isinstance(v, str) else None

    def model_name(self) -> Optional[str]:
        v = self.metadata.get("general.name")
        return v if isinstance(v, str) else None

    def tensor_names(self) -> List[str]:
        return list(self.tensors)

    def get_u32(self, key: str) -> Optional[int]:
        """Value of a key stored as u32, None when missing or of another type (metadata.rs:111-113)."""
        return self.metadata[key] if self.metadata_types.get(key) == 4 else None

    def get_f32(self, key: str) -> Optional[float]:
        return self.metadata[key] if self.metadata_types.get(key) == 6 else None

    # -- tensor data ---------------------------------------------------------
    def tensor_data(self, name: str) -> np.ndarray:
        """Raw bytes of a tensor as a read-only uint8 view of the file (reader.rs:297-340)."""
        info = self.tensors.get(name)
        if info is None:
            raise TensorNotFound(name)
        start = self.data_offset + info.offset
        return np.frombuffer(self._buf, dtype=np.uint8, count=info.checked_byte_size(), offset=start)

    def tensor_f32(self, name: str) -> np.ndarray:
        """Unquantized tensor (F32 / F16 / BF16 / F64 / integer types) as f32 of the stored shape."""
        info = self.tensors.get(name)
        if info is None:
            raise TensorNotFound(name)
        raw = self.tensor_data(name)
        t = info.dtype
        if t == "BF16":
            out = (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
        elif t in _NP_OF:
            out = raw.view(_NP_OF[t]).astype(np.float32)
        else:
            raise GgufError(f"{name}: {t} is block-quantized; use quantized()")
        return out.reshape(info.shape)

    def quantized(self, name: str, backend=None):
        """The tensor's raw blocks as an api.QuantizedTensor (no dequantization). Formats the
        library has no product for raise api.Unsupported, as DynTensor::from_quantized's
        callers do for an unknown QuantType."""
        from . import api
        info = self.tensors.get(name)
        if info is None:
            raise TensorNotFound(name)
        fmt = QUANT_OF.get(info.dtype)
        if fmt is None and info.dtype in ("F32", "BF16", "F16"):
            # unquantized tensors go through the same entry points as dense weights (the reference's
            # read_tensor_f32 passthrough, reader.rs:253-284): f32 and bf16 as stored, f16 widened
            # exactly to f32
            from .formats import QuantFormat
            raw = self.tensor_data(name)
            if info.dtype == "F16":
                raw = raw.view("<f2").astype(np.float32).view(np.uint8)
            dense = QuantFormat.BF16_DENSE if info.dtype == "BF16" else QuantFormat.F32_DENSE
            return api.QuantizedTensor(raw, dense, info.shape, None, backend)
        if fmt is None:
            raise api.Unsupported(f"{name}: no quantized product for GGUF dtype {info.dtype}")
        return api.QuantizedTensor(self.tensor_data(name), fmt, info.shape, None, backend)

    def close(self):
        if isinstance(self._buf, mmap.mmap):
            try:
                self._buf.close()
            except BufferError:   # numpy views of the mapping are still alive
                pass
        if self._keep is not None:
            self._keep.close()
            self._keep = None


_NP_OF = {"F32": "<f4", "F16": "<f2", "F64": "<f8", "I8": "i1", "I16": "<i2", "I32": "<i4", "I64": "<i8"}


# --------------------------------------------------------------------------- #
# writer
# --------------------------------------------------------------------------- #
def _pack_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(type_id: int, v) -> bytes:
    if type_id in _SCALAR_FMT:
        return struct.pack("<" + _SCALAR_FMT[type_id], v)
    if type_id == 7:
        return struct.pack("<B", 1 if v else 0)
    if type_id == 8:
        return _pack_string(v)
    if type_id == 9:
        elem, items = v
        return struct.pack("<IQ", elem, len(items)) + b"".join(_pack_value(elem, x) for x in items)
    raise UnknownMetadataType(f"type id {type_id}")


@dataclass
class Typed:
    """Metadata value with an explicit GGUF type id; arrays carry `(element type id, items)`."""
    type_id: int
    value: object


def _infer_type(v) -> Tuple[int, object]:
    if isinstance(v, bool):
        return 7, v
    if isinstance(v, int):
        return (4, v) if 0 <= v < (1 << 32) else ((10, v) if v >= 0 else (11, v))
    if isinstance(v, float):
        return 6, v
    if isinstance(v, str):
        return 8, v
    if isinstance(v, (list, tuple)):
        if not v:
            return 9, (4, [])
        elem = _infer_type(v[0])[0]
        return 9, (elem, list(v))
    raise TypeError(f"no GGUF metadata type for {type(v).__name__}")


def write_gguf(path_or_none, metadata: Dict[str, object], tensors: Sequence[Tuple[str, Sequence[int], str, object]],
               *, magic: int = GGUF_MAGIC, version: int = 3) -> bytes:
    """Serialise a GGUF v3 file; returns the bytes and writes them to `path_or_none` when given.

    `metadata` values are Python scalars / strings / lists (types inferred: int -> u32 when it
    fits, float -> f32) or `Typed(type_id, value)` for an explicit type; `tensors` are
    `(name, shape, dtype name, data)` with `data` the raw bytes in the file's layout (numpy
    array or bytes). Tensor data are laid out in order, each aligned to 32 bytes.
    """
    head = struct.pack("<IIQQ", magic, version, len(tensors), len(metadata))
    body = bytearray()
    for k, v in metadata.items():
        t, val = (v.type_id, v.value) if isinstance(v, Typed) else _infer_type(v)
        body += _pack_string(k) + struct.pack("<I", t) + _pack_value(t, val)
    blobs, off = [], 0
    for name, shape, dtype, data in tensors:
        raw = data.tobytes() if hasattr(data, "tobytes") else bytes(data)
        _, bs, ts = DTYPES[DTYPE_ID[dtype]]
        numel = int(np.prod([int(s) for s in shape], dtype=object)) if len(shape) else 1
        if len(raw) != (numel // bs) * ts:
            raise ValueError(f"{name}: {len(raw)} bytes for shape {tuple(shape)} of {dtype}, expected {(numel // bs) * ts}")
        body += _pack_string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", int(s)) for s in shape)
        body += struct.pack("<IQ", DTYPE_ID[dtype], off)
        blobs.append((off, raw))
        off = -(-(off + len(raw)) // ALIGNMENT) * ALIGNMENT
    out = bytearray(head + body)
    data_offset = -(-len(out) // ALIGNMENT) * ALIGNMENT
    out += b"\0" * (data_offset - len(out))
    for o, raw in blobs:
        out += b"\0" * (data_offset + o - len(out)) + raw
    out = bytes(out)
    if path_or_none is not None:
        with open(path_or_none, "wb") as f:
            f.write(out)
    return out


# --------------------------------------------------------------------------- #
# Qwen3: configuration, tensor names, loader
# --------------------------------------------------------------------------- #
@dataclass
class Qwen3Config:
    """Fields of the reference's Qwen3Config as read from GGUF metadata (arch_qwen3.rs:62-135)."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int


def qwen3_config_from_gguf(f: GgufFile) -> Qwen3Config:
    arch = f.architecture()
    if arch is not None and arch not in ("qwen2", "qwen3"):
        raise ArchitectureMismatch(f'expected "qwen2 or qwen3", got "{arch}"')
    prefix = "qwen2" if f.get_u32("qwen2.embedding_length") is not None else "qwen3"

    def need(key):
        v = f.get_u32(f"{prefix}.{key}")
        if v is None:
            raise MissingMetadata(f"{prefix}.{key}")
        return v

    hidden = need("embedding_length")
    layers = need("block_count")
    heads = need("attention.head_count")
    kv = f.get_u32(f"{prefix}.attention.head_count_kv")
    kv = heads if kv is None else kv
    ffn = need("feed_forward_length")
    eps = f.get_f32(f"{prefix}.attention.layer_norm_rms_epsilon")
    theta = f.get_f32(f"{prefix}.rope.freq_base")
    ctx = f.get_u32(f"{prefix}.context_length")
    vocab = f.get_u32(f"{prefix}.vocab_size")
    if vocab is None:
        emb = f.tensors.get("token_embd.weight")
        if emb is None:
            raise MissingMetadata(f"{prefix}.vocab_size (and no token_embd.weight tensor)")
        vocab = emb.shape[0]
    return Qwen3Config(vocab, hidden, ffn, layers, heads, kv, hidden // heads, 1e-6 if eps is None else eps,
                       1_000_000.0 if theta is None else theta, 32768 if ctx is None else ctx)


_LAYER_SUFFIX = {
    "attn_norm.weight": "input_layernorm.weight", "attn_q.weight": "self_attn.q_proj.weight",
    "attn_k.weight": "self_attn.k_proj.weight", "attn_v.weight": "self_attn.v_proj.weight",
    "attn_output.weight": "self_attn.o_proj.weight", "attn_q_norm.weight": "self_attn.q_norm.weight",
    "attn_k_norm.weight": "self_attn.k_norm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
}
_GLOBAL = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
           "output.weight": "lm_head.weight"}


def gguf_to_hf_name(name: str) -> Optional[str]:
    """GGUF tensor name -> the model's weight name, None for names the model does not use
    (arch_qwen3.rs:147-184)."""
    if name in _GLOBAL:
        return _GLOBAL[name]
    if name.startswith("blk."):
        rest = name[4:]
        dot = rest.find(".")
        if dot < 0:
            return None
        suffix = _LAYER_SUFFIX.get(rest[dot + 1:])
        return None if suffix is None else f"model.layers.{rest[:dot]}.{suffix}"
    return None


def load_qwen3_decoder(f: GgufFile, backend=None, *, max_seq: Optional[int] = None, act_dtype: Optional[int] = None,
                       tp=(0, 1), comm=None):
    """Build a decoder.Decoder from a Qwen3 GGUF file.

    Projection weights stay in their quantized blocks (every block format the reference decodes
    goes to the device as stored and is multiplied there); norms are read as f32; the embedding table
    is decoded once to bf16 on the device. `output.weight` falls back to the embedding tensor
    when the file ties them (arch_qwen3.rs:231-236). With tp = (rank, world) the decoder holds
    that rank's shards of the projections and `comm` carries the exchanges.
    Returns (decoder, config).
    """
    import torch

    from . import api, decoder
    b = backend or api.gpu_backend()
    c = qwen3_config_from_gguf(f)
    rank, world = tp
    cfg = decoder.DecoderConfig(hidden=c.hidden_size, n_heads=c.num_attention_heads, n_kv_heads=c.num_key_value_heads,
                                head_dim=c.head_dim, ffn=c.intermediate_size, n_layers=c.num_hidden_layers,
                                vocab=c.vocab_size, max_seq=max_seq or c.max_position_embeddings, rms_eps=c.rms_norm_eps,
                                rope_theta=c.rope_theta, act_dtype=api.BF16 if act_dtype is None else act_dtype,
                                tp_rank=rank, tp_world=world)
    dec = decoder.Decoder(b, cfg)
    if comm is not None:
        dec.set_comm(comm)
    axis = {"attn_q": 0, "attn_k": 0, "attn_v": 0, "ffn_gate": 0, "ffn_up": 0, "attn_output": 1, "ffn_down": 1}

    def need(name):
        if name not in f.tensors:
            raise TensorNotFound(name)
        return name

    def proj(name, short=None):
        w = f.quantized(need(name), b)
        if world > 1 and short in axis:
            w = w.shard(axis[short], rank, world)
        return w

    def norm(name):
        return np.ascontiguousarray(f.tensor_f32(need(name)).reshape(-1))

    for li in range(c.num_hidden_layers):
        p = f"blk.{li}."
        ws = [proj(p + s + ".weight", s) for s in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")]
        dec.set_layer(li, *ws, norm(p + "attn_norm.weight"), norm(p + "ffn_norm.weight"), norm(p + "attn_q_norm.weight"),
                      norm(p + "attn_k_norm.weight"))
    emb_info = f.tensors[need("token_embd.weight")]
    if emb_info.dtype in QUANT_OF:
        emb_q = f.quantized("token_embd.weight", b)
        embed = emb_q.dequantize().to(torch.bfloat16)
        emb_q.release()
    else:
        embed = torch.from_numpy(f.tensor_f32("token_embd.weight")).to(f"cuda:{b.device}").to(torch.bfloat16)
    head_name = "output.weight" if "output.weight" in f.tensors else "token_embd.weight"
    dec.set_head(embed.contiguous(), norm("output_norm.weight"), proj(head_name))
    return dec, c


# --------------------------------------------------------------------------- #
# gpt-oss: tensor names
# --------------------------------------------------------------------------- #
_GPTOSS_LAYER = dict(_LAYER_SUFFIX)
for _s in ("attn_q_norm.weight", "attn_k_norm.weight", "ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"):
    del _GPTOSS_LAYER[_s]
_GPTOSS_LAYER.update({
    "attn_q.bias": "self_attn.q_proj.bias", "attn_k.bias": "self_attn.k_proj.bias", "attn_v.bias": "self_attn.v_proj.bias",
    "attn_output.bias": "self_attn.o_proj.bias", "attn_sinks": "self_attn.sinks", "ffn_router.weight": "mlp.router.weight",
    "ffn_router.bias": "mlp.router.bias", "ffn_experts_gate_up": "mlp.experts.gate_up_proj",
    "ffn_experts_gate_up_bias": "mlp.experts.gate_up_proj_bias", "ffn_experts_down": "mlp.experts.down_proj",
    "ffn_experts_down_bias": "mlp.experts.down_proj_bias",
})


def gptoss_map_tensor_name(name: str) -> Optional[str]:
    """GGUF tensor name -> gpt-oss weight name (crates/nn-gptoss/src/gguf_loader.rs:35-96); the
    layer field must be a non-negative decimal integer."""
    if name in _GLOBAL:
        return _GLOBAL[name]
    layer = gptoss_layer_index(name)
    if layer is None:
        return None
    rest = name[4:]
    dot = rest.find(".")
    suffix = _GPTOSS_LAYER.get(rest[dot + 1:])
    return None if suffix is None else f"model.layers.{rest[:dot]}.{suffix}"


def gptoss_layer_index(name: str) -> Optional[int]:
    """Layer index of `blk.{i}.xxx`, None for other names (gguf_loader.rs:98-106)."""
    if not name.startswith("blk."):
        return None
    rest = name[4:]
    dot = rest.find(".")
    if dot < 0:
        return None
    field = rest[:dot]
    digits = field[1:] if field.startswith("+") else field   # Rust's usize parser accepts a leading '+'
    if not digits or not digits.isascii() or not digits.isdigit():
        return None
    return int(digits)
