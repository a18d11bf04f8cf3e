"""Host-side mirror of the decode loop of the reference's Qwen3 model around the library's
quantized products: Qwen3DecoderLayer / Qwen3Attention / Qwen3MLP forward
(crates/nn-qwen3/src/layers.rs:40-47,94-167,205-226) and the greedy generation loop
(crates/nn-core/src/layers/generation/autoregressive.rs:229-247), for one sequence.

``Decoder`` binds nnq_decoder_* of the C ABI. Weights stay owned by the caller
(``api.DeviceWeight`` / ``api.QuantizedTensor``); token and position live on the device, so
``step`` can be captured in a CUDA graph once and replayed per token (``generate`` does that).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from . import api


class _Config(ctypes.Structure):
    _fields_ = [("hidden", ctypes.c_int32), ("n_heads", ctypes.c_int32), ("n_kv_heads", ctypes.c_int32),
                ("head_dim", ctypes.c_int32), ("ffn", ctypes.c_int32), ("n_layers", ctypes.c_int32),
                ("vocab", ctypes.c_int32), ("max_seq", ctypes.c_int32), ("rms_eps", ctypes.c_float),
                ("rope_theta", ctypes.c_double), ("act_dtype", ctypes.c_int32), ("tp_rank", ctypes.c_int32),
                ("tp_world", ctypes.c_int32)]


@dataclass
class DecoderConfig:
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 12288
    n_layers: int = 36
    vocab: int = 151936
    max_seq: int = 2560
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    act_dtype: int = api.BF16
    tp_rank: int = 0
    tp_world: int = 1


class _DevArray:
    """Device memory of the library seen as an array (torch.as_tensor makes a view of it)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


class Decoder:
    def __init__(self, backend: api.Backend, cfg: DecoderConfig):
        self.backend, self.cfg = backend, cfg
        c = _Config(cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.n_layers, cfg.vocab,
                    cfg.max_seq, cfg.rms_eps, cfg.rope_theta, cfg.act_dtype, cfg.tp_rank, cfg.tp_world)
        h = ctypes.c_void_p()
        backend.check(backend._lib.nnq_decoder_create(backend._ctx, ctypes.byref(c), ctypes.byref(h)))
        self._handle = h
        self._keep = []   # tensors the library holds pointers to

    def set_layer(self, layer: int, q, k, v, o, gate, up, down, in_norm, post_norm, q_norm, k_norm):
        """Projections: quantized weights; norms: contiguous f32 torch tensors (any device) or numpy arrays."""
        ws = [q, k, v, o, gate, up, down]
        self._keep.extend(ws)
        norms = [self._ptr(t) for t in (in_norm, post_norm, q_norm, k_norm)]
        self.backend.check(self.backend._lib.nnq_decoder_set_layer(self._handle, layer, *[w.handle() for w in ws], *norms))

    def set_head(self, embed_bf16, final_norm, lm_head):
        self._keep.extend([embed_bf16, lm_head])
        self.backend.check(self.backend._lib.nnq_decoder_set_head(self._handle, embed_bf16.data_ptr(), self._ptr(final_norm),
                                                                  lm_head.handle()))

    def set_comm(self, peer):
        """Tensor parallel: the PeerComm whose slots carry the o / down exchanges (max_bytes >= 8 * hidden)."""
        self._keep.append(peer)
        self.backend.check(self.backend._lib.nnq_decoder_set_comm(self._handle, peer._handle))

    @staticmethod
    def _ptr(t):
        if hasattr(t, "data_ptr"):
            return t.data_ptr()
        return t.ctypes.data   # numpy

    def reset(self, token: int, pos: int, stream=None):
        self.backend.check(self.backend._lib.nnq_decoder_reset(self._handle, token, pos, api._stream_ptr(stream)))

    def prefill(self, tokens, start_pos: int = 0, stream=None):
        """Prompt pass over `tokens` (a sequence of ids) at positions start_pos ..: fills the caches,
        leaves the last prompt token's logits and its greedy successor as the next input."""
        import numpy as np
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        self.backend.check(self.backend._lib.nnq_decoder_prefill(self._handle, arr.ctypes.data, int(arr.size), int(start_pos),
                                                                 api._stream_ptr(stream)))

    def step(self, stream=None):
        self.backend.check(self.backend._lib.nnq_decoder_step(self._handle, api._stream_ptr(stream)))

    def step_raw(self, stream_ptr) -> int:
        return self.backend._lib.nnq_decoder_step(self._handle, stream_ptr)

    def state(self, stream=None):
        t, p, n = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        self.backend.check(self.backend._lib.nnq_decoder_state(self._handle, ctypes.byref(t), ctypes.byref(p), ctypes.byref(n),
                                                               api._stream_ptr(stream)))
        return t.value, p.value, n.value

    def buffers(self):
        """(key cache, value cache, logits, tokens) as torch views of the library's device memory."""
        import torch
        k, v, lg, tk = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        self.backend.check(self.backend._lib.nnq_decoder_buffers(self._handle, ctypes.byref(k), ctypes.byref(v), ctypes.byref(lg),
                                                                 ctypes.byref(tk)))
        c = self.cfg
        dev = torch.device("cuda", self.backend.device)
        shape = (c.n_layers, c.n_kv_heads // c.tp_world, c.max_seq, c.head_dim)
        return (torch.as_tensor(_DevArray(k.value, shape, "<f4"), device=dev),
                torch.as_tensor(_DevArray(v.value, shape, "<f4"), device=dev),
                torch.as_tensor(_DevArray(lg.value, (c.vocab,), "<f4"), device=dev),
                torch.as_tensor(_DevArray(tk.value, (c.max_seq,), "<i4"), device=dev))

    def generate(self, first_token: int, pos: int, n_tokens: int, use_graph: bool = True):
        """Greedy decode of n_tokens starting with `first_token` at position `pos`; returns the
        generated token ids (a list) — one captured graph replayed per token."""
        import torch
        dev = torch.device("cuda", self.backend.device)
        stream = torch.cuda.Stream(device=dev)
        self.reset(first_token, pos, stream)
        with torch.cuda.stream(stream):
            if use_graph and n_tokens > 1:
                self.step(stream)   # warm-up outside capture (lazy module loading, attribute set-up)
                stream.synchronize()
                self.reset(first_token, pos, stream)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    self.step(torch.cuda.current_stream())
                for _ in range(n_tokens):
                    g.replay()
            else:
                for _ in range(n_tokens):
                    self.step(stream)
            stream.synchronize()
        self.backend.device_status(stream)
        toks = self.buffers()[3]
        return toks[pos:pos + n_tokens].cpu().tolist()

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_decoder_destroy(self._handle)
            self._handle = None
            self._keep = []
