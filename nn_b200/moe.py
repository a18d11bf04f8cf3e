"""Host-side mirror of the reference's quantized MoE block (gpt-oss): same roles as
``QuantizedDecoderLayer::moe_forward`` / ``expert_forward``
(crates/nn-gptoss/src/quantized_model.rs:99-194) and ``GptOssMoeBlock::forward``
(crates/nn-gptoss/src/layers.rs:254), computed through the C ABI (nnq_moe_*)."""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import api
from .formats import QuantFormat

LAYOUT_KN_GPTOSS, LAYOUT_NK = 0, 1


def _u8(a):
    return None if a is None else np.ascontiguousarray(a, np.uint8).reshape(-1)


def _f32(a):
    return np.ascontiguousarray(a, np.float32)


class MoeBlock:
    """Router + quantized experts of one decoder layer.

    router_w [E, H], router_b [E]; expert tensors as raw quantized bytes:
      layout KN_GPTOSS: gate_up logical [E, H, 2I], down [E, I, H] (nn-gptoss Mxfp4Tensor, blocks along N)
      layout NK:        gate_up logical [E, 2I, H], down [E, H, I] (any format, blocks along K)
    gate_up_bias [E, 2I], down_bias [E, H].
    """

    def __init__(self, n_experts, hidden, inter, top_k, swiglu_limit, router_w, router_b, layout, fmt,
                 gate_up, gate_up_scales, gate_up_bias, down, down_scales, down_bias, backend=None,
                 expert_range=None):
        self.backend = backend or api.gpu_backend()
        self.n_experts, self.hidden, self.inter, self.top_k = n_experts, hidden, inter, top_k
        b = self.backend
        rw, rb = _f32(router_w), _f32(router_b)
        gu, gus, gub = _u8(gate_up), _u8(gate_up_scales), _f32(gate_up_bias)
        dn, dns, dnb = _u8(down), _u8(down_scales), _f32(down_bias)
        if rw.shape != (n_experts, hidden) or rb.shape != (n_experts,):
            raise api.InvalidShape("router weight must be [E, hidden] and router bias [E]")
        e0, ec = expert_range if expert_range is not None else (0, n_experts)
        if gub.shape != (ec, 2 * inter) or dnb.shape != (ec, hidden):
            raise api.BiasMismatch("expert biases must be [E, 2*inter] and [E, hidden]")
        h = ctypes.c_void_p()
        p = lambda a: None if a is None else a.ctypes.data
        n = lambda a: 0 if a is None else a.size
        # expert_range = (first expert, count): an expert-parallel shard holding only those experts'
        # tensors; the router always covers all experts
        b.check(b._lib.nnq_moe_create_shard(b._ctx, n_experts, e0, ec, hidden, inter, top_k,
                                            ctypes.c_float(swiglu_limit), p(rw), p(rb), int(layout),
                                            int(QuantFormat(fmt)), p(gu), n(gu), p(gus), n(gus), p(gub), p(dn),
                                            n(dn), p(dns), n(dns), p(dnb), ctypes.byref(h)))
        self._handle = h

    def forward(self, x):
        """x [.., hidden] (torch CUDA f32 / bf16) -> f32 [.., hidden]."""
        import torch
        b = self.backend
        if x.shape[-1] != self.hidden:
            raise api.ShapeMismatch(f"input last dim {x.shape[-1]} != hidden {self.hidden}")
        xs = x.contiguous()
        t = math.prod(xs.shape[:-1])
        y = torch.empty(xs.shape, dtype=torch.float32, device=xs.device)
        b.check(b._lib.nnq_moe_forward(b._ctx, self._handle, xs.data_ptr(), api._dtype_code(xs), t, y.data_ptr(),
                                       api._stream_ptr(None)))
        return y

    __call__ = forward

    def route(self, x):
        """(expert indices [T, k] int32, renormalised weights [T, k] f32)."""
        import torch
        b = self.backend
        xs = x.contiguous()
        t = math.prod(xs.shape[:-1])
        idx = torch.empty((t, self.top_k), dtype=torch.int32, device=xs.device)
        wt = torch.empty((t, self.top_k), dtype=torch.float32, device=xs.device)
        b.check(b._lib.nnq_moe_route(b._ctx, self._handle, xs.data_ptr(), api._dtype_code(xs), t, idx.data_ptr(),
                                     wt.data_ptr(), api._stream_ptr(None)))
        return idx, wt

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_moe_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.release()
        except Exception:
            pass
