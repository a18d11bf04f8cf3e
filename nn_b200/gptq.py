"""Host-side mirror of the reference's GPTQ / AWQ loaders
(crates/nn-core/src/layers/quantized/gptq_loader.rs, awq_loader.rs): ``GptqFormat``,
``AwqFormat``, ``unpack_gptq_qweight`` (:69), ``unpack_gptq_qzeros`` (:101), ``dequantize_gptq``
(:139), ``GptqLinear`` (:203-312), ``load_gptq_linear`` (:329), ``unpack_awq_qweight`` and
``load_awq_linear`` (awq_loader.rs:54,74), over nnq_gptq_* / nnq_gq_* of the C ABI.

The reference expands the 4-bit codes to an f32 weight at load and multiplies dense afterwards;
``load_gptq_linear`` here keeps the codes packed on the device (repacked once so that a 32-bit word
holds eight in-features of one output row) and the product decodes them as it streams."""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional

from . import api
from .formats import QuantFormat
from .weight_quant import GroupWeight, _stream


@dataclass
class GptqFormat:
    group_size: int = 128
    bits: int = 4
    act_order: bool = False


@dataclass
class AwqFormat:
    group_size: int = 128
    bits: int = 4


def _u32(torch, t, dev):
    """Packed words arrive as int32 / uint32 torch tensors or numpy uint32 arrays: same bits."""
    if not torch.is_tensor(t):
        import numpy as np
        t = torch.from_numpy(np.ascontiguousarray(t, dtype=np.uint32).view(np.int32))
    if t.dtype not in (torch.int32, getattr(torch, "uint32", torch.int32)):
        raise api.InvalidArgument(f"packed tensor must hold 32-bit words, got {t.dtype}")
    return t.to(dev).contiguous()


def unpack_gptq_qweight(packed, backend: Optional[api.Backend] = None):
    """u32 [in_features / 8, out_features] -> f32 [in_features, out_features], values 0..15."""
    torch = api._torch()
    b = backend or api.gpu_backend()
    dev = torch.device("cuda", b.device)
    if len(packed.shape) != 2:
        raise api.RankMismatch(f"expected a 2-D packed tensor, got rank {len(packed.shape)}")
    p = _u32(torch, packed, dev)
    rows, cols = p.shape
    out = torch.empty((rows * 8, cols), dtype=torch.float32, device=dev)
    b.check(b._lib.nnq_gptq_unpack_qweight(b._ctx, p.data_ptr(), rows, cols, out.data_ptr(), _stream(torch, dev)))
    return out


unpack_awq_qweight = unpack_gptq_qweight   # awq_loader.rs:54-56 delegates


def unpack_gptq_qzeros(packed, backend: Optional[api.Backend] = None):
    """u32 [groups, out_features / 8] -> f32 [groups, out_features], values 0..15."""
    torch = api._torch()
    b = backend or api.gpu_backend()
    dev = torch.device("cuda", b.device)
    if len(packed.shape) != 2:
        raise api.RankMismatch(f"expected a 2-D packed tensor, got rank {len(packed.shape)}")
    p = _u32(torch, packed, dev)
    groups, cols = p.shape
    out = torch.empty((groups, cols * 8), dtype=torch.float32, device=dev)
    b.check(b._lib.nnq_gptq_unpack_qzeros(b._ctx, p.data_ptr(), groups, cols, out.data_ptr(), _stream(torch, dev)))
    return out


def dequantize_gptq(q_weight, scales, zeros, group_size: int, backend: Optional[api.Backend] = None):
    """(q - zeros[group]) * scales[group] over unpacked f32 values [in_features, out_features]."""
    torch = api._torch()
    b = backend or api.gpu_backend()
    dev = torch.device("cuda", b.device)
    k, n = q_weight.shape
    if scales.shape[1] != n:
        raise api.ShapeMismatch(f"expected scales [{scales.shape[0]}, {n}], got {list(scales.shape)}")
    if tuple(zeros.shape) != tuple(scales.shape):
        raise api.ShapeMismatch(f"expected zeros {list(scales.shape)}, got {list(zeros.shape)}")
    q = q_weight.to(device=dev, dtype=torch.float32).contiguous()
    s = scales.to(device=dev, dtype=torch.float32).contiguous()
    z = zeros.to(device=dev, dtype=torch.float32).contiguous()
    out = torch.empty((k, n), dtype=torch.float32, device=dev)
    b.check(b._lib.nnq_gptq_dequantize(b._ctx, q.data_ptr(), s.data_ptr(), z.data_ptr(), k, n, s.shape[0], int(group_size),
                                       out.data_ptr(), _stream(torch, dev)))
    return out


class GptqLinear:
    """``GptqLinear``: ``forward(x) = x @ W^T + bias``. Built either from packed components
    (``load_gptq_linear`` / ``load_awq_linear``: the codes stay packed) or, as the reference's
    ``GptqLinear::new``, from an already dequantized f32 weight [out_features, in_features]."""

    def __init__(self, weight, bias=None, format: Optional[GptqFormat] = None, backend: Optional[api.Backend] = None):
        torch = api._torch()
        self.backend = backend or api.gpu_backend()
        self.format = format or GptqFormat()
        dev = torch.device("cuda", self.backend.device)
        self._pad = 0
        if isinstance(weight, GroupWeight):
            self._packed: Optional[GroupWeight] = weight
            self._dense = None
            self.out_features, self.in_features = weight.out_features, weight.in_features
        else:
            if len(weight.shape) != 2:
                raise api.RankMismatch(f"expected a 2-D weight, got rank {len(weight.shape)}")
            self._packed = None
            w = torch.as_tensor(weight).to(device=dev, dtype=torch.float32).contiguous()
            self.out_features, self.in_features = int(w.shape[0]), int(w.shape[1])
            self._pad = (-self.in_features) % 32   # the dense product works on 32-value units along K
            if self._pad:
                w = torch.nn.functional.pad(w, (0, self._pad)).contiguous()
            self._dense = api.DeviceWeight.from_device(self.backend, QuantFormat.F32_DENSE, w.view(torch.uint8).reshape(-1),
                                                       self.out_features, self.in_features + self._pad)
        if bias is not None:
            if tuple(bias.shape) != (self.out_features,):
                raise api.ShapeMismatch(f"expected bias [{self.out_features}], got {list(bias.shape)}")
            bias = torch.as_tensor(bias).to(device=dev, dtype=torch.float32).contiguous()
        self._bias = bias

    def weight(self):
        """f32 [out_features, in_features]."""
        if self._packed is not None:
            return self._packed.dequantize()
        return self._dense.dequantize()[:, : self.in_features]

    def bias(self):
        return self._bias

    def forward(self, x, out_dtype=None, check_finite: bool = True):
        torch = api._torch()
        if x.dim() == 0:
            raise api.RankMismatch("expected rank >= 1, got 0")
        if x.shape[-1] != self.in_features:
            raise api.ShapeMismatch(f"expected last dimension {self.in_features}, got {x.shape[-1]}")
        if self._packed is not None:
            y = self._packed.linear(x, self._bias, out_dtype)
        else:
            dev = torch.device("cuda", self.backend.device)
            x = x.to(dev)
            if self._pad:
                x = torch.nn.functional.pad(x, (0, self._pad))
            y = api.quantized_linear(x, self._dense, self._bias, out_dtype)
        if check_finite and not bool(torch.isfinite(y).all()):   # check_output_finite (gptq_loader.rs:309); reads the result back
            raise api.ValueOutOfRange("GptqLinear: non-finite output")
        return y

    __call__ = forward

    def release(self):
        for w in (self._packed, self._dense):
            if w is not None:
                w.release()
        self._packed = self._dense = None


def load_gptq_linear(qweight, scales, qzeros, bias=None, group_size: int = 128, backend: Optional[api.Backend] = None) -> GptqLinear:
    """qweight u32 [in_features / 8, out_features], scales f32 [groups, out_features], qzeros u32
    [groups, out_features / 8], optional bias f32 [out_features]."""
    torch = api._torch()
    b = backend or api.gpu_backend()
    dev = torch.device("cuda", b.device)
    for name, t in (("qweight", qweight), ("scales", scales), ("qzeros", qzeros)):
        if len(t.shape) != 2:
            raise api.RankMismatch(f"{name}: expected a 2-D tensor, got rank {len(t.shape)}")
    qw, qz = _u32(torch, qweight, dev), _u32(torch, qzeros, dev)
    sc = torch.as_tensor(scales).to(device=dev, dtype=torch.float32).contiguous()
    k, n = qw.shape[0] * 8, qw.shape[1]
    groups = sc.shape[0]
    if sc.shape[1] != n:
        raise api.ShapeMismatch(f"expected scales [{groups}, {n}], got {list(sc.shape)}")
    if qz.shape[0] != groups or qz.shape[1] * 8 != n:
        raise api.ShapeMismatch(f"expected zeros [{groups}, {n}], got [{qz.shape[0]}, {qz.shape[1] * 8}]")
    h = ctypes.c_void_p()
    b.check(b._lib.nnq_gq_create_gptq(b._ctx, qw.data_ptr(), sc.data_ptr(), qz.data_ptr(), n, k, groups, int(group_size),
                                      _stream(torch, dev), ctypes.byref(h)))
    return GptqLinear(GroupWeight(b, h.value), bias, GptqFormat(int(group_size), 4, False), b)


load_awq_linear = load_gptq_linear   # awq_loader.rs:74-96: the same unpacking, dequantization and layer
