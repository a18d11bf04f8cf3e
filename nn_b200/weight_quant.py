"""Host-side mirror of the reference's INT4 / INT8 per-group weight quantization
(crates/nn-core/src/layers/quantized/weight_quant.rs): ``QuantDtype``, ``QuantizationConfig``,
``QuantizedTensor``, ``quantize_per_group`` (:232), ``dequantize`` (:381), ``quantized_matmul``
(:451), over nnq_group_* / nnq_gq_* of the C ABI. Tensors are torch CUDA tensors; the codes stay
packed on the device and ``quantized_matmul`` does not expand them to f32."""
from __future__ import annotations

import ctypes
import enum
import math
from dataclasses import dataclass
from typing import Optional

from . import api


class QuantDtype(enum.Enum):
    Int4 = 4
    Int8 = 8

    def bits(self) -> int:
        return self.value


@dataclass
class QuantizationConfig:
    dtype: QuantDtype = QuantDtype.Int4
    group_size: int = 128
    symmetric: bool = True

    @classmethod
    def int4(cls, group_size: int) -> "QuantizationConfig":
        return cls(QuantDtype.Int4, group_size, True)

    @classmethod
    def int8(cls, group_size: int) -> "QuantizationConfig":
        return cls(QuantDtype.Int8, group_size, True)


def _stream(torch, dev):
    return api._stream_ptr(torch.cuda.current_stream(dev))


class GroupWeight:
    """Device-resident group-quantized weight (nnq_gq_weight): the operand of the products."""

    def __init__(self, backend: api.Backend, handle: int):
        self.backend, self._handle = backend, handle
        n, k, g, groups = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        bits, streaming = ctypes.c_int(), ctypes.c_int()
        backend.check(backend._lib.nnq_gq_info(handle, ctypes.byref(n), ctypes.byref(k), ctypes.byref(bits), ctypes.byref(g),
                                               ctypes.byref(groups), ctypes.byref(streaming)))
        self.out_features, self.in_features = n.value, k.value
        self.bits, self.group_size, self.groups, self.streaming = bits.value, g.value, groups.value, bool(streaming.value)

    def dequantize(self):
        torch = api._torch()
        dev = torch.device("cuda", self.backend.device)
        out = torch.empty((self.out_features, self.in_features), dtype=torch.float32, device=dev)
        self.backend.check(self.backend._lib.nnq_gq_dequantize(self._handle, out.data_ptr(), _stream(torch, dev)))
        return out

    def linear(self, x, bias=None, out_dtype=None):
        """y[*, N] = x[*, K] . w^T (+ bias)."""
        torch = api._torch()
        if x.dim() == 0:
            raise api.RankMismatch("expected rank >= 1, got 0")
        if x.shape[-1] != self.in_features:
            raise api.ShapeMismatch(f"expected last dimension {self.in_features}, got {x.shape[-1]}")
        dev = torch.device("cuda", self.backend.device)
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.float()
        x = x.to(dev).contiguous()
        m = math.prod(x.shape[:-1]) if x.dim() > 1 else 1
        y = torch.empty((*x.shape[:-1], self.out_features), dtype=out_dtype or torch.float32, device=dev)
        b = self.backend
        b.check(b._lib.nnq_gq_linear(self._handle, x.data_ptr(), api._dtype_code(x), m,
                                     bias.data_ptr() if bias is not None else None, y.data_ptr(), api._dtype_code(y),
                                     _stream(torch, dev)))
        return y

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_gq_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.release()
        except Exception:
            pass


class QuantizedTensor:
    """``QuantizedTensor`` (weight_quant.rs:153-215): packed codes (uint8), scales f32 and
    zero_points int32 per group (device tensors), the configuration and the shape."""

    def __init__(self, quantized_data, scales, zero_points, config: QuantizationConfig, shape, backend: Optional[api.Backend] = None):
        self.quantized_data, self.scales, self.zero_points = quantized_data, scales, zero_points
        self.config, self.shape = config, [int(shape[0]), int(shape[1])]
        self.backend = backend or api.gpu_backend()
        self._weight: Optional[GroupWeight] = None

    def out_features(self) -> int:
        return self.shape[0]

    def in_features(self) -> int:
        return self.shape[1]

    def num_groups_per_row(self) -> int:
        return self.shape[1] // self.config.group_size

    def total_groups(self) -> int:
        return self.shape[0] * self.num_groups_per_row()

    def memory_bytes(self) -> int:
        return self.quantized_data.numel() + self.scales.numel() * 4 + self.zero_points.numel() * 4

    def f32_memory_bytes(self) -> int:
        return self.shape[0] * self.shape[1] * 4

    def compression_ratio(self) -> float:
        mb = self.memory_bytes()
        return 0.0 if mb == 0 else self.f32_memory_bytes() / mb

    def device_weight(self) -> GroupWeight:
        """The resident operand, created on first use (a load-time step)."""
        if self._weight is None:
            torch = api._torch()
            b = self.backend
            n, k = self.shape
            expected = n * self.num_groups_per_row()
            if self.scales.numel() != expected:
                raise api.DataLengthMismatch(f"scales: expected {expected} entries, got {self.scales.numel()}")
            if self.zero_points.numel() != expected:
                raise api.DataLengthMismatch(f"zero_points: expected {expected} entries, got {self.zero_points.numel()}")
            h = ctypes.c_void_p()
            dev = torch.device("cuda", b.device)
            b.check(b._lib.nnq_gq_create_per_group(b._ctx, self.quantized_data.data_ptr(), self.scales.data_ptr(),
                                                   self.zero_points.data_ptr(), n, k, self.config.dtype.bits(),
                                                   int(self.config.group_size), _stream(torch, dev), ctypes.byref(h)))
            self._weight = GroupWeight(b, h.value)
        return self._weight

    def release(self):
        if self._weight is not None:
            self._weight.release()
            self._weight = None


def quantize_per_group(weights, config: QuantizationConfig, backend: Optional[api.Backend] = None) -> QuantizedTensor:
    """f32 [out_features, in_features] -> QuantizedTensor with the reference's codes, scales and
    zero points, bit for bit."""
    torch = api._torch()
    b = backend or api.gpu_backend()
    if len(weights.shape) != 2:
        raise api.RankMismatch(f"expected a 2-D weight, got rank {len(weights.shape)}")
    dev = torch.device("cuda", b.device)
    w = torch.as_tensor(weights).to(device=dev, dtype=torch.float32).contiguous()
    n, k = w.shape
    g = int(config.group_size)
    bits = config.dtype.bits()
    gpr = k // g if g > 0 and k % g == 0 else 0
    q = torch.zeros(n * k if bits == 8 else (n * k + 1) // 2, dtype=torch.uint8, device=dev)
    scale = torch.zeros(n * gpr, dtype=torch.float32, device=dev)
    zp = torch.zeros(n * gpr, dtype=torch.int32, device=dev)
    b.check(b._lib.nnq_group_quantize(b._ctx, w.data_ptr(), n, k, bits, g, int(bool(config.symmetric)), q.data_ptr(),
                                      scale.data_ptr(), zp.data_ptr(), _stream(torch, dev)))
    return QuantizedTensor(q, scale, zp, QuantizationConfig(config.dtype, g, config.symmetric), [n, k], b)


def dequantize(qt: QuantizedTensor):
    """f32 [out_features, in_features], bit-identical to the reference's dequantize."""
    torch = api._torch()
    b = qt.backend
    n, k = qt.shape
    expected = n * qt.num_groups_per_row()
    if qt.scales.numel() != expected:
        raise api.DataLengthMismatch(f"expected {expected} scales, got {qt.scales.numel()}")
    dev = torch.device("cuda", b.device)
    out = torch.empty((n, k), dtype=torch.float32, device=dev)
    b.check(b._lib.nnq_group_dequantize(b._ctx, qt.quantized_data.data_ptr(), qt.scales.data_ptr(), qt.zero_points.data_ptr(),
                                        n, k, qt.config.dtype.bits(), int(qt.config.group_size), out.data_ptr(),
                                        _stream(torch, dev)))
    return out


def quantized_matmul(input, weight: QuantizedTensor, out_dtype=None):
    """``input @ weight^T`` for input [*, in_features]; output [*, out_features]."""
    if input.dim() == 0:
        raise api.RankMismatch("expected rank >= 1, got 0")
    if input.shape[-1] != weight.in_features():
        raise api.ShapeMismatch(f"expected last dimension {weight.in_features()}, got {input.shape[-1]}")
    return weight.device_weight().linear(input, None, out_dtype)
