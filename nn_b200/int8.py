"""Host-side mirror of the reference's INT8 per-channel layer (W8A16):
``quantize_per_channel`` / ``dequantize_per_channel`` (crates/nn-core/src/layers/quantized/int8.rs:82-185)
and ``Int8Linear`` (int8_linear.rs:31-213), over nnq_int8_* of the C ABI. Tensors are torch CUDA
tensors; the weight stays one byte per element on the device and is never expanded to f32 in
``forward``."""
from __future__ import annotations

import math
from typing import Optional

from . import api

SYMMETRIC, ASYMMETRIC = 0, 1   # Int8Mode


class Int8QuantParams:
    """Per-output-channel parameters: scale f32 [N], zero_point int32 [N] (device tensors)."""

    def __init__(self, scale, zero_point):
        self.scale, self.zero_point = scale, zero_point


def _stream(torch, dev):
    return api._stream_ptr(torch.cuda.current_stream(dev))


def quantize_per_channel(weights, mode: int, backend: Optional[api.Backend] = None):
    """f32 [out_features, in_features] -> (uint8 tensor of the signed codes, Int8QuantParams)."""
    torch = api._torch()
    b = backend or api.gpu_backend()
    if len(weights.shape) != 2:
        raise api.RankMismatch(f"expected a 2-D weight, got rank {len(weights.shape)}")
    dev = torch.device("cuda", b.device)
    w = torch.as_tensor(weights).to(device=dev, dtype=torch.float32).contiguous()
    n, k = w.shape
    q = torch.empty((n, k), dtype=torch.uint8, device=dev)
    scale = torch.empty(n, dtype=torch.float32, device=dev)
    zp = torch.empty(n, dtype=torch.int32, device=dev)
    b.check(b._lib.nnq_int8_quantize_per_channel(b._ctx, w.data_ptr(), n, k, int(mode), q.data_ptr(), scale.data_ptr(),
                                                 zp.data_ptr(), _stream(torch, dev)))
    return q, Int8QuantParams(scale, zp)


def dequantize_per_channel(quantized, params: Int8QuantParams, backend: Optional[api.Backend] = None):
    torch = api._torch()
    b = backend or api.gpu_backend()
    if len(quantized.shape) != 2:
        raise api.RankMismatch(f"expected a 2-D weight, got rank {len(quantized.shape)}")
    n, k = quantized.shape
    for name, t in (("scale", params.scale), ("zero_point", params.zero_point)):
        if t.numel() != n:
            raise api.DataLengthMismatch(f"{name}: expected {n} entries, got {t.numel()}")
    out = torch.empty((n, k), dtype=torch.float32, device=quantized.device)
    b.check(b._lib.nnq_int8_dequantize_per_channel(b._ctx, quantized.data_ptr(), params.scale.data_ptr(),
                                                   params.zero_point.data_ptr(), n, k, out.data_ptr(),
                                                   _stream(torch, quantized.device)))
    return out


class Int8Linear:
    def __init__(self, weight_int8, params: Int8QuantParams, bias=None, backend: Optional[api.Backend] = None):
        if len(weight_int8.shape) != 2:
            raise api.RankMismatch(f"expected a 2-D weight, got rank {len(weight_int8.shape)}")
        self.out_features, self.in_features = int(weight_int8.shape[0]), int(weight_int8.shape[1])
        if params.scale.numel() != self.out_features:
            raise api.DataLengthMismatch(f"scale: expected {self.out_features} entries, got {params.scale.numel()}")
        if params.zero_point.numel() != self.out_features:
            raise api.DataLengthMismatch(f"zero_point: expected {self.out_features} entries, got {params.zero_point.numel()}")
        if bias is not None and tuple(bias.shape) != (self.out_features,):
            raise api.ShapeMismatch(f"bias shape mismatch: expected [{self.out_features}], got {list(bias.shape)}")
        self.weight_int8, self.params, self.bias = weight_int8.contiguous(), params, bias
        self.backend = backend or api.gpu_backend()

    @classmethod
    def from_linear(cls, weight, bias=None, mode: int = SYMMETRIC, backend: Optional[api.Backend] = None) -> "Int8Linear":
        q, params = quantize_per_channel(weight, mode, backend)
        if bias is not None:
            bias = api._torch().as_tensor(bias).to(device=q.device, dtype=api._torch().float32).contiguous()
        return cls(q, params, bias, backend)

    def dequantize(self):
        """(f32 weight [N, K], bias)."""
        return dequantize_per_channel(self.weight_int8, self.params, self.backend), self.bias

    def quant_params(self) -> Int8QuantParams:
        return self.params

    def memory_bytes(self) -> int:
        n, k = self.out_features, self.in_features
        return n * k + n * 4 + n + (n * 4 if self.bias is not None else 0)

    def f32_memory_bytes(self) -> int:
        n, k = self.out_features, self.in_features
        return n * k * 4 + (n * 4 if self.bias is not None else 0)

    def compression_ratio(self) -> float:
        return self.f32_memory_bytes() / self.memory_bytes()

    def forward(self, x, out_dtype=None, check_finite: bool = True):
        torch = api._torch()
        if x.dim() == 0:
            raise api.RankMismatch("expected rank >= 1, got 0")
        if x.shape[-1] != self.in_features:
            raise api.ShapeMismatch(f"expected last dimension {self.in_features}, got {x.shape[-1]}")
        b = self.backend
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.float()
        x = x.to(self.weight_int8.device).contiguous()
        m = math.prod(x.shape[:-1]) if x.dim() > 1 else 1
        odt = out_dtype or torch.float32
        y = torch.empty((*x.shape[:-1], self.out_features), dtype=odt, device=x.device)
        b.check(b._lib.nnq_int8_linear(b._ctx, self.weight_int8.data_ptr(), self.params.scale.data_ptr(),
                                       self.params.zero_point.data_ptr(), self.out_features, self.in_features,
                                       x.data_ptr(), api._dtype_code(x), m, self.bias.data_ptr() if self.bias is not None else None,
                                       y.data_ptr(), api._dtype_code(y), _stream(torch, x.device)))
        if check_finite and not bool(torch.isfinite(y).all()):   # check_output_finite (int8_linear.rs:210); reads the result back
            raise api.ValueOutOfRange("Int8Linear: non-finite output")
        return y

    __call__ = forward
