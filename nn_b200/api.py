"""Host-side mirror of the reference's operator interface for the quantized matmul path.

Same names, argument meaning and error behaviour as nn-core's
``quantized_matmul_q4_0`` / ``quantized_matmul_q8_0`` / ``quantized_linear``
(crates/nn-core/src/dyn_tensor/quantized_matmul.rs:296,335,367),
``DynTensor::from_quantized`` / ``dequantize`` / ``is_quantized``
(crates/nn-core/src/dyn_tensor/quantized.rs:270-322), ``QLinear``
(crates/nn-core/src/layers/quantized/linear.rs:292-399) and the backend registry
(crates/nn-core/src/dyn_tensor/gpu.rs:156-170). Everything computes through the C ABI
of libnnq_b200.so; torch is used only to own device memory and streams.

The reference is Rust and no Rust toolchain exists in this environment, so this mirror
is Python over ctypes; a Rust shim would bind the same symbols.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence

import numpy as np

from . import _lib
from .formats import GEOMETRY, QuantFormat

# --------------------------------------------------------------------------- #
# errors: TensorError and QuantizedMatmulError of the reference
# --------------------------------------------------------------------------- #


class TensorError(Exception):
    """Base of every error this package raises (nn-core ``TensorError``)."""


class Unsupported(TensorError):
    """``TensorError::Unsupported``; QuantizedMatmulError converts into it
    (crates/nn-core/src/dyn_tensor/quantized_matmul.rs:78-82)."""


class NotQuantized(Unsupported):
    pass


class WrongQuantType(Unsupported):
    pass


class ShapeMismatch(Unsupported):
    pass


class WeightRank(Unsupported):
    pass


class BiasMismatch(Unsupported):
    pass


class InvalidShape(TensorError):
    pass


class DataLengthMismatch(TensorError):
    pass


class RankMismatch(TensorError):
    pass


class InvalidArgument(TensorError):
    pass


class ValueOutOfRange(TensorError):
    """``TensorError::ValueOutOfRange``: a non-finite value reached an encoder."""


class BackendFailure(TensorError):
    """``TensorError::BackendFailure{domain: Cuda, kind, message}``."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


_STATUS_ERRORS = {
    1: InvalidArgument, 2: NotQuantized, 3: WrongQuantType, 4: ShapeMismatch, 5: WeightRank, 6: BiasMismatch,
    7: InvalidShape, 8: DataLengthMismatch, 9: RankMismatch, 10: Unsupported, 11: ValueOutOfRange,
}
_BACKEND_KINDS = {20: "OutOfMemory", 21: "DispatchFailed", 22: "Timeout", 23: "NoDevice", 24: "Other"}

F32, BF16 = 0, 1
PATH_AUTO, PATH_GENERIC, PATH_SKINNY, PATH_TENSOR = 0, 1, 2, 3


def _torch():
    import torch
    return torch


# --------------------------------------------------------------------------- #
# backend (context) and its registry
# --------------------------------------------------------------------------- #


class Backend:
    """One nnq context on one CUDA device (the reference's ``GpuFullBackend`` object)."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        ctx = ctypes.c_void_p()
        st = self._lib.nnq_init(int(device), ctypes.byref(ctx))
        if st != 0:
            raise BackendFailure(_BACKEND_KINDS.get(st, "Other"),
                                 f"nnq_init(device={device}): {self._lib.nnq_status_str(st).decode()}")
        self._ctx = ctx
        self.device = int(device)

    def backend_name(self) -> str:
        return "nnq-b200"

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.nnq_destroy(self._ctx)
            self._ctx = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def check(self, status: int):
        if status == 0:
            return
        msg = self._lib.nnq_last_error(self._ctx).decode() or self._lib.nnq_status_str(status).decode()
        if status in _STATUS_ERRORS:
            raise _STATUS_ERRORS[status](msg)
        raise BackendFailure(_BACKEND_KINDS.get(status, "Other"), msg)

    def set_path(self, path: int):
        self.check(self._lib.nnq_set_path(self._ctx, int(path)))

    def device_status(self, stream=None):
        self.check(self._lib.nnq_device_status(self._ctx, _stream_ptr(stream)))

    def launch_count(self) -> int:
        return int(self._lib.nnq_launch_count(self._ctx))


_BACKEND: Optional[Backend] = None


def register_gpu_backend(backend: Backend) -> bool:
    """Install the process-wide backend once; later calls are ignored and return False
    (``OnceLock`` semantics of crates/nn-core/src/dyn_tensor/gpu.rs:156-162)."""
    global _BACKEND
    if _BACKEND is not None:
        return False
    _BACKEND = backend
    return True


def gpu_backend() -> Backend:
    """The registered backend; creates one on device 0 on first use."""
    global _BACKEND
    if _BACKEND is None:
        _BACKEND = Backend(0)
    return _BACKEND


def _stream_ptr(stream) -> ctypes.c_void_p:
    if stream is None:
        torch = _torch()
        stream = torch.cuda.current_stream()
    return ctypes.c_void_p(int(getattr(stream, "cuda_stream", stream)))


# --------------------------------------------------------------------------- #
# quantized tensor
# --------------------------------------------------------------------------- #


def _as_bytes(a) -> np.ndarray:
    if isinstance(a, (bytes, bytearray, memoryview)):
        return np.frombuffer(bytes(a), np.uint8)
    return np.ascontiguousarray(a, np.uint8).reshape(-1)


class QuantizedTensor:
    """Raw block-quantized bytes plus logical shape: the ``TensorStorage::Quantized``
    variant of DynTensor. The logical dtype is f32. A device copy is made on first use."""

    def __init__(self, data, quant_type: QuantFormat, shape: Sequence[int], scales=None,
                 backend: Optional[Backend] = None):
        self.quant_type = QuantFormat(quant_type)
        self.shape = tuple(int(s) for s in shape)
        g = GEOMETRY[self.quant_type]
        numel = math.prod(self.shape) if self.shape else 1
        if numel % g.elems != 0:
            raise InvalidShape(f"element count {numel} is not a multiple of {self.quant_type.name} "
                               f"block size {g.elems}")
        self.data = _as_bytes(data)
        blocks = numel // g.elems
        if self.data.size != blocks * g.bytes:
            raise DataLengthMismatch(f"expected {blocks * g.bytes} bytes, got {self.data.size}")
        self.scales = _as_bytes(scales) if scales is not None else None
        if g.scale_bytes and (self.scales is None or self.scales.size != blocks * g.scale_bytes):
            raise DataLengthMismatch(f"expected {blocks * g.scale_bytes} scale bytes")
        self._backend = backend
        self._handle = None

    # -- reference API -----------------------------------------------------
    @classmethod
    def from_quantized(cls, data, quant_type, shape, scales=None, backend=None) -> "QuantizedTensor":
        return cls(data, quant_type, shape, scales, backend)

    def dims(self):
        return self.shape

    def is_quantized(self) -> bool:
        return True

    def rank(self) -> int:
        return len(self.shape)

    # -- device side -------------------------------------------------------
    @property
    def backend(self) -> Backend:
        if self._backend is None:
            self._backend = gpu_backend()
        return self._backend

    def handle(self) -> ctypes.c_void_p:
        """nnq_weight of a 2-D tensor (uploaded once, like Linear's cached device weight)."""
        if self._handle is None:
            if len(self.shape) != 2:
                raise WeightRank(f"quantized weight must be 2-D [out_features, in_features], got rank {len(self.shape)}")
            b = self.backend
            h = ctypes.c_void_p()
            sp, sn = (self.scales.ctypes.data, self.scales.size) if self.scales is not None else (None, 0)
            b.check(b._lib.nnq_weight_create(b._ctx, int(self.quant_type), self.data.ctypes.data, self.data.size,
                                             sp, sn, self.shape[0], self.shape[1], ctypes.byref(h)))
            self._handle = h
        return self._handle

    def shard(self, axis: int, rank: int, world: int) -> "DeviceWeight":
        """Tensor-parallel shard: axis 0 splits rows (column-parallel), axis 1 splits K in
        whole blocks (row-parallel)."""
        if len(self.shape) != 2:
            raise WeightRank(f"quantized weight must be 2-D, got rank {len(self.shape)}")
        b = self.backend
        h = ctypes.c_void_p()
        sp, sn = (self.scales.ctypes.data, self.scales.size) if self.scales is not None else (None, 0)
        b.check(b._lib.nnq_weight_create_shard(b._ctx, int(self.quant_type), self.data.ctypes.data, self.data.size,
                                               sp, sn, self.shape[0], self.shape[1], axis, rank, world,
                                               ctypes.byref(h)))
        return DeviceWeight(b, h)

    def dequantize(self):
        """f32 tensor of the logical shape, on the backend's device (bit-exact decode)."""
        torch = _torch()
        b = self.backend
        dev = torch.device("cuda", b.device)
        numel = math.prod(self.shape) if self.shape else 1
        out = torch.empty(numel, dtype=torch.float32, device=dev)
        if len(self.shape) == 2:
            b.check(b._lib.nnq_dequantize(b._ctx, self.handle(), out.data_ptr(), _stream_ptr(None)))
        else:
            raw = torch.from_numpy(self.data).to(dev)
            sc = torch.from_numpy(self.scales).to(dev) if self.scales is not None else None
            n = ctypes.c_int64()
            b.check(b._lib.nnq_dequantize_raw(b._ctx, int(self.quant_type), raw.data_ptr(), raw.numel(),
                                              sc.data_ptr() if sc is not None else None,
                                              sc.numel() if sc is not None else 0, numel, out.data_ptr(),
                                              ctypes.byref(n), _stream_ptr(None)))
        return out.reshape(self.shape)

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_weight_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.release()
        except Exception:
            pass


class DeviceWeight:
    """Owning wrapper of an nnq_weight created directly on the device (e.g. a TP shard)."""

    def __init__(self, backend: Backend, handle: ctypes.c_void_p):
        self.backend = backend
        self._handle = handle
        fmt, n, k = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64()
        nb, sb = ctypes.c_size_t(), ctypes.c_size_t()
        backend.check(backend._lib.nnq_weight_info(handle, ctypes.byref(fmt), ctypes.byref(n), ctypes.byref(k),
                                                   ctypes.byref(nb), ctypes.byref(sb)))
        self.quant_type = QuantFormat(fmt.value)
        self.shape = (n.value, k.value)
        self.nbytes = nb.value + sb.value

    @classmethod
    def from_device(cls, backend: Backend, quant_type, data, n: int, k: int, scales=None,
                    shard=None) -> "DeviceWeight":
        """Wrap raw blocks already resident on the device (torch uint8 tensors). With
        shard=(axis, rank, world) only that tensor-parallel shard is kept."""
        h = ctypes.c_void_p()
        sp, sn = (scales.data_ptr(), scales.numel()) if scales is not None else (None, 0)
        if shard is None:
            backend.check(backend._lib.nnq_weight_create(backend._ctx, int(quant_type), data.data_ptr(),
                                                         data.numel(), sp, sn, n, k, ctypes.byref(h)))
        else:
            axis, rank, world = shard
            backend.check(backend._lib.nnq_weight_create_shard(backend._ctx, int(quant_type), data.data_ptr(),
                                                               data.numel(), sp, sn, n, k, axis, rank, world,
                                                               ctypes.byref(h)))
        return cls(backend, h)

    def handle(self):
        return self._handle

    def is_quantized(self):
        return True

    def dims(self):
        return self.shape

    def rank(self):
        return 2

    def dequantize(self):
        torch = _torch()
        out = torch.empty(self.shape, dtype=torch.float32, device=torch.device("cuda", self.backend.device))
        self.backend.check(self.backend._lib.nnq_dequantize(self.backend._ctx, self._handle, out.data_ptr(),
                                                            _stream_ptr(None)))
        return out

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_weight_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.release()
        except Exception:
            pass


def from_quantized(data, quant_type, shape, scales=None) -> QuantizedTensor:
    """``DynTensor::from_quantized(data, quant_type, shape)``."""
    return QuantizedTensor(data, quant_type, shape, scales)


def quantize(values, quant_type, backend: Optional[Backend] = None):
    """Encode f32 values into blocks on the device with the reference's encoders:
    ``Q4_K_GGML`` = ``BlockQ4K::quantize`` as ``QLinear::from_linear`` applies it
    (crates/nn-core/src/layers/quantized/linear.rs:95-162,309-343), ``MXFP4_CORE`` =
    ``quantize_tensor`` (mxfp4.rs:307-329), ``MXFP4_GPTOSS`` = ``Mxfp4Tensor::quantize``
    (crates/nn-gptoss/src/quantize.rs:122-153). `values`: torch tensor (moved to the backend's
    device as f32) or numpy array; the tail block is zero-padded. Returns (uint8 device tensor
    of blocks, uint8 device tensor of scale bytes or None). A non-finite value raises
    ValueOutOfRange where the reference does."""
    torch = _torch()
    b = backend or gpu_backend()
    fmt = QuantFormat(quant_type)
    dev = torch.device("cuda", b.device)
    v = torch.as_tensor(values).to(device=dev, dtype=torch.float32).contiguous().reshape(-1)
    g = GEOMETRY[fmt]
    nb = (v.numel() + g.elems - 1) // g.elems
    out = torch.empty(nb * g.bytes, dtype=torch.uint8, device=dev)
    sc = torch.empty(nb * g.scale_bytes, dtype=torch.uint8, device=dev) if g.scale_bytes else None
    blocks = ctypes.c_int64()
    b.check(b._lib.nnq_quantize(b._ctx, int(fmt), v.data_ptr() if v.numel() else None, v.numel(),
                                out.data_ptr() if nb else None, out.numel(), sc.data_ptr() if sc is not None and nb else None,
                                sc.numel() if sc is not None else 0, ctypes.byref(blocks),
                                _stream_ptr(torch.cuda.current_stream(dev))))
    assert blocks.value == nb
    return out, sc


# --------------------------------------------------------------------------- #
# the op API
# --------------------------------------------------------------------------- #


def _is_quantized(w) -> bool:
    return isinstance(w, (QuantizedTensor, DeviceWeight))


def _dtype_code(t) -> int:
    torch = _torch()
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise Unsupported(f"activation dtype {t.dtype} is not supported (f32 or bf16)")


def _matmul(input, weight, out_dtype=None):
    """x[.., M, K] * W^T -> [.., M, N]. torch CUDA tensors stay on the device; numpy arrays
    and torch CPU tensors take the host entry point (copies inside the call)."""
    torch = _torch()
    dims = tuple(input.shape)
    if len(dims) < 2:
        raise RankMismatch(f"expected rank >= 2, got {len(dims)}")
    n, k = weight.dims()
    if dims[-1] != k:
        raise ShapeMismatch(f"quantized matmul shape mismatch: input last dim {dims[-1]} != weight in_features {k}")
    m = math.prod(dims[:-1])
    b = weight.backend
    h = weight.handle()
    out_shape = dims[:-1] + (n,)
    if isinstance(input, np.ndarray) or not input.is_cuda:
        host = input if isinstance(input, np.ndarray) else input.numpy()
        if host.dtype != np.float32:
            raise Unsupported("host activations must be f32")
        host = np.ascontiguousarray(host)
        y = np.empty(out_shape, np.float32)
        b.check(b._lib.nnq_linear_host(b._ctx, h, host.ctypes.data, F32, m, None, y.ctypes.data, F32))
        return y if isinstance(input, np.ndarray) else torch.from_numpy(y)
    x = input.contiguous()
    ydt = x.dtype if out_dtype is None else out_dtype
    y = torch.empty(out_shape, dtype=ydt, device=x.device)
    b.check(b._lib.nnq_linear(b._ctx, h, x.data_ptr(), _dtype_code(x), m, None, y.data_ptr(), _dtype_code(y),
                              _stream_ptr(None)))
    return y


def _quantized_matmul_typed(input, weight, expected: QuantFormat, out_dtype=None):
    # order of checks follows validate_quantized_weight then validate_input
    # (crates/nn-core/src/dyn_tensor/quantized_matmul.rs:87-143)
    if not _is_quantized(weight):
        raise NotQuantized(f"weight tensor is not quantized (expected {expected.name})")
    if weight.quant_type != expected:
        raise WrongQuantType(f"weight quantization type mismatch: expected {expected.name}, "
                             f"got {weight.quant_type.name}")
    if weight.rank() != 2:
        raise WeightRank(f"quantized weight must be 2-D [out_features, in_features], got rank {weight.rank()}")
    return _matmul(input, weight, out_dtype)


def quantized_matmul_q4_0(input, weight, out_dtype=None):
    """``input @ weight^T`` with Q4_0 weights -> [.., M, N]."""
    return _quantized_matmul_typed(input, weight, QuantFormat.Q4_0, out_dtype)


def quantized_matmul_q8_0(input, weight, out_dtype=None):
    """``input @ weight^T`` with Q8_0 weights -> [.., M, N]."""
    return _quantized_matmul_typed(input, weight, QuantFormat.Q8_0, out_dtype)


def quantized_matmul(input, weight, out_dtype=None):
    """Format-agnostic product: the quantized branch of ``DynTensor::matmul``
    (crates/nn-core/src/dyn_tensor/ops/mod.rs:284-297) without the dequantize detour."""
    if not _is_quantized(weight):
        raise NotQuantized("weight tensor is not quantized")
    if weight.rank() != 2:
        raise WeightRank(f"quantized weight must be 2-D [out_features, in_features], got rank {weight.rank()}")
    return _matmul(input, weight, out_dtype)


def quantized_linear(input, weight, bias=None, out_dtype=None):
    """``y = input @ weight^T + bias``; the format comes from the weight. As in the
    reference the product is formed first and the bias shape is checked afterwards
    (crates/nn-core/src/dyn_tensor/quantized_matmul.rs:367-405)."""
    if not _is_quantized(weight):
        raise Unsupported("quantized_linear: weight is not quantized")
    if weight.rank() != 2:
        raise WeightRank(f"quantized weight must be 2-D [out_features, in_features], got rank {weight.rank()}")
    if bias is None:
        return _matmul(input, weight, out_dtype)
    torch = _torch()
    dims = tuple(input.shape)
    if len(dims) < 2:
        raise RankMismatch(f"expected rank >= 2, got {len(dims)}")
    n, k = weight.dims()
    if dims[-1] != k:
        raise ShapeMismatch(f"quantized matmul shape mismatch: input last dim {dims[-1]} != weight in_features {k}")
    if tuple(bias.shape) != (n,):
        raise BiasMismatch(f"bias shape mismatch: expected [{n}], got {list(bias.shape)}")
    m = math.prod(dims[:-1])
    b = weight.backend
    out_shape = dims[:-1] + (n,)
    if isinstance(input, np.ndarray) or not input.is_cuda:
        host = np.ascontiguousarray(input if isinstance(input, np.ndarray) else input.numpy(), np.float32)
        hb = np.ascontiguousarray(bias if isinstance(bias, np.ndarray) else bias.cpu().numpy(), np.float32)
        y = np.empty(out_shape, np.float32)
        b.check(b._lib.nnq_linear_host(b._ctx, weight.handle(), host.ctypes.data, F32, m, hb.ctypes.data,
                                       y.ctypes.data, F32))
        return y if isinstance(input, np.ndarray) else torch.from_numpy(y)
    x = input.contiguous()
    bias_dev = bias.to(device=x.device, dtype=torch.float32).contiguous()
    ydt = x.dtype if out_dtype is None else out_dtype
    y = torch.empty(out_shape, dtype=ydt, device=x.device)
    b.check(b._lib.nnq_linear(b._ctx, weight.handle(), x.data_ptr(), _dtype_code(x), m, bias_dev.data_ptr(),
                              y.data_ptr(), _dtype_code(y), _stream_ptr(None)))
    return y


def _linear_batch_host(inputs, weights, biases):
    """Host tensors (numpy f32): one staged copy in, one out, one synchronisation for the batch."""
    count = len(weights)
    b = weights[0].backend
    xs = [np.ascontiguousarray(x, dtype=np.float32) for x in inputs]
    # inputs given as the same array object share their device copy (and one launch)
    for i in range(count):
        for j in range(i):
            if inputs[i] is inputs[j]:
                xs[i] = xs[j]
    m = math.prod(xs[0].shape[:-1])
    ys = []
    for x, w in zip(xs, weights):
        n, k = w.dims()
        if x.shape[-1] != k:
            raise ShapeMismatch(f"input last dim {x.shape[-1]} != weight in_features {k}")
        ys.append(np.empty(tuple(x.shape[:-1]) + (n,), np.float32))
    VP = ctypes.c_void_p * count
    wh = VP(*[w.handle().value for w in weights])
    xp = VP(*[x.ctypes.data for x in xs])
    yp = VP(*[y.ctypes.data for y in ys])
    bp, keep = None, []
    if biases is not None:
        keep = [np.ascontiguousarray(bb, dtype=np.float32) if bb is not None else None for bb in biases]
        bp = VP(*[(t.ctypes.data if t is not None else None) for t in keep])
    b.check(b._lib.nnq_linear_batch_host(b._ctx, count, wh, xp, F32, m, bp, yp, F32))
    return ys


def linear_batch(inputs, weights, biases=None, out_dtype=None):
    """Several products in one call (same M and dtype): q/k/v or gate/up of a decoder layer.
    numpy inputs take the host entry point (nnq_linear_batch_host) and return numpy arrays."""
    if isinstance(inputs[0], np.ndarray):
        return _linear_batch_host(inputs, weights, biases)
    torch = _torch()
    count = len(weights)
    b = weights[0].backend
    xs = [x.contiguous() for x in inputs]
    m = math.prod(xs[0].shape[:-1])
    ydt = xs[0].dtype if out_dtype is None else out_dtype
    ys = []
    for x, w in zip(xs, weights):
        n, k = w.dims()
        if x.shape[-1] != k:
            raise ShapeMismatch(f"input last dim {x.shape[-1]} != weight in_features {k}")
        ys.append(torch.empty(tuple(x.shape[:-1]) + (n,), dtype=ydt, device=x.device))
    VP = ctypes.c_void_p * count
    wh = VP(*[w.handle().value for w in weights])
    xp = VP(*[x.data_ptr() for x in xs])
    yp = VP(*[y.data_ptr() for y in ys])
    bp = None
    keep = []
    if biases is not None:
        keep = [bb.to(device=xs[0].device, dtype=torch.float32).contiguous() if bb is not None else None
                for bb in biases]
        bp = VP(*[(t.data_ptr() if t is not None else None) for t in keep])
    b.check(b._lib.nnq_linear_batch(b._ctx, count, wh, xp, _dtype_code(xs[0]), m, bp, yp, _dtype_code(ys[0]),
                                    _stream_ptr(None)))
    return ys


# --------------------------------------------------------------------------- #
# QLinear
# --------------------------------------------------------------------------- #


class QLinear:
    """Linear layer over quantized weights: ``forward(x) = x @ W^T (+ bias)``.

    The reference's ``QLinear::forward`` dequantizes the whole weight and then calls a
    dense matmul on every call (crates/nn-core/src/layers/quantized/linear.rs:366-399);
    here the blocks are decoded inside the product kernel and never materialised.
    """

    def __init__(self, weight: QuantizedTensor, bias=None):
        if not _is_quantized(weight):
            raise NotQuantized("QLinear needs a quantized weight")
        if weight.rank() != 2:
            raise WeightRank(f"quantized weight must be 2-D [out_features, in_features], got rank {weight.rank()}")
        if bias is not None and tuple(bias.shape) != (weight.dims()[0],):
            raise BiasMismatch(f"bias shape mismatch: expected [{weight.dims()[0]}], got {list(bias.shape)}")
        self.weight = weight
        self.bias = bias

    @classmethod
    def from_linear(cls, weight, bias=None, backend: Optional[Backend] = None) -> "QLinear":
        """``QLinear::from_linear(linear, GgmlDType::Q4K)`` (linear.rs:309-343): quantize an f32
        [out_features, in_features] weight to nn-core's Q4_K blocks on the device. The product
        needs blocks that do not straddle rows: in_features must be a multiple of 256."""
        if len(weight.shape) != 2:
            raise WeightRank(f"weight must be 2-D [out_features, in_features], got rank {len(weight.shape)}")
        n, k = int(weight.shape[0]), int(weight.shape[1])
        if k % 256:
            raise Unsupported(f"in_features {k} is not a multiple of the Q4_K block (256)")
        b = backend or gpu_backend()
        blocks, _ = quantize(weight, QuantFormat.Q4_K_GGML, b)
        return cls(DeviceWeight.from_device(b, QuantFormat.Q4_K_GGML, blocks, n, k), bias)

    def is_quantized(self) -> bool:
        return True

    def forward(self, xs, out_dtype=None):
        return quantized_linear(xs, self.weight, self.bias, out_dtype)

    __call__ = forward

    def dequantize(self):
        """(f32 weight [N, K], bias): ``QLinear::dequantize``."""
        return self.weight.dequantize(), self.bias
