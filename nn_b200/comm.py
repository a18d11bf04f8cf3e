"""Tensor-parallel exchange between the ranks of one box (one process per GPU).

``PeerComm`` wraps the library's one-shot all-reduce over peer-mapped buffers (nnq_comm_*);
the handle exchange goes through ``torch.distributed`` (any backend: it is host data)."""
from __future__ import annotations

import ctypes

from . import api


class PeerComm:
    def __init__(self, backend: api.Backend, rank: int, world: int, max_bytes: int = 1 << 16, group=None,
                 exchange_handles: bool = True):
        self.backend, self.rank, self.world = backend, rank, world
        h = ctypes.c_void_p()
        backend.check(backend._lib.nnq_comm_create(backend._ctx, rank, world, max_bytes, ctypes.byref(h)))
        self._handle = h
        if world > 1 and exchange_handles:
            import torch.distributed as dist
            mine = ctypes.create_string_buffer(64)
            backend.check(backend._lib.nnq_comm_get_handle(h, mine))
            gathered = [None] * world
            dist.all_gather_object(gathered, bytes(mine.raw), group=group)
            blob = ctypes.create_string_buffer(b"".join(gathered), 64 * world)
            backend.check(backend._lib.nnq_comm_open_peers(h, blob))
            dist.barrier(group=group)

    def local_buffer(self) -> int:
        """Device address of this rank's exchange buffer (for open_local_peers of the other ranks)."""
        p = ctypes.c_void_p()
        self.backend.check(self.backend._lib.nnq_comm_local_buffer(self._handle, ctypes.byref(p)))
        return p.value

    def open_local_peers(self, buffers):
        """Single-process set-up: `buffers[r]` is rank r's local_buffer(), valid in this process."""
        arr = (ctypes.c_void_p * self.world)(*[ctypes.c_void_p(b) for b in buffers])
        self.backend.check(self.backend._lib.nnq_comm_open_local_peers(self._handle, arr))

    def set_spin_limit(self, polls: int):
        """Bound of the device-side waits (polls of a flag); a wait that runs out surfaces as
        BackendFailure(kind="Timeout") from Backend.device_status()."""
        self.backend.check(self.backend._lib.nnq_comm_set_spin_limit(self._handle, int(polls)))

    def all_reduce(self, tensor, stream=None):
        """In-place sum over the ranks of a contiguous f32 / bf16 CUDA tensor."""
        b = self.backend
        b.check(b._lib.nnq_comm_all_reduce(self._handle, tensor.data_ptr(), api._dtype_code(tensor), tensor.numel(),
                                           api._stream_ptr(stream)))
        return tensor

    def all_reduce_raw(self, ptr: int, dtype_code: int, count: int, stream_ptr):
        return self.backend._lib.nnq_comm_all_reduce(self._handle, ptr, dtype_code, count, stream_ptr)

    def linear_raw(self, weight_handle, x_ptr: int, x_dt: int, m: int, bias_ptr, y_ptr: int, y_dt: int, stream_ptr):
        """Row-parallel product fused with its all-reduce (nnq_comm_linear); returns the status."""
        return self.backend._lib.nnq_comm_linear(self._handle, weight_handle, x_ptr, x_dt, m, bias_ptr, y_ptr, y_dt,
                                                 stream_ptr)

    def linear(self, x, weight, bias=None, out_dtype=None, stream=None):
        """y = sum over ranks of x_r @ W_r^T (+ bias once); x is this rank's [M, K/world] slice."""
        import torch
        m = x.shape[0] if x.dim() > 1 else 1
        y = torch.empty((m, weight.shape[0]), dtype=out_dtype or torch.float32, device=x.device)
        b = self.backend
        b.check(self.linear_raw(weight.handle(), x.data_ptr(), api._dtype_code(x), m,
                                bias.data_ptr() if bias is not None else None, y.data_ptr(), api._dtype_code(y),
                                api._stream_ptr(stream)))
        return y

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_comm_destroy(self._handle)
            self._handle = None
