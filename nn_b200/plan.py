"""Compiled product plan: a recorded sequence of one-token products run as one kernel launch.

Mirrors, for the quantized products, the reference's compiled dispatch plan (built once, replayed
per step: ``CompiledModel::builder(..).build()`` crates/nn-metal/src/compiled_model.rs:305-311,
``run_steps`` crates/nn-metal/src/compiled_model_execute.rs:124). Everything computes through the
C ABI (``nnq_plan_*``); torch only owns the buffers.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

from . import api

ANALYZE_DEPS = 1


class ProductPlan:
    """Groups of products that share their input, added in the order a decoder layer issues them
    (q / k / v, o, gate / up, down ...). ``run`` gives what the same ``quantized_linear`` calls give
    when made one after another."""

    def __init__(self, backend: Optional[api.Backend] = None, x_dtype=None, y_dtype=None, analyze_deps: bool = False):
        torch = api._torch()
        self.backend = backend or api.gpu_backend()
        self.x_dtype = x_dtype or torch.bfloat16
        self.y_dtype = y_dtype or torch.float32
        h = ctypes.c_void_p()
        b = self.backend
        b.check(b._lib.nnq_plan_create(b._ctx, _code(self.x_dtype), _code(self.y_dtype), ANALYZE_DEPS if analyze_deps else 0,
                                       ctypes.byref(h)))
        self._handle = h
        self._keep = []   # tensors and weights the plan points at

    def add(self, weights: Sequence, x, ys: Sequence, biases: Optional[Sequence] = None):
        """One group: ys[i] = x @ weights[i]^T (+ biases[i]); x is a [K] or [1, K] tensor."""
        b = self.backend
        n = len(weights)
        if len(ys) != n or (biases is not None and len(biases) != n):
            raise api.InvalidArgument("weights, outputs and biases must have the same length")
        if x.dtype != self.x_dtype or any(y.dtype != self.y_dtype for y in ys):
            raise api.InvalidArgument("tensor dtypes must match the plan's")
        VP = ctypes.c_void_p
        wh = (VP * n)(*[w.handle().value for w in weights])
        yp = (VP * n)(*[y.data_ptr() for y in ys])
        bp = None
        if biases is not None:
            bp = (VP * n)(*[(bi.data_ptr() if bi is not None else None) for bi in biases])
        b.check(b._lib.nnq_plan_add(self._handle, n, wh, x.data_ptr(), bp, yp))
        self._keep.append((list(weights), x, list(ys), list(biases) if biases is not None else None))

    def add_reduced(self, comm, weight, x, y, bias=None):
        """A row-parallel product summed over the ranks of ``comm`` inside the kernel."""
        b = self.backend
        if x.dtype != self.x_dtype or y.dtype != self.y_dtype:
            raise api.InvalidArgument("tensor dtypes must match the plan's")
        b.check(b._lib.nnq_plan_add_reduced(self._handle, comm._handle, weight.handle(), x.data_ptr(),
                                            bias.data_ptr() if bias is not None else None, y.data_ptr()))
        self._keep.append((comm, weight, x, y, bias))

    def finalize(self):
        self.backend.check(self.backend._lib.nnq_plan_finalize(self._handle))
        return self

    def run(self, stream=None):
        self.backend.check(self.backend._lib.nnq_plan_run(self._handle, api._stream_ptr(stream)))

    def run_raw(self, stream_ptr) -> int:
        return self.backend._lib.nnq_plan_run(self._handle, stream_ptr)

    def reset(self, stream=None):
        self.backend.check(self.backend._lib.nnq_plan_reset(self._handle, api._stream_ptr(stream)))

    def set_spin_limit(self, polls: int):
        self.backend.check(self.backend._lib.nnq_plan_set_spin_limit(self._handle, int(polls)))

    def info(self) -> dict:
        g, c, s = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        sm, tb = ctypes.c_size_t(), ctypes.c_size_t()
        self.backend.check(self.backend._lib.nnq_plan_info(self._handle, ctypes.byref(g), ctypes.byref(c), ctypes.byref(s),
                                                           ctypes.byref(sm), ctypes.byref(tb)))
        return {"groups": g.value, "ctas": c.value, "stages": s.value, "smem_bytes": sm.value, "table_bytes": tb.value}

    def dependency(self, group: int) -> int:
        d = ctypes.c_int()
        self.backend.check(self.backend._lib.nnq_plan_dependency(self._handle, int(group), ctypes.byref(d)))
        return d.value

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_plan_destroy(self._handle)
            self._handle = None
            self._keep = []

    def __del__(self):  # pragma: no cover
        try:
            self.release()
        except Exception:
            pass


def _code(dtype) -> int:
    torch = api._torch()
    if dtype == torch.float32:
        return api.F32
    if dtype == torch.bfloat16:
        return api.BF16
    raise api.InvalidArgument(f"unsupported dtype {dtype}")


def geometry(row_tiles: int, k_tiles: int, ctas: int):
    """(largest tile count of any CTA, most CTAs a row tile is spread over): host arithmetic only."""
    from . import _lib
    lib = _lib.load()
    mt, pm = ctypes.c_int(), ctypes.c_int()
    st = lib.nnq_plan_geometry(row_tiles, k_tiles, ctas, ctypes.byref(mt), ctypes.byref(pm))
    if st != 0:
        raise api.InvalidArgument("bad plan geometry")
    return mt.value, pm.value
