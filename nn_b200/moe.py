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

    def forward_routed(self, rows, experts, weights, slots: int = 1):
        """The expert MLPs over rows whose routing the caller supplies: experts / weights are
        [n, slots] (int32 global expert indices / f32); rows routed to experts this block does not
        hold contribute nothing. Returns f32 [n, hidden]."""
        import torch
        b = self.backend
        rows = rows.contiguous()
        n = rows.shape[0]
        y = torch.empty((n, self.hidden), dtype=torch.float32, device=rows.device)
        if n:
            b.check(b._lib.nnq_moe_forward_routed(b._ctx, self._handle, rows.data_ptr(), api._dtype_code(rows), n, slots,
                                                  experts.contiguous().data_ptr(), weights.contiguous().data_ptr(), y.data_ptr(),
                                                  api._stream_ptr(None)))
        return y

    def release(self):
        if self._handle is not None:
            self.backend._lib.nnq_moe_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.release()
        except Exception:
            pass


# --------------------------------------------------------------------------- #
# expert parallelism with token dispatch (all-to-all)
# --------------------------------------------------------------------------- #

def dispatch_plan(idx, n_experts: int, world: int):
    """Index arithmetic of the token dispatch, on whatever device `idx` lives ([T, k] expert
    indices of the local tokens; torch tensor). Experts are split evenly over the ranks, rank r
    holding experts [r * E / world, (r + 1) * E / world). Returns
      order        [T*k] int64: the assignments (flat index t * k + slot) sorted by expert, ties in
                   flat order (stable) -- hence sorted by destination rank too;
      send_experts [T*k] int32: the expert of each sorted assignment;
      src_token    [T*k] int32: the token whose activations that assignment sends;
      send_counts  [world] int64: assignments per destination rank;
      pos          [T, k] int32: where (t, slot) sits in the sorted order (the row that comes back).
    """
    import torch
    t, k = idx.shape
    per_rank = n_experts // world
    flat = idx.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    send_experts = flat[order]
    send_counts = torch.bincount(send_experts // per_rank, minlength=world)
    pos = torch.empty(t * k, dtype=torch.int64, device=idx.device)
    pos[order] = torch.arange(t * k, dtype=torch.int64, device=idx.device)
    return (order, send_experts.to(torch.int32), (order // k).to(torch.int32), send_counts,
            pos.reshape(t, k).to(torch.int32))


def gather_rows(backend, x, index):
    """out[i, :] = x[index[i], :] (library kernel; index int32 on the device)."""
    import torch
    x = x.contiguous()
    out = torch.empty((index.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    if index.shape[0]:
        backend.check(backend._lib.nnq_moe_gather_rows(backend._ctx, x.data_ptr(), api._dtype_code(x), index.contiguous().data_ptr(),
                                                       index.shape[0], x.shape[1], out.data_ptr(), api._stream_ptr(None)))
    return out


def combine_rows(backend, rows, idx, wt, pos):
    """y[t, :] = sum over the slots of token t, in expert-index order, of wt[t, s] * rows[pos[t, s], :]."""
    import torch
    t, k = idx.shape
    y = torch.empty((t, rows.shape[1]), dtype=torch.float32, device=rows.device)
    if t:
        backend.check(backend._lib.nnq_moe_combine_rows(backend._ctx, rows.contiguous().data_ptr(), idx.contiguous().data_ptr(),
                                                        wt.contiguous().data_ptr(), pos.contiguous().data_ptr(), t, rows.shape[1], k,
                                                        y.data_ptr(), api._stream_ptr(None)))
    return y


class ExpertParallelMoe:
    """One MoE block over `world` ranks: every rank holds its own tokens and E / world experts
    (``shard`` built with ``expert_range=(rank * E / world, E / world)``, router replicated).
    forward: route locally -> sort the assignments by expert and gather their rows (library
    kernel) -> all-to-all (NCCL) -> the owners run their experts over the received rows (library
    kernels, routing supplied) -> all-to-all back -> weighted sum per token in expert-index order
    (library kernel). Same result as the single-device block on the concatenated tokens
    (crates/nn-gptoss/src/quantized_model.rs:132-194)."""

    def __init__(self, shard: MoeBlock, rank: int, world: int, group=None):
        if shard.n_experts % world:
            raise api.InvalidShape(f"{shard.n_experts} experts do not split evenly over {world} ranks")
        self.shard, self.rank, self.world, self.group = shard, rank, world, group

    def _exchange(self, rows, send_counts, recv_counts):
        import torch
        import torch.distributed as dist
        out = torch.empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(out, rows.contiguous(), list(recv_counts), list(send_counts), group=self.group)
        return out

    def forward(self, x):
        import torch
        import torch.distributed as dist
        s, b = self.shard, self.shard.backend
        if x.shape[-1] != s.hidden:
            raise api.ShapeMismatch(f"input last dim {x.shape[-1]} != hidden {s.hidden}")
        xs = x.contiguous().reshape(-1, s.hidden)
        t, k = xs.shape[0], s.top_k
        dev = xs.device
        idx, wt = s.route(xs)
        order, send_experts, src_token, send_counts, pos = dispatch_plan(idx, s.n_experts, self.world)
        # how many rows every rank sends to every other one (host-visible: the split sizes)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.cpu().tolist(), recv_counts.cpu().tolist()
        send_rows = gather_rows(b, xs, src_token)
        recv_rows = self._exchange(send_rows, sc, rc)
        recv_experts = self._exchange(send_experts, sc, rc)
        ones = torch.ones(recv_rows.shape[0], dtype=torch.float32, device=dev)
        out_rows = s.forward_routed(recv_rows, recv_experts, ones, 1)
        back = self._exchange(out_rows, rc, sc)          # rows return in this rank's sorted send order
        y = combine_rows(b, back, idx, wt, pos)
        return y.reshape(tuple(x.shape[:-1]) + (s.hidden,))

    __call__ = forward
