"""The allocation-free MoE entry point (nnq_moe_forward_static) against the regular one.

Some callers cannot let a library allocate on the device: a server whose memory pool owns the
whole GPU, or a decode loop that must never hit the device-wide synchronisation an allocation
brings. For them the library keeps a fixed scratch area in its own device image. This test calls
the entry point through the C ABI twice in a row (the area is shared and keeps the previous
call's contents) and checks both results against nnq_moe_forward on the same inputs, then checks
that an oversized call is refused. The file sorts last so that a failure here cannot hide
another test's result in a run that stops at the first failure; it sets up its own inputs and
also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api, moe
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3  # the bar the other product tests use; the two entry points should in fact agree exactly


def _block(E, H, I, k, seed):
    s = F.Stream(seed)
    rw = (s.normal(E * H) * 0.5).astype(np.float32).reshape(E, H)
    rb = (s.normal(E) * 0.1).astype(np.float32)
    bgu = (s.normal(E * 2 * I) * 0.1).astype(np.float32).reshape(E, 2 * I)
    bd = (s.normal(E * H) * 0.1).astype(np.float32).reshape(E, H)
    gu, gus = F.gen_weight(Q.MXFP4_GPTOSS, seed + 1, E * H, 2 * I)
    dn, dns = F.gen_weight(Q.MXFP4_GPTOSS, seed + 2, E * I, H)
    return moe.MoeBlock(E, H, I, k, 7.0, rw, rb, moe.LAYOUT_KN_GPTOSS, Q.MXFP4_GPTOSS, gu, gus, bgu, dn, dns, bd)


def _static_forward(blk, x):
    b = blk.backend
    y = torch.full(x.shape, float("nan"), dtype=torch.float32, device=x.device)
    st = b._lib.nnq_moe_forward_static(b._ctx, blk._handle, x.data_ptr(), api._dtype_code(x), x.shape[0],
                                       y.data_ptr(), api._stream_ptr(None))
    return st, y


def test_static_scratch_entry_point_matches_regular_one_twice():
    E, H, I, k = 8, 256, 256, 4
    blk = _block(E, H, I, k, 4242)
    for call, T in enumerate((16, 5)):      # second call: different size, stale contents in the area
        x = torch.from_numpy(F.gen_activations(900 + call, T, H, bf16=True)).to(DEV)
        want = blk(x)
        st, got = _static_forward(blk, x)
        assert st == 0, blk.backend._lib.nnq_last_error(blk.backend._ctx)
        torch.cuda.synchronize()
        blk.backend.device_status()
        assert torch.isfinite(got).all()
        err = float((got - want).abs().max() / want.abs().max())
        assert err <= TOL, err
    blk.release()


def test_static_scratch_rejects_oversized_call():
    E, H, I, k = 8, 256, 256, 4
    blk = _block(E, H, I, k, 77)
    T = 4096  # 16384 routed rows * (3*256 + 256) * 4 B = 64 MiB > 8 MiB
    x = torch.zeros(T, H, device=DEV)
    st, _ = _static_forward(blk, x)
    assert st == 10  # NNQ_ERR_UNSUPPORTED
    msg = blk.backend._lib.nnq_last_error(blk.backend._ctx).decode()
    assert "scratch" in msg and "8388608" in msg
    # the context is still usable
    st, y = _static_forward(blk, x[:2].contiguous())
    assert st == 0
    torch.cuda.synchronize()
    blk.release()
