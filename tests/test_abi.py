"""The C-ABI library builds, loads and exports every symbol include/nnq.h declares.
No compute calls: runs without a GPU."""
import ctypes
import os
import re

import pytest

from nn_b200 import _lib, build
from nn_b200.formats import GEOMETRY, QuantFormat

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nnq.h")).read()
    return sorted(set(re.findall(r"^NNQ_API [^;(]*?\b(nnq_\w+)\(", text, re.M)))


def test_library_builds_for_sm100a():
    path = build.build()
    assert os.path.exists(path)
    assert "compute_100a" in " ".join(build.NVCC_FLAGS)


def test_every_declared_symbol_is_exported_and_typed():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/nnq.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in names, f"{name} bound in python but not declared in include/nnq.h"


def test_geometry_matches_reference_tables():
    lib = _lib.load()
    for fmt, g in GEOMETRY.items():
        e, b, s = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        assert lib.nnq_format_geometry(int(fmt), ctypes.byref(e), ctypes.byref(b), ctypes.byref(s)) == 0
        assert (e.value, b.value, s.value) == (g.elems, g.bytes, g.scale_bytes)
    # crates/nn-gguf/src/dequant.rs:84-114 and crates/nn-core/src/layers/quantized/mxfp4.rs:42-48
    assert (GEOMETRY[QuantFormat.Q8_0].elems, GEOMETRY[QuantFormat.Q8_0].bytes) == (32, 34)
    assert (GEOMETRY[QuantFormat.Q4_K].elems, GEOMETRY[QuantFormat.Q4_K].bytes) == (256, 144)
    assert (GEOMETRY[QuantFormat.Q6_K].elems, GEOMETRY[QuantFormat.Q6_K].bytes) == (256, 210)
    assert (GEOMETRY[QuantFormat.MXFP4_CORE].elems, GEOMETRY[QuantFormat.MXFP4_CORE].bytes) == (32, 17)
    assert lib.nnq_format_geometry(99, None, None, None) != 0


def test_status_strings_and_version():
    lib = _lib.load()
    assert lib.nnq_version() >= 1
    assert lib.nnq_status_str(0) == b"ok"
    for code in (1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 20, 21, 22, 23, 24):
        assert lib.nnq_status_str(code) not in (b"", b"unknown status")


def test_init_without_device_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _lib.load()
    ctx = ctypes.c_void_p()
    assert lib.nnq_init(0, ctypes.byref(ctx)) == 23  # NNQ_ERR_NO_DEVICE
    assert not ctx.value
    from nn_b200 import api
    with pytest.raises(api.BackendFailure):
        api.Backend(0)
