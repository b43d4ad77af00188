"""The C-ABI library loads and exports every symbol include/w4a16.h declares (no compute without a GPU),
and the host-side argument checks of the launcher follow the reference's error contract."""
import ctypes
import os
import re

import pytest

import __graft_entry__ as entry

pkg = entry.load_package()
from awesome_cute_b200 import _lib  # noqa: E402


def declared_symbols():
    text = open(os.path.join(entry.ROOT, "include", "w4a16.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(w4a16_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 11
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(raw, name), name
        assert name in _lib.SYMBOLS, "header symbol %s has no ctypes binding" % name
    assert sorted(_lib.SYMBOLS) == names


def test_cpp_launcher_symbol_present():
    # the C++-linkage twin with the reference's name (marlin_cute_kernel.cu:28-31), mangled
    out = os.popen("nm -D --defined-only '%s'" % _lib.LIB_PATH).read()
    assert re.search(r"\b_Z11marlin_cutePKvS0_PvS1_iiiS1_iiP11CUstream_stiiii\b", out), out[-2000:]


def test_workspace_rule():
    L = _lib.lib
    assert L.w4a16_workspace_ints(4096, 16) == 4096 // 128 * 16   # marlin.py:85
    assert L.w4a16_workspace_ints(256, 8) == 16
    assert L.w4a16_workspace_ints(0, 16) == 0


def _gemm(m, n, k, gs, tk=-1, tn=-1, ptr=0x1000):
    p = ctypes.c_void_p(ptr)
    return _lib.lib.w4a16_marlin_gemm(p, p, p, p, m, n, k, p, gs, 0, None, tk, tn, -1, 16)


def test_error_codes_follow_the_reference_without_touching_the_device():
    # marlin_test.py:96-121 (test_errors): k = 64 with tiles (128,128) and (256,256) must fail
    assert _gemm(16, 256, 64, -1, 128, 128) == _lib.ERR_PROB_SHAPE
    assert _gemm(16, 256, 64, -1, 256, 256) == _lib.ERR_PROB_SHAPE
    assert _gemm(16, 256, 64, 32, 256, 256) == _lib.ERR_PROB_SHAPE      # the 2-row scale case: groupsize 32
    # automatic tiles: m <= 16 -> (128,128); larger -> (64,256)  (marlin_cute_kernel.cu:39-49)
    assert _gemm(16, 256, 64, -1) == _lib.ERR_PROB_SHAPE                 # k % 128
    assert _gemm(17, 128, 64, -1) == _lib.ERR_PROB_SHAPE                 # n % 256
    # divisible shape but no such kernel instance (marlin_cute_kernel.cu:95-107)
    assert _gemm(16, 256, 256, -1, 256, 256) == _lib.ERR_KERN_SHAPE
    assert _gemm(32, 256, 256, -1, 128, 128) == _lib.ERR_KERN_SHAPE      # (128,128) exists for one m-block only
    assert _gemm(16, 256, 256, 64) == _lib.ERR_KERN_SHAPE                # group size 64
    # the shape check comes before the empty-problem early return (marlin_cute_kernel.cu:56-60)
    assert _gemm(0, 256, 64, -1) == _lib.ERR_PROB_SHAPE
    assert _gemm(0, 256, 128, -1) == _lib.OK
    assert _gemm(16, 0, 128, -1) == _lib.OK
    assert _gemm(16, 256, 0, -1) == _lib.OK
    # new failure kind: misaligned / null operands never alias the reference's codes
    assert _gemm(16, 256, 128, -1, ptr=0x1008) == _lib.ERR_ARG
    assert _gemm(16, 256, 128, -1, ptr=0) == _lib.ERR_ARG


def test_python_mul_raises_like_the_binding():
    import torch
    A = torch.zeros((16, 64), dtype=torch.half)
    C = torch.zeros((16, 256), dtype=torch.half)
    B = torch.zeros((4, 512), dtype=torch.int)
    s = torch.zeros((3, 256), dtype=torch.half)
    with pytest.raises(RuntimeError, match="not compatible with 3 groups"):   # marlin_gemm.cpp:27-28
        pkg.mul(A, B, C, s, torch.zeros(32, dtype=torch.int))
    s = torch.zeros((1, 256), dtype=torch.half)
    with pytest.raises(RuntimeError, match="workspace must be of size at least 32"):  # marlin_gemm.cpp:29-31
        pkg.mul(A, B, C, s, torch.zeros(8, dtype=torch.int))
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        pkg.mul(A, B, C, s, torch.zeros(32, dtype=torch.int))


def test_layer_constructor_contract():
    with pytest.raises(ValueError):
        pkg.Layer(256, 256, groupsize=64)       # marlin.py:70-71
    with pytest.raises(ValueError):
        pkg.Layer(192, 256)                     # marlin.py:72-73
    with pytest.raises(ValueError):
        pkg.Layer(256, 128)
    layer = pkg.Layer(256, 512, groupsize=128)
    assert tuple(layer.B.shape) == (16, 1024) and tuple(layer.s.shape) == (2, 512)
    assert layer.workspace.numel() == 512 // 128 * 16
