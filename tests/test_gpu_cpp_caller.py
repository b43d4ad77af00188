"""The C++-linkage launcher `marlin_cute`, called by a C++ program that carries the reference's own declaration
(gemm/marlin_gemm/marlin_gemm.cpp:6-9) and calls it as the reference's binding does (:36-39): once with the default
arguments, once with every argument and a cudaStream_t.  Output against the CPU oracle."""
import os
import subprocess

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu

EXE = os.path.join(entry.ROOT, "tests", "cpp", "marlin_cute_call")


@pytest.mark.parametrize("m,n,k,gs", [(16, 512, 1024, 128), (3, 256, 2048, -1), (200, 512, 1024, 128)])
def test_cpp_caller_with_defaults_and_with_stream(tmp_path, m, n, k, gs):
    from gpu_common import orc, pkg
    assert os.path.exists(EXE), "tests/cpp/marlin_cute_call is built by __graft_entry__.build()"
    A, q, s = orc.make_problem(m, n, k, gs, seed=m + n)
    B, sp = pkg.pack_weights(q), pkg.permute_scales(s)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        np.array([m, n, k, s.shape[0]], np.int32).tofile(f)
        A.tofile(f)
        B.tofile(f)
        sp.tofile(f)
    r = subprocess.run([EXE, str(fin), str(fout)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.returncode, r.stderr[-2000:])
    raw = np.fromfile(fout, np.uint8)
    rcs = raw[:8].view(np.int32)
    assert list(rcs) == [0, 0]
    C = raw[8:].view(np.float16).reshape(2, m, n).astype(np.float32)
    ref = orc.c_gemm(A, q, s, gs)
    for i in range(2):
        ok, err, bound = orc.tolerance_ok(C[i], ref)
        assert ok, "call %d: max|err| %.4g > %.4g" % (i + 1, err, bound)
    assert np.array_equal(C[0], C[1])     # same kernel, same split: the two calls agree bit for bit
