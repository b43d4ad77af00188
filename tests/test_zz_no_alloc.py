"""The allocation-free entry point w4a16_marlin_gemm_builtin_scratch, called through the C ABI.

Some callers cannot let this library call cudaMalloc: the framework they run in has reserved the whole
device, or they sit on a latency path where an allocation stalls every stream.  For them the library carries
its stream-K scratch as a device array compiled into the .so.  This test checks that the variant computes
what w4a16_marlin_gemm computes, on two calls in a row (the second call finds the array as the first one left
it), and that it refuses sizes beyond its fixed scratch with a clear message.

The file name sorts last on purpose: if this added entry point breaks, a run that stops at the first failure
has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from gpu_common import DEV, check, orc, pack_problem, pkg
    from awesome_cute_b200 import _lib


def _call(fn, At, Bt, st, C, ws, m, n, k, gs):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(0).cuda_stream)
    with torch.cuda.device(0):
        return fn(p(At), p(Bt), p(C), p(st), m, n, k, p(ws), gs, 0, stream, -1, -1, -1, 16)


@pytest.mark.parametrize("m,n,k,gs", [(16, 1024, 4096, 128), (48, 512, 2048, -1)])
def test_builtin_scratch_matches_allocating_entry_point_twice(m, n, k, gs):
    L = _lib.lib
    A, q, s = orc.make_problem(m, n, k, gs, seed=77)
    At, Bt, st = pack_problem(A, q, s)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)
    C_ref = torch.zeros((m, n), dtype=torch.half, device=DEV)
    assert _call(L.w4a16_marlin_gemm, At, Bt, st, C_ref, ws, m, n, k, gs) == _lib.OK
    pkg.device_status(0)
    want = orc.c_gemm(A, q, s, gs)
    check(C_ref, want, "allocating entry point")
    outs = []
    for call in range(2):   # the second call reuses the array exactly as the first left it
        C = torch.full((m, n), float("nan"), dtype=torch.half, device=DEV)
        rc = _call(L.w4a16_marlin_gemm_builtin_scratch, At, Bt, st, C, ws, m, n, k, gs)
        assert rc == _lib.OK, (rc, _lib.last_cuda_error())
        pkg.device_status(0)
        check(C, want, "built-in scratch, call %d" % call)                 # the tolerance every GPU test uses
        outs.append(C)
    assert torch.equal(outs[0], outs[1]), "the second call must find the array as the first call left it"
    if m <= 16:
        # up to 16 rows both entry points launch the same kernel with the same split: identical bits.  (Past 16 rows
        # the allocating entry point may take CTA pairs, which the built-in scratch is not sized for.)
        assert torch.equal(outs[0], C_ref)
    assert int(ws.abs().sum().item()) == 0


def test_builtin_scratch_rejects_sizes_beyond_its_array():
    L = _lib.lib
    m, n, k, gs = 65, 512, 256, 128      # one row more than the built-in scratch is sized for
    A, q, s = orc.make_problem(m, n, k, gs, seed=78)
    At, Bt, st = pack_problem(A, q, s)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)
    C = torch.zeros((m, n), dtype=torch.half, device=DEV)
    assert _call(L.w4a16_marlin_gemm_builtin_scratch, At, Bt, st, C, ws, m, n, k, gs) == _lib.ERR_ARG
    assert "exceeds the built-in scratch limit" in _lib.last_cuda_error()
    assert float(C.abs().sum()) == 0.0   # nothing was launched
    # the reference's shape errors keep their codes here too
    assert _call(L.w4a16_marlin_gemm_builtin_scratch, At, Bt, st, C, ws, 16, n, 64, -1) == _lib.ERR_PROB_SHAPE


def test_builtin_scratch_bounded_wait_runs_out_and_the_array_recovers():
    """The finisher of a split tile waits for a partial tile nobody writes: after the limit the kernel gives up,
    the status says so, the built-in array is put back into its idle state and the next call is correct."""
    import time
    L = _lib.lib
    m, n, k, gs = 16, 256, 2048, 128
    A, q, s = orc.make_problem(m, n, k, gs, seed=79)
    At, Bt, st = pack_problem(A, q, s)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)
    C = torch.zeros((m, n), dtype=torch.half, device=DEV)
    want = orc.c_gemm(A, q, s, gs)
    assert _call(L.w4a16_marlin_gemm_builtin_scratch, At, Bt, st, C, ws, m, n, k, gs) == _lib.OK   # set-up done
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    # a stream that never ran the allocating entry point, so that the status read is the built-in word's
    side = torch.cuda.Stream(device=DEV)
    stream = ctypes.c_void_p(side.cuda_stream)
    torch.cuda.synchronize()
    t0 = time.time()
    with torch.cuda.device(0):
        rc = L.w4a16_selftest_unanswered_wait(p(At), p(Bt), p(C), p(st), m, n, k, gs, 0, stream, -300)
    assert rc == _lib.OK, _lib.last_cuda_error()
    assert L.w4a16_device_status(0, stream) == _lib.ERR_TIMEOUT
    assert "built-in scratch" in _lib.last_cuda_error()
    assert 0.25 < time.time() - t0 < 3.0
    assert L.w4a16_device_status(0, stream) == _lib.OK
    C.zero_()
    with torch.cuda.stream(side), torch.cuda.device(0):
        rc = L.w4a16_marlin_gemm_builtin_scratch(p(At), p(Bt), p(C), p(st), m, n, k, p(ws), gs, 0, stream, -1, -1, -1, 16)
    assert rc == _lib.OK
    side.synchronize()
    check(C, want, "after the timeout")
