"""Shared helpers of the GPU parity tests (the CUDA path is reached through the C ABI only)."""
import numpy as np
import torch

import __graft_entry__ as entry
from oracle import oracle as orc

pkg = entry.load_package()
DEV = torch.device("cuda:0")


def to_dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def pack_problem(A, q, s):
    """numpy operands -> (A, B, s_packed) on the device, packed by the shipped C++ packer."""
    return to_dev(A), to_dev(pkg.pack_weights(q)), to_dev(pkg.permute_scales(s))


def run_mul(At, Bt, st, m, n, thread_k=-1, thread_n=-1, sms=-1, fn=None, ws=None):
    C = torch.zeros((m, n), dtype=torch.half, device=DEV)
    if ws is None:
        ws = torch.zeros(max(n // 128 * 16, 1), dtype=torch.int, device=DEV)
    (fn or pkg.mul)(At, Bt, C, st, ws, thread_k, thread_n, sms)
    pkg.device_status(0)
    assert int(ws.abs().sum().item()) == 0, "workspace must be left all zero"
    return C


def check(C, C_ref, what=""):
    Cn = C.float().cpu().numpy()
    ok, err, bound = orc.tolerance_ok(Cn, C_ref)
    rel = float(np.mean(np.abs(Cn - C_ref)) / max(np.mean(np.abs(C_ref)), 1e-30))  # the reference's own metric, marlin_test.py:74
    assert ok, "%s max|err| %.4g > 1e-2*max|ref| = %.4g (rel-mean %.4g)" % (what, err, bound, rel)
    assert rel < 0.005, "%s rel-mean err %.4g" % (what, rel)     # the threshold of marlin_test.py:75
    return err, bound, rel


def run_problem(m, n, k, thread_k=-1, thread_n=-1, groupsize=-1, seed=0, sms=-1, fn=None):
    """marlin_test.py:59-76 with the oracle in place of torch.matmul and an assertion in place of a print."""
    A, q, s = orc.make_problem(m, n, k, groupsize, seed)
    At, Bt, st = pack_problem(A, q, s)
    C = run_mul(At, Bt, st, m, n, thread_k, thread_n, sms, fn)
    return check(C, orc.c_gemm(A, q, s, groupsize), "m=%d n=%d k=%d g=%d sms=%d" % (m, n, k, groupsize, sms))
