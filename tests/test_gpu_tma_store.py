"""The TMA-store epilogue (finished tiles staged in shared memory and written by cp.async.bulk.tensor stores through
a tensor map over C, rows past m clipped by the map) in all three kernels, against the CPU oracle.  The reference
stages its output tile through shared memory too (gemm/marlin_gemm/marlin_cute_trait.h:754-799).

Which epilogue the plain GEMM uses is read from W4A16_TMA_STORE once at load time, so both settings run in child
processes: whichever is not the default is covered here, and the two must agree bit for bit (same accumulation,
same conversion, only the way to memory differs)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CODE = r"""
import sys, os, hashlib
sys.path.insert(0, os.getcwd()); sys.path.insert(0, os.path.join(os.getcwd(), 'tests'))
import numpy as np, torch
from gpu_common import orc, pkg, pack_problem, run_mul, check
cases = [
    # decode kernel: ragged rows, stream-K and cluster forms, both scale kinds
    (3, 512, 1024, 128, -1), (16, 512, 2048, -1, -1), (1, 4096, 4096, 128, -1), (12, 4096, 2048, -1, -1), (16, 12288, 1024, 128, -1),
    (16, 512, 2048, 128, 7),
    # general kernel: 17..64 rows with an explicit split, 128- and 192-row tiles, ragged, per-channel
    (24, 512, 1024, 128, 5), (64, 256, 2048, -1, 9), (118, 512, 1024, 128, -1), (118, 256, 512, -1, -1), (200, 512, 1024, 128, 11),
    # CTA pairs: 33..64 rows, and batches past 128 rows with a ragged last tile
    (48, 512, 4096, 128, -1), (577, 4096, 8192, 128, -1), (577, 1024, 8192, -1, -1),
]
digest = hashlib.sha256()
for (m, n, k, gs, sms) in cases:
    A, q, s = orc.make_problem(m, n, k, gs, seed=m + n + k)
    At, Bt, st = pack_problem(A, q, s)
    C = run_mul(At, Bt, st, m, n, sms=sms)
    if n * k <= 4096 * 4096:
        check(C, orc.c_gemm(A, q, s, gs), "m=%d n=%d k=%d g=%d sms=%d" % (m, n, k, gs, sms))
    else:
        for n0 in (0, n - 256):
            ref = orc.c_gemm(A, np.ascontiguousarray(q[:, n0:n0 + 256]), np.ascontiguousarray(s[:, n0:n0 + 256]), gs)
            check(C[:, n0:n0 + 256], ref, "m=%d n=%d k=%d window %d" % (m, n, k, n0))
    digest.update(C.cpu().numpy().tobytes())
print('digest', digest.hexdigest())
"""


def _run(setting):
    env = dict(os.environ, W4A16_TMA_STORE=setting)
    r = subprocess.run([sys.executable, "-c", CODE], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "digest" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout.strip().split()[-1]


def test_tma_store_and_register_store_epilogues_agree_with_the_oracle_and_with_each_other():
    with_tma = _run("1")
    without = _run("0")
    assert with_tma == without
