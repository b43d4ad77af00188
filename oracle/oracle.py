"""CPU oracle for the W4A16 Marlin GEMM path -- TEST INFRASTRUCTURE ONLY.

Two independent restatements of the reference algorithm live here:

* ``np_*`` functions: numpy, following the reference's Python line by line
  (gemm/marlin_gemm/marlin.py:29-57 ``_get_perms``; :92-131 ``Layer.pack``;
  gemm/marlin_gemm/marlin_test.py:22-31 dequantise; :64 matmul).
* ``c_*`` functions: ctypes doors onto ``liboracle.so`` (w4a16_oracle.c, plain C with OpenMP),
  which is what the large parity cases and the bench's CPU-baseline leg time.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s cpu_baseline / reference arm may
import this module.  The shipped library never does.

Parity pin: ``tests/golden/*.npz`` were produced by the reference's own ``marlin.py`` (imported on
CPU by ``tests/golden/make_golden.py``); ``tests/test_oracle.py`` holds both restatements to them.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


# ----------------------------------------------------------------------------- numpy restatement
def np_get_perms():
    """marlin.py:29-57."""
    perm = []
    for i in range(32):
        perm1 = []
        col = i // 4
        for block in (0, 1):
            for row in (2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1):
                perm1.append(16 * row + col + 8 * block)
        for j in range(4):
            perm.extend(p + 256 * j for p in perm1)
    perm = np.array(perm, dtype=np.int64)
    interleave = np.array([0, 2, 4, 6, 1, 3, 5, 7])
    perm = perm.reshape(-1, 8)[:, interleave].ravel()
    scale_perm = np.array([i + 8 * j for i in range(8) for j in range(8)])
    scale_perm_single = np.array([2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)])
    return perm, scale_perm, scale_perm_single


def np_pack_weights(q):
    """q: uint8 codes [k, n] -> int32 [k/16, 2n]  (marlin.py:119-129)."""
    k, n = q.shape
    perm, _, _ = np_get_perms()
    w = q.astype(np.uint32).reshape(k // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(k // 16, n * 16)
    res = w.reshape(-1, perm.size)[:, perm].reshape(w.shape)
    out = np.zeros((res.shape[0], res.shape[1] // 8), dtype=np.uint32)
    for i in range(8):
        out |= res[:, i::8] << np.uint32(4 * i)
    return out.view(np.int32)


def np_unpack_weights(B, k, n):
    """Inverse of np_pack_weights through the closed form of the layout:
    word B[r][c], c = 128*blk + 4*lane + j, nibble i holds W[kk][nn] with
    nn = 64*blk + 16*j + lane//4 + 8*((i>>1)&1),  kk = 16*r + 2*(lane%4) + (i>>2) + 8*(i&1)."""
    Bu = B.view(np.uint32).reshape(k // 16, 2 * n)
    q = np.zeros((k, n), dtype=np.uint8)
    r, c = np.meshgrid(np.arange(k // 16), np.arange(2 * n), indexing="ij")
    blk, lane, j = c // 128, (c % 128) // 4, c % 4
    for i in range(8):
        nn = 64 * blk + 16 * j + lane // 4 + 8 * ((i >> 1) & 1)
        kk = 16 * r + 2 * (lane % 4) + (i >> 2) + 8 * (i & 1)
        q[kk, nn] = (Bu >> np.uint32(4 * i)) & np.uint32(0xF)
    return q


def np_permute_scales(s):
    """s: fp16 [groups, n] natural order -> packed order (marlin.py:111-118)."""
    _, sp, sps = np_get_perms()
    groups, n = s.shape
    p = sp if groups > 1 else sps
    return np.ascontiguousarray(s.reshape(-1, p.size)[:, p].reshape(groups, n))


def np_unpermute_scales(s_packed):
    _, sp, sps = np_get_perms()
    groups, n = s_packed.shape
    p = sp if groups > 1 else sps
    out = np.empty_like(s_packed).reshape(-1, p.size)
    out[:, p] = s_packed.reshape(-1, p.size)
    return out.reshape(groups, n)


def np_quantize(w, s, groupsize):
    """w fp16 [k, n], s fp16 [groups, n] -> codes (marlin.py:108-110: round(w/s)+8, clamp 0..15)."""
    k, n = w.shape
    g = k if groupsize == -1 else groupsize
    sfull = np.repeat(s, g, axis=0)
    quo = (w.astype(np.float16) / sfull.astype(np.float16)).astype(np.float16)
    return np.clip(np.rint(quo.astype(np.float32)).astype(np.int32) + 8, 0, 15).astype(np.uint8)


def np_dequant(q, s, groupsize):
    """marlin_test.py:31: ref = (w - 8).half() * s, the product rounded to fp16."""
    k, n = q.shape
    g = k if groupsize == -1 else groupsize
    sfull = np.repeat(s.astype(np.float16), g, axis=0)
    return ((q.astype(np.int32) - 8).astype(np.float16) * sfull).astype(np.float16)


def np_gemm(A, q, s, groupsize):
    """marlin_test.py:64 with fp32 accumulation: C = A_fp32 @ ref_fp32."""
    return A.astype(np.float32) @ np_dequant(q, s, groupsize).astype(np.float32)


# ----------------------------------------------------------------------------- C restatement
def build(force=False):
    """Compile liboracle.so."""
    so = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(_HERE, "w4a16_oracle.c")):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        L.oracle_pack_weights.argtypes = [vp, ci, ci, vp]
        L.oracle_unpack_weights.argtypes = [vp, ci, ci, vp]
        L.oracle_permute_scales.argtypes = [vp, ci, ci, vp]
        L.oracle_unpermute_scales.argtypes = [vp, ci, ci, vp]
        L.oracle_quantize.argtypes = [vp, vp, ci, ci, ci, vp]
        L.oracle_dequant.argtypes = [vp, vp, ci, ci, ci, vp]
        L.oracle_gemm.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp]
        L.oracle_gemm_packed.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp]
        L.oracle_get_perms.argtypes = [vp, vp, vp]
        _LIB = L
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


def c_get_perms():
    perm = np.zeros(1024, np.int32)
    sp = np.zeros(64, np.int32)
    sps = np.zeros(32, np.int32)
    lib().oracle_get_perms(_p(perm), _p(sp), _p(sps))
    return perm, sp, sps


def c_pack_weights(q):
    q = _c(q, np.uint8)
    k, n = q.shape
    B = np.empty((k // 16, 2 * n), np.int32)
    rc = lib().oracle_pack_weights(_p(q), k, n, _p(B))
    assert rc == 0, rc
    return B


def c_unpack_weights(B, k, n):
    B = _c(B, np.int32)
    q = np.empty((k, n), np.uint8)
    rc = lib().oracle_unpack_weights(_p(B), k, n, _p(q))
    assert rc == 0, rc
    return q


def c_permute_scales(s):
    s = _c(s.view(np.uint16), np.uint16)
    out = np.empty_like(s)
    rc = lib().oracle_permute_scales(_p(s), s.shape[0], s.shape[1], _p(out))
    assert rc == 0, rc
    return out.view(np.float16)


def c_unpermute_scales(sp):
    sp = _c(sp.view(np.uint16), np.uint16)
    out = np.empty_like(sp)
    rc = lib().oracle_unpermute_scales(_p(sp), sp.shape[0], sp.shape[1], _p(out))
    assert rc == 0, rc
    return out.view(np.float16)


def c_quantize(w, s, groupsize):
    w = _c(w.view(np.uint16), np.uint16)
    s = _c(s.view(np.uint16), np.uint16)
    k, n = w.shape
    q = np.empty((k, n), np.uint8)
    rc = lib().oracle_quantize(_p(w), _p(s), k, n, groupsize, _p(q))
    assert rc == 0, rc
    return q


def c_dequant(q, s, groupsize):
    q = _c(q, np.uint8)
    s = _c(s.view(np.uint16), np.uint16)
    k, n = q.shape
    ref = np.empty((k, n), np.uint16)
    rc = lib().oracle_dequant(_p(q), _p(s), k, n, groupsize, _p(ref))
    assert rc == 0, rc
    return ref.view(np.float16)


def c_gemm(A, q, s, groupsize):
    """A fp16 [m,k], q uint8 [k,n], s fp16 [groups,n] natural order -> C fp32 [m,n]."""
    A = _c(A.view(np.uint16), np.uint16)
    q = _c(q, np.uint8)
    s = _c(s.view(np.uint16), np.uint16)
    m, k = A.shape
    n = q.shape[1]
    C = np.zeros((m, n), np.float32)
    rc = lib().oracle_gemm(_p(A), _p(q), _p(s), m, n, k, groupsize, _p(C))
    assert rc == 0, rc
    return C


def c_gemm_packed(A, B, s_packed, groupsize):
    """Same GEMM from the operands the kernel receives (Marlin-packed B, permuted s)."""
    A = _c(A.view(np.uint16), np.uint16)
    B = _c(B, np.int32)
    s_packed = _c(s_packed.view(np.uint16), np.uint16)
    m, k = A.shape
    n = B.shape[1] // 2
    C = np.zeros((m, n), np.float32)
    rc = lib().oracle_gemm_packed(_p(A), _p(B), _p(s_packed), m, n, k, groupsize, _p(C))
    assert rc == 0, rc
    return C


def num_threads():
    return int(lib().oracle_num_threads())


def use_all_cores():
    """Run the C loops on every core this process may use, whatever OMP_NUM_THREADS the launcher exported."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().oracle_set_num_threads(ctypes.c_int(n))
    return num_threads()


# ----------------------------------------------------------------------------- seeded inputs
def make_problem(m, n, k, groupsize, seed):
    """Synthetic operands with the distributions the benchmark configs name:
    A ~ N(0,1) fp16; codes uniform on 0..15 (zero-point 8); scales uniform in [0.005, 0.02] fp16."""
    rng = np.random.default_rng(seed)
    g = k if groupsize == -1 else groupsize
    A = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    s = rng.uniform(0.005, 0.02, size=(k // g, n)).astype(np.float16)
    return A, q, s


def tolerance_ok(C, C_ref):
    """The acceptance rule: max |C - C_ref| <= 1e-2 * max |C_ref| (fp32 compare)."""
    C = np.asarray(C, np.float32)
    C_ref = np.asarray(C_ref, np.float32)
    if C_ref.size == 0:
        return True, 0.0, 0.0
    err = float(np.max(np.abs(C - C_ref)))
    bound = 1e-2 * float(np.max(np.abs(C_ref)))
    return err <= bound, err, bound
