"""GPU parity on exactly the shapes the benchmark times: the prefill configs (M in {1024, 4096} on the four
Llama-2-7B linears) and the Llama-2-70B layers with their column-shard widths for 1/2/4/8 GPUs at M in {16, 4096}.

The reference's own list of model shapes is gemm/marlin_gemm/marlin_test.py:133-167 (it runs them at batch 1 and 16
and only prints a loss).  Here the CUDA path runs the full problem through the C ABI and the CPU oracle checks
column windows x a row subset (the oracle needs seconds for a window, hours for 4096 x 57344 x 8192), with the
tolerance of tests/gpu_common.py: max|C - C_ref| <= 1e-2 max|C_ref| and relative-mean error < 0.005.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from gpu_common import DEV, check, orc, pkg, run_mul, to_dev

GS = 128


def _rows(m):
    """Row subset: the first rows, the rows around the 128- and 192-row tile edges, the last rows (<= 64 rows)."""
    if m <= 64:
        return np.arange(m)
    picks = list(range(0, 8)) + list(range(124, 132)) + list(range(188, 196)) + list(range(m // 2, m // 2 + 8))
    picks += list(range(m - 24, m))
    return np.array(sorted(set(r for r in picks if 0 <= r < m)))


def _windows(n_local, width=256):
    """First, middle and last column window of a shard."""
    mid = (n_local // 2) // width * width
    return sorted(set([0, mid, n_local - width]))


def _check_windows(C, A, q, s, col0, n_local, what):
    rows = _rows(A.shape[0])
    A_sub = np.ascontiguousarray(A[rows])
    rows_t = torch.from_numpy(rows).to(C.device)
    for w0 in _windows(n_local):
        g0 = col0 + w0     # the window in the whole layer's column numbering
        ref = orc.c_gemm(A_sub, np.ascontiguousarray(q[:, g0:g0 + 256]), np.ascontiguousarray(s[:, g0:g0 + 256]), GS)
        check(C[rows_t][:, w0:w0 + 256], ref, "%s window %d" % (what, w0))


@pytest.mark.parametrize("n,k", [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)])
def test_prefill_llama7b_shapes(n, k):
    """M in {1024, 4096} on the four 7B shapes: the shapes of the prefill figures (192-row tiles on CTA pairs,
    whole-tile waves, ragged last batch tile)."""
    A, q, s = orc.make_problem(4096, n, k, GS, seed=n + k)
    Bt, st = to_dev(pkg.pack_weights(q)), to_dev(pkg.permute_scales(s))
    for m in (4096, 1024):
        Am = np.ascontiguousarray(A[:m])
        C = run_mul(to_dev(Am), Bt, st, m, n)
        _check_windows(C, Am, q, s, 0, n, "m=%d n=%d k=%d" % (m, n, k))
        del C


@pytest.mark.parametrize("n_full,k", [(57344, 8192), (8192, 28672)])
def test_llama70b_layers_and_their_shards(n_full, k):
    """The 70B gate-up (57344 x 8192) and down (8192 x 28672) layers whole and cut for 2, 4 and 8 GPUs with
    w4a16_shard_columns, at M = 16 and M = 4096.  The whole gate-up layer at M = 4096 is the case where the launcher
    switches the tile order of the whole-tile waves to batch-first by itself."""
    A, q, s = orc.make_problem(4096, n_full, k, GS, seed=n_full)
    B_full, s_full = pkg.pack_weights(q), pkg.permute_scales(s)
    A16 = np.ascontiguousarray(A[:16])
    At4096, At16 = to_dev(A), to_dev(A16)
    for world in (1, 2, 4, 8):
        rank = world - 1 if world > 1 else 0      # the last shard: its columns end at the layer's edge
        n_local = n_full // world
        if world == 1:
            B_r, s_r = B_full, s_full
        else:
            B_r, s_r = pkg.shard_columns(B_full, s_full, rank, world)
        Bt, st = to_dev(B_r), to_dev(s_r)
        for m, At, Am in ((16, At16, A16), (4096, At4096, A)):
            C = run_mul(At, Bt, st, m, n_local)
            _check_windows(C, Am, q, s, rank * n_local, n_local, "world=%d m=%d n_local=%d k=%d" % (world, m, n_local, k))
            del C
        del Bt, st
        torch.cuda.empty_cache()


@pytest.mark.parametrize("m,n,k,what", [
    (128, 1024, 4096, "4 pair tiles cut 2 ways: 8 pairs, each inside one tile"),
    (128, 2048, 8192, "8 pair tiles cut 4 ways"),
    (96, 4096, 4096, "16 pair tiles of one ragged batch tile"),
    (128, 512, 4096, "two pair tiles cut 2 ways"),
    (128, 4096, 512, "too few stages per pair: single-CTA kernel, 32 tiles of 4 stages, one each"),
    (256, 4096, 4096, "two batch tiles of 128 rows, 64 pairs"),
    (576, 12288, 4096, "144 tiles = 2 whole waves on 72 of the 74 pairs, no stream-K part"),
    (200, 4096, 11008, "stage count without a usable divisor: the even cut"),
])
def test_worker_counts_of_few_wide_tiles(m, n, k, what):
    """Batches of 65+ rows on layers with fewer tiles than workers: the launcher prices the even cut against cuts that
    line up with the tiles and takes a worker count of its own (fewer CTAs or CTA pairs than the device has).  Each of
    these takes a different branch of that choice; the 1024-row cases are in test_prefill_llama7b_shapes."""
    A, q, s = orc.make_problem(m, n, k, GS, seed=m + n + k)
    Bt, st = to_dev(pkg.pack_weights(q)), to_dev(pkg.permute_scales(s))
    C = run_mul(to_dev(A), Bt, st, m, n)
    rows = _rows(m)
    A_sub = np.ascontiguousarray(A[rows])
    rows_t = torch.from_numpy(rows).to(C.device)
    for w0 in _windows(n):
        ref = orc.c_gemm(A_sub, np.ascontiguousarray(q[:, w0:w0 + 256]), np.ascontiguousarray(s[:, w0:w0 + 256]), GS)
        check(C[rows_t][:, w0:w0 + 256], ref, "%s (m=%d n=%d k=%d) window %d" % (what, m, n, k, w0))
