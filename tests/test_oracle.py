"""The oracle against the golden vectors produced by the reference's own marlin.py
(tests/golden/make_golden.py).  Integer work must be bit-exact."""
import glob
import os

import numpy as np
import pytest

from oracle import oracle as orc

CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "g*.npz")))


def load(golden_dir, name):
    return dict(np.load(os.path.join(golden_dir, name + ".npz")))


def test_cases_present():
    assert len(CASES) == 4


def test_perm_tables(golden_dir):
    g = np.load(os.path.join(golden_dir, "perms.npz"))
    for perm, sp, sps in (orc.np_get_perms(), orc.c_get_perms()):
        assert np.array_equal(perm, g["perm"])
        assert np.array_equal(sp, g["scale_perm"])
        assert np.array_equal(sps, g["scale_perm_single"])


@pytest.mark.parametrize("name", CASES)
def test_quantize_matches_reference(golden_dir, name):
    g = load(golden_dir, name)
    gs = int(g["groupsize"])
    # Layer.pack re-quantises the fake-quantised weights (marlin.py:108-110) and must recover the codes
    for fn in (orc.np_quantize, orc.c_quantize):
        assert np.array_equal(fn(g["ref"], g["s"], gs), g["q"])


@pytest.mark.parametrize("name", CASES)
def test_pack_bit_exact(golden_dir, name):
    g = load(golden_dir, name)
    for fn in (orc.np_pack_weights, orc.c_pack_weights):
        assert np.array_equal(fn(g["q"]), g["B"])
    for fn in (orc.np_permute_scales, orc.c_permute_scales):
        assert np.array_equal(fn(g["s"]).view(np.uint16), g["s_packed"].view(np.uint16))


@pytest.mark.parametrize("name", CASES)
def test_unpack_roundtrip(golden_dir, name):
    g = load(golden_dir, name)
    k, n = int(g["k"]), int(g["n"])
    assert np.array_equal(orc.np_unpack_weights(g["B"], k, n), g["q"])
    assert np.array_equal(orc.c_unpack_weights(g["B"], k, n), g["q"])
    for fn in (orc.np_unpermute_scales, orc.c_unpermute_scales):
        assert np.array_equal(fn(g["s_packed"]).view(np.uint16), g["s"].view(np.uint16))


@pytest.mark.parametrize("name", CASES)
def test_dequant_bit_exact(golden_dir, name):
    g = load(golden_dir, name)
    gs = int(g["groupsize"])
    for fn in (orc.np_dequant, orc.c_dequant):
        assert np.array_equal(fn(g["q"], g["s"], gs).view(np.uint16), g["ref"].view(np.uint16))


@pytest.mark.parametrize("name", CASES)
def test_gemm_matches_reference_matmul(golden_dir, name):
    g = load(golden_dir, name)
    gs = int(g["groupsize"])
    want = g["C_ref32"]
    scale = np.max(np.abs(want))
    for C in (orc.np_gemm(g["A"], g["q"], g["s"], gs), orc.c_gemm(g["A"], g["q"], g["s"], gs),
              orc.c_gemm_packed(g["A"], g["B"], g["s_packed"], gs)):
        # fp32 accumulation in a different order: agree to fp32 rounding noise
        assert np.max(np.abs(C - want)) <= 1e-5 * scale
        # and the reference's own fp16 result is inside the acceptance band around the oracle
        ok, err, bound = orc.tolerance_ok(g["C_ref16"].astype(np.float32), C)
        assert ok, (err, bound)


BIG = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "big_*.npz")))


def big_operands(golden_dir, name):
    """A layer-sized golden case: operands regenerated from tests/golden/synth.py, the reference's scales and fp32
    product from the fixture, its other results as SHA-256 digests."""
    import hashlib
    import sys
    sys.path.insert(0, golden_dir)
    from synth import synth_fp16
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    m, n, k, seed = int(g["m"]), int(g["n"]), int(g["k"]), int(g["seed"])
    sha = lambda x: hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest()
    return g, synth_fp16(m, k, seed + 1000), synth_fp16(k, n, seed), sha


def test_big_cases_present():
    assert len(BIG) == 2


@pytest.mark.parametrize("name", BIG)
def test_big_case_every_stage_matches_reference(golden_dir, name):
    """2048 x 4096 g128 and 1024 x 2048 per-channel through every step of the reference's pipeline
    (marlin_test.py:18-55, marlin.py:92-131): codes, fake-quantised weights, packed words, permuted scales bit-exact
    (by digest), the product to fp32 rounding noise."""
    g, A, w, sha = big_operands(golden_dir, name)
    gs = int(g["groupsize"])
    s = g["s"]
    for quant, deq, pack, perm in ((orc.np_quantize, orc.np_dequant, orc.np_pack_weights, orc.np_permute_scales),
                                   (orc.c_quantize, orc.c_dequant, orc.c_pack_weights, orc.c_permute_scales)):
        q = quant(w, s, gs)
        assert sha(q) == str(g["sha_q"])
        assert sha(deq(q, s, gs)) == str(g["sha_ref"])
        assert sha(pack(q)) == str(g["sha_B"])
        assert sha(perm(s)) == str(g["sha_s_packed"])
    want = g["C_ref32"]
    q = orc.c_quantize(w, s, gs)
    for C in (orc.c_gemm(A, q, s, gs), orc.c_gemm_packed(A, orc.c_pack_weights(q), orc.c_permute_scales(s), gs)):
        assert np.max(np.abs(C - want)) <= 1e-5 * np.max(np.abs(want))


def test_gemm_edge_shapes():
    # empty problems return zeros without touching memory (marlin_cute_kernel.cu:59-60)
    A, q, s = orc.make_problem(0, 256, 128, 128, 0)
    assert orc.c_gemm(A, q, s, 128).shape == (0, 256)
    # ragged m, one group, per-channel
    for (m, n, k, gs) in [(1, 256, 128, 128), (3, 320, 64, -1), (17, 64, 256, 128)]:
        A, q, s = orc.make_problem(m, n, k, gs, 7)
        want = orc.np_gemm(A, q, s, gs)
        got = orc.c_gemm(A, q, s, gs)
        assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))


def test_closed_form_layout_random():
    rng = np.random.default_rng(5)
    q = rng.integers(0, 16, size=(64, 192), dtype=np.uint8)
    B = orc.c_pack_weights(q)
    assert np.array_equal(orc.np_unpack_weights(B, 64, 192), q)
