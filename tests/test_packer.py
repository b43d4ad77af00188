"""The shipped C++ packer (closed-form layout) against the golden vectors of the reference packer and
against the oracle's table-driven restatement.  Bit-exact."""
import glob
import os

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import oracle as orc

pkg = entry.load_package()
CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "g*.npz")))


@pytest.mark.parametrize("name", CASES)
def test_pack_matches_reference_golden(golden_dir, name):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    k, n = int(g["k"]), int(g["n"])
    assert np.array_equal(pkg.pack_weights(g["q"]), g["B"])
    assert np.array_equal(pkg.unpack_weights(g["B"], k, n), g["q"])
    assert np.array_equal(pkg.permute_scales(g["s"]).view(np.uint16), g["s_packed"].view(np.uint16))
    assert np.array_equal(pkg.unpermute_scales(g["s_packed"]).view(np.uint16), g["s"].view(np.uint16))


@pytest.mark.parametrize("name", CASES)
def test_quantize_pack_is_layer_pack(golden_dir, name):
    """Layer.pack end to end: fake-quantised weights + scales -> the reference's B and s."""
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    k, n, gs = int(g["k"]), int(g["n"]), int(g["groupsize"])
    if k % 128 or n % 256:
        pytest.skip("Layer's public constructor rejects this shape (marlin.py:72-73)")
    if gs == k:
        gs = -1
    B, sp = pkg.quantize_pack(np.ascontiguousarray(g["ref"].T), g["s"], gs)
    assert np.array_equal(B, g["B"])
    assert np.array_equal(sp.view(np.uint16), g["s_packed"].view(np.uint16))


@pytest.mark.parametrize("name", ["big_g128_m16_n2048_k4096", "big_gm1_m16_n1024_k2048"])
def test_big_case_shipped_packer_matches_reference(golden_dir, name):
    """The layer-sized golden cases through the shipped packer: the reference's packed words and permuted scales by
    digest, from the fake-quantised weights as Layer.pack gets them and from the codes."""
    from test_oracle import big_operands
    g, _, w, sha = big_operands(golden_dir, name)
    gs, s = int(g["groupsize"]), g["s"]
    q = orc.c_quantize(w, s, gs)
    assert sha(pkg.pack_weights(q)) == str(g["sha_B"])
    assert sha(pkg.permute_scales(s)) == str(g["sha_s_packed"])
    B, sp = pkg.quantize_pack(np.ascontiguousarray(orc.c_dequant(q, s, gs).T), s, gs)
    assert sha(B) == str(g["sha_B"])
    assert sha(sp) == str(g["sha_s_packed"])


@pytest.mark.parametrize("k,n,groups", [(16, 64, 1), (128, 256, 1), (256, 4096, 2), (1024, 704, 8), (4096, 128, 32)])
def test_pack_matches_oracle_random(k, n, groups):
    rng = np.random.default_rng(k * 31 + n)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    s = rng.uniform(0.005, 0.02, size=(groups, n)).astype(np.float16)
    B = pkg.pack_weights(q)
    assert np.array_equal(B, orc.c_pack_weights(q))
    assert np.array_equal(pkg.unpack_weights(B, k, n), q)
    sp = pkg.permute_scales(s)
    assert np.array_equal(sp.view(np.uint16), orc.np_permute_scales(s).view(np.uint16))
    assert np.array_equal(pkg.unpermute_scales(sp).view(np.uint16), s.view(np.uint16))


def test_pack_rejects_bad_shapes():
    with pytest.raises(ValueError):
        pkg.pack_weights(np.zeros((8, 64), np.uint8))      # k % 16
    with pytest.raises(ValueError):
        pkg.pack_weights(np.zeros((16, 32), np.uint8))     # n % 64
    with pytest.raises(ValueError):
        pkg.quantize_pack(np.zeros((256, 64), np.float16), np.ones((1, 256), np.float16), -1)  # k % 128
    with pytest.raises(ValueError):
        pkg.quantize_pack(np.zeros((256, 128), np.float16), np.ones((2, 256), np.float16), 64)  # group size


def test_empty_pack():
    assert pkg.pack_weights(np.zeros((0, 64), np.uint8)).shape == (0, 128)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_columns_is_a_pure_slice(world):
    """Packing a column slice of the codes == slicing the packed layer (both permutations are local
    to 64-column blocks), for weights and for group scales."""
    k, n = 256, 1024 * 2
    rng = np.random.default_rng(world)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    s = rng.uniform(0.005, 0.02, size=(k // 128, n)).astype(np.float16)
    B, sp = pkg.pack_weights(q), pkg.permute_scales(s)
    ns = n // world
    for r in range(world):
        Bs, ss = pkg.shard_columns(B, sp, r, world)
        assert np.array_equal(Bs, pkg.pack_weights(np.ascontiguousarray(q[:, r * ns:(r + 1) * ns])))
        assert np.array_equal(ss.view(np.uint16),
                              pkg.permute_scales(np.ascontiguousarray(s[:, r * ns:(r + 1) * ns])).view(np.uint16))


def test_shard_rejects_ragged():
    B = np.zeros((8, 2 * 384), np.int32)
    sp = np.zeros((1, 384), np.float16)
    with pytest.raises(ValueError):
        pkg.shard_columns(B, sp, 0, 2)   # 192 columns per rank is not a multiple of 128


def test_blob_roundtrip_and_shard_on_load(tmp_path):
    k, n = 256, 1024
    rng = np.random.default_rng(8)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    s = rng.uniform(0.005, 0.02, size=(k // 128, n)).astype(np.float16)
    B, sp = pkg.pack_weights(q), pkg.permute_scales(s)
    path = tmp_path / "layer.w4a16"
    pkg.save_packed(path, B, sp)
    assert path.stat().st_size == 64 + B.nbytes + sp.nbytes
    B2, sp2, gs = pkg.load_packed(path)
    assert gs == 128 and np.array_equal(B2, B) and np.array_equal(sp2.view(np.uint16), sp.view(np.uint16))
    for world in (2, 4):
        for r in range(world):
            Bs, ss, _ = pkg.load_packed(path, r, world)
            want_B, want_s = pkg.shard_columns(B, sp, r, world)
            assert np.array_equal(Bs, want_B) and np.array_equal(ss.view(np.uint16), want_s.view(np.uint16))
    with pytest.raises(ValueError):
        pkg.load_packed(path, 0, 16)            # 64 columns per rank: not a multiple of 128
    # per-channel layer
    s1 = rng.uniform(0.005, 0.02, size=(1, n)).astype(np.float16)
    pkg.save_packed(path, B, pkg.permute_scales(s1))
    assert pkg.load_packed(path)[2] == -1


def test_blob_rejects_foreign_files(tmp_path):
    path = tmp_path / "junk.bin"
    path.write_bytes(b"not a packed layer" * 10)
    with pytest.raises(ValueError):
        pkg.load_packed(path)
    with pytest.raises(ValueError):
        pkg.load_packed(tmp_path / "missing.w4a16")
