"""The launcher's choice of kernel and work cut, through w4a16_plan (host arithmetic only: runs without a GPU).

The reference picks its kernel in the `CALL_IF` table at the end of its launcher (gemm/marlin_gemm/
marlin_cute_kernel.cu:62-115: thread_k x thread_n x batch blocks x group size) and always launches one CTA per SM.
Here the choice depends on the problem; these cases pin it for a 148-SM B200, one per branch."""
import __graft_entry__ as entry

pkg = entry.load_package()


def plan(m, n, k, g=128, **kw):
    rc, d = pkg.plan(m, n, k, g, **kw)
    assert rc == 0
    return d


def test_decode_forms():
    # the four layers of the benchmark's step at m = 16
    d = plan(16, 4096, 4096)
    assert (d["kernel"], d["ctas_per_worker"], d["workers"], d["stages_per_worker"]) == ("decode_cluster", 4, 128, 4)
    d = plan(16, 4096, 11008)
    assert (d["kernel"], d["ctas_per_worker"], d["workers"]) == ("decode_cluster", 4, 128)
    d = plan(16, 12288, 4096)      # 96 tiles on 148 SMs: one whole tile per CTA, no fix-up
    assert (d["kernel"], d["workers"], d["stages_per_worker"]) == ("decode", 96, 16)
    d = plan(16, 22016, 4096)      # more tiles than SMs: stream-K
    assert (d["kernel"], d["workers"], d["stages_per_worker"]) == ("decode", 145, 19)
    # the same for every m <= 16, grouped or per-channel
    assert plan(1, 4096, 4096) == plan(16, 4096, 4096) == plan(16, 4096, 4096, -1)
    # deep layers stay on stream-K, very narrow deep shards take clusters of eight
    assert plan(16, 8192, 28672)["kernel"] == "decode"
    d = plan(16, 1024, 28672)
    assert (d["kernel"], d["ctas_per_worker"], d["workers"]) == ("decode_cluster", 8, 64)
    # a very narrow layer is not cut one stage per CTA (one tile 112 ways: 57 us) but into a few long pieces (13 us)
    d = plan(16, 128, 28672)
    assert (d["kernel"], d["workers"], d["stages_per_worker"]) == ("decode", 14, 8)
    # k not a multiple of 256: the general kernel with 128-k stages
    d = plan(16, 4096, 4224)
    assert (d["kernel"], d["tile_rows"], d["k_per_stage"]) == ("single", 16, 128)
    # an explicit split count is honoured and keeps the stream-K form
    d = plan(16, 4096, 4096, sms=37)
    assert (d["kernel"], d["workers"]) == ("decode", 37)


def test_small_batches_on_pairs():
    for m, tm in ((17, 32), (32, 32), (33, 64), (64, 64)):
        d = plan(m, 4096, 4096)
        assert (d["kernel"], d["tile_rows"], d["k_per_stage"], d["ctas_per_worker"]) == ("pairs", tm, 256, 2)


def test_few_wide_tiles_are_cut_along_the_tiles():
    # 16 pair tiles of 32 stages: cut 2 ways (32 pairs of 16 stages), not 4.6 ways over 74 pairs
    d = plan(128, 4096, 4096)
    assert (d["kernel"], d["tile_rows"], d["workers"], d["stages_per_worker"]) == ("pairs", 128, 32, 16)
    # 4 pair tiles: 8 pairs
    assert plan(128, 1024, 4096)["workers"] == 8
    # two batch tiles of 128 rows
    d = plan(256, 4096, 4096)
    assert (d["tile_rows"], d["workers"], d["stages_per_worker"]) == (128, 64, 16)
    # many tiles, few per pair: the even cut stays
    d = plan(100, 12288, 4096)
    assert (d["kernel"], d["workers"]) == ("pairs", 74)
    # too few stages per pair for the pairs: single CTAs, cut along the tiles as well
    d = plan(128, 4096, 512)
    assert (d["kernel"], d["workers"], d["stages_per_worker"]) == ("single", 32, 4)


def test_large_batches():
    # 96 tiles on 74 pairs: 64 pairs of one and a half tiles each
    d = plan(1024, 4096, 4096)
    assert (d["kernel"], d["tile_rows"], d["workers"], d["whole_tile_waves"], d["stages_per_worker"]) == ("pairs", 192, 64, 0, 48)
    # 288 tiles: four whole waves on 72 pairs, nothing left for stream-K
    d = plan(1024, 12288, 4096)
    assert (d["workers"], d["whole_tile_waves"], d["stages_per_worker"]) == (72, 4, 0)
    # whole waves, then stream-K over all pairs
    d = plan(4096, 22016, 4096)
    assert (d["kernel"], d["tile_rows"], d["workers"]) == ("pairs", 192, 74) and d["whole_tile_waves"] >= 20
    # a batch of 129..  rows: 192-row tiles unless 128-row tiles waste fewer rows
    assert plan(384, 22016, 4096)["tile_rows"] == 192
    assert plan(256, 22016, 4096)["tile_rows"] == 128


def test_other_device_sizes_and_refusals():
    assert plan(1024, 4096, 4096, device_sms=132)["workers"] <= 66
    assert plan(0, 4096, 4096)["kernel"] == "none"                       # nothing to do (marlin_cute_kernel.cu:59-60)
    assert pkg.plan(16, 4100, 4096)[0] == 1                              # W4A16_ERR_PROB_SHAPE, as the GEMM call
    assert pkg.plan(16, 4096, 4096, 64)[0] == 2                          # W4A16_ERR_KERN_SHAPE: group size 64
    assert pkg.plan(16, 4096, 4096, device_sms=1)[0] == 5                # W4A16_ERR_ARG


def test_every_plan_covers_its_problem():
    """Whatever the launcher chooses, the workers' ranges cover every (tile, k-stage) of the problem, nobody is asked
    for more workers than the device has, and the tile sizes are ones the kernels are built for.  2000 seeded shapes
    on three device sizes."""
    import numpy as np
    rng = np.random.default_rng(11)
    for _ in range(2000):
        m = int(rng.choice([1, 3, 16, 17, 31, 32, 48, 64, 65, 100, 128, 129, 200, 256, 384, 500, 1024, 4096]))
        n = int(rng.integers(1, 120)) * 256
        k = int(rng.integers(1, 120)) * 128
        g = int(rng.choice([128, -1]))
        sms = int(rng.choice([132, 148, 160]))
        rc, d = pkg.plan(m, n, k, g, device_sms=sms)
        assert rc == 0, (m, n, k, g, rc)
        tm, ks, w, per = d["tile_rows"], d["k_per_stage"], d["workers"], d["stages_per_worker"]
        assert tm in (16, 32, 64, 128, 192) and ks in (64, 128, 256) and k % ks == 0 and w >= 1, (m, n, k, d)
        k_iters = k // ks
        m_tiles = -(-m // tm)
        if d["kernel"] == "pairs":
            tiles = n // 256 * m_tiles
            assert 2 * w <= sms
            left = tiles - d["whole_tile_waves"] * w
            assert left >= 0 and w * per >= left * k_iters, (m, n, k, d)
        elif d["kernel"] == "decode_cluster":
            tiles = n // 128
            cl = d["ctas_per_worker"]
            assert m <= 16 and w == tiles * cl and w <= sms and cl in (2, 4, 8)
            assert per >= 2 and per * cl <= k_iters < (per + 1) * cl + cl, (m, n, k, d)
        else:
            tiles = n // 128 * m_tiles
            assert d["kernel"] in ("single", "decode") and w <= sms
            assert (d["kernel"] == "decode") == (m <= 16 and k % 256 == 0)
            assert w * per >= tiles * k_iters, (m, n, k, d)
            assert (w - 1) * per < tiles * k_iters, (m, n, k, d)      # no worker without work
