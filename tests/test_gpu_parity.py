"""GPU parity tests: the sm_100a kernel, called through the C ABI, against the CPU oracle.

Shape lists follow the reference's own test file (gemm/marlin_gemm/marlin_test.py:78-167); where that
file only prints a loss, these assert  max|C - C_ref| <= 1e-2 * max|C_ref|  (fp32 compare, fp32
accumulation in the oracle) and the reference's relative-mean metric < 0.005 (marlin_test.py:74-75).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from gpu_common import DEV, check, orc, pack_problem, pkg, run_mul, run_problem, to_dev


def test_simt_cross_check():
    run_problem(16, 512, 1024, groupsize=128, fn=pkg.mul_simt)
    run_problem(3, 512, 192, 64, 256, groupsize=-1, fn=pkg.mul_simt)


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 12, 16, 24, 32, 48, 64, 118, 128, 152, 768, 1024])
def test_tiles(m):  # marlin_test.py:78-84
    for thread_k, thread_n in [(64, 256), (128, 128)]:
        if m > 16 and thread_k == 128:
            continue
        run_problem(m, 2 * 256, 1024, thread_k, thread_n, seed=m)


@pytest.mark.parametrize("k", [3 * 64 + 64 * 4 * 2 + 64 * i for i in range(1, 4)])
def test_k_stages_divisibility(k):  # marlin_test.py:86-89
    run_problem(16, 2 * 256, k, 64, 256, seed=k)


@pytest.mark.parametrize("k", [64, 128, 192])
def test_very_few_stages(k):  # marlin_test.py:91-94
    run_problem(16, 2 * 256, k, 64, 256, seed=k)


def test_errors():  # marlin_test.py:96-121
    m, n, k = 16, 256, 64
    A, q, s = orc.make_problem(m, n, k, -1, 0)
    At, Bt, st = pack_problem(A, q, s)
    C = torch.zeros((m, n), dtype=torch.half, device=DEV)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)
    with pytest.raises(RuntimeError, match="not compatible with thread_k=128"):
        pkg.mul(At, Bt, C, st, ws, 128, 128, -1)
    with pytest.raises(RuntimeError, match="not compatible with thread_k=256"):
        pkg.mul(At, Bt, C, st, ws, 256, 256, -1)
    s2 = torch.zeros((2, n), dtype=torch.half, device=DEV)
    with pytest.raises(RuntimeError):
        pkg.mul(At, Bt, C, s2, ws, 256, 256, -1)
    assert float(C.abs().sum()) == 0.0   # nothing was launched


@pytest.mark.parametrize("groupsize", [128, -1])
@pytest.mark.parametrize("n,k", [(256, 512), (256, 1024), (256 * 128, 1024)])
def test_groups(groupsize, n, k):  # marlin_test.py:123-131
    run_problem(16, n, k, 128, 128, groupsize, seed=n + k)


LLAMA = {  # marlin_test.py:133-167, (k, n) per layer
    "7B": [(4096, 3 * 4096), (4096, 4096), (4096, 2 * 10752), (10752, 4096)],
    "13B": [(5120, 3 * 5120), (5120, 5120), (5120, 2 * 13568), (13568, 5120)],
    "33B": [(6656, 3 * 6656), (6656, 6656), (6656, 2 * 17664), (17664, 6656)],
    "70B": [(8192, 3 * 8192), (8192, 8192), (8192, 2 * 21760), (21760, 8192)],
}


@pytest.mark.parametrize("model", sorted(LLAMA))
def test_llama_shapes(model):
    for k, n in LLAMA[model]:
        for batch in [1, 16]:
            run_problem(batch, n, k, 128, 128, -1, seed=batch)


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16, 32, 64])
@pytest.mark.parametrize("n,k", [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)])
def test_decode_sweep_g128(m, n, k):
    """The benchmark's decode configs (Llama-2-7B layer shapes, group 128)."""
    run_problem(m, n, k, groupsize=128, seed=m)


@pytest.mark.parametrize("m,n,k,gs,form", [
    (16, 2048, 4096, 128, "clusters of 8"), (5, 2048, 8192, -1, "clusters of 8"),
    (16, 4096, 2048, 128, "clusters of 4"), (1, 4096, 11008 - 11008 % 256, -1, "clusters of 4, uneven k shares"),
    (16, 8192, 1024, 128, "clusters of 2"), (9, 8192, 2048, -1, "clusters of 2"),
    (16, 12288, 512, 128, "one whole tile per CTA"), (3, 12288, 1024, -1, "one whole tile per CTA"),
    (16, 19200, 1024, 128, "stream-K, 150 tiles over 148 CTAs"), (16, 5120, 5120, 128, "stream-K, 40 tiles"),
])
def test_decode_kernel_forms(m, n, k, gs, form):
    """Every way the m <= 16 kernel splits a layer on a whole B200: one cluster per tile with the partial tiles
    reduced over distributed shared memory (2, 4 and 8 ranks, also with uneven k shares), one whole tile per CTA, and
    stream-K with the fix-up through L2; group and per-channel scales.  Oracle on column windows for the wide ones."""
    A, q, s = orc.make_problem(m, n, k, gs, seed=n + k + m)
    At, Bt, st = pack_problem(A, q, s)
    C = run_mul(At, Bt, st, m, n)
    for n0 in sorted(set([0, (n // 2) // 256 * 256, n - 256])):
        ref = orc.c_gemm(A, np.ascontiguousarray(q[:, n0:n0 + 256]), np.ascontiguousarray(s[:, n0:n0 + 256]), gs)
        check(C[:, n0:n0 + 256], ref, "%s, window %d" % (form, n0))
    C2 = run_mul(At, Bt, st, m, n)
    assert torch.equal(C, C2), form     # the order of the additions is fixed in every form


@pytest.mark.parametrize("sms", [1, 2, 3, 5, 7, 31, 64, 147, 148])
def test_stream_k_split_counts(sms):
    """Every way of cutting tiles between CTAs, including CTAs that hold only a middle slice of one tile."""
    run_problem(16, 512, 2048, groupsize=128, seed=sms, sms=sms)
    run_problem(40, 256, 4096, groupsize=-1, seed=sms, sms=sms)
    run_problem(200, 512, 1024, groupsize=128, seed=sms, sms=sms)


@pytest.mark.parametrize("m", [129, 192, 200, 384, 577, 2048])
def test_wide_batch_tiles(m):
    """Batches past 128 rows: the launcher picks 128- or 192-row tiles by padding; ragged last tiles."""
    run_problem(m, 512, 1024, groupsize=128, seed=m)
    run_problem(m, 256, 512, 64, 256, groupsize=-1, seed=m + 1)


@pytest.mark.parametrize("m", [16, 128])
def test_stream_k_large_k(m):
    """Skinny-m / large-k config: N=8192, K=28672 (oracle on a column window to stay in seconds)."""
    n, k, gs = 8192, 28672, 128
    A, q, s = orc.make_problem(m, n, k, gs, 11)
    At, Bt, st = pack_problem(A, q, s)
    C = run_mul(At, Bt, st, m, n)
    for n0 in (0, 3968, 8192 - 256):
        ref = orc.c_gemm(A, np.ascontiguousarray(q[:, n0:n0 + 256]), np.ascontiguousarray(s[:, n0:n0 + 256]), gs)
        check(C[:, n0:n0 + 256], ref, "window %d" % n0)


def test_repeated_calls_share_scratch_and_workspace():
    """One workspace and one stream over many calls (marlin_profiling.py:59-70 does this); different
    shapes back to back so partial tiles of one call are overwritten by the next."""
    ws = torch.zeros(4096 // 128 * 16, dtype=torch.int, device=DEV)
    probs = []
    for i, (m, n, k, gs) in enumerate([(16, 512, 2048, 128), (64, 1024, 1024, -1), (16, 512, 2048, 128), (130, 256, 512, 128)]):
        A, q, s = orc.make_problem(m, n, k, gs, 100 + i)
        probs.append((A, q, s, gs) + pack_problem(A, q, s))
    outs = []
    for rep in range(3):
        for (A, q, s, gs, At, Bt, st) in probs:
            C = torch.zeros((A.shape[0], q.shape[1]), dtype=torch.half, device=DEV)
            pkg.mul(At, Bt, C, st, ws)
            outs.append((C, A, q, s, gs))
    pkg.device_status(0)
    assert int(ws.abs().sum().item()) == 0
    for (C, A, q, s, gs) in outs:
        check(C, orc.c_gemm(A, q, s, gs))


def test_deterministic():
    A, q, s = orc.make_problem(16, 1024, 4096, 128, 5)
    At, Bt, st = pack_problem(A, q, s)
    C1 = run_mul(At, Bt, st, 16, 1024)
    C2 = run_mul(At, Bt, st, 16, 1024)
    assert torch.equal(C1, C2)


def test_tc_matches_simt_bitwise_close():
    """Two independent device implementations on the same operands."""
    A, q, s = orc.make_problem(48, 512, 1024, 128, 9)
    At, Bt, st = pack_problem(A, q, s)
    C1 = run_mul(At, Bt, st, 48, 512).float()
    C2 = run_mul(At, Bt, st, 48, 512, fn=pkg.mul_simt).float()
    assert float((C1 - C2).abs().max()) <= 2e-3 * float(C2.abs().max())


def test_golden_from_reference_packer(golden_dir):
    """Operands packed by the REFERENCE's Layer.pack (stored fixtures) through the kernel, against the
    reference's own matmul result stored beside them."""
    import glob, os
    for path in sorted(glob.glob(os.path.join(golden_dir, "g*.npz"))):
        g = np.load(path)
        m, n, k, gs = int(g["m"]), int(g["n"]), int(g["k"]), int(g["groupsize"])
        if g["s_packed"].shape[0] == 1:
            gs = -1
        tk, tn = (128, 128) if k % 128 == 0 else (64, 256)
        C = run_mul(to_dev(g["A"]), to_dev(g["B"]), to_dev(g["s_packed"]), m, n, tk, tn)
        check(C, g["C_ref32"], os.path.basename(path))


@pytest.mark.parametrize("name", ["big_g128_m16_n2048_k4096", "big_gm1_m16_n1024_k2048"])
def test_big_golden_against_reference_product(golden_dir, name):
    """The layer-sized golden cases through the kernel: operands packed by the shipped packer (whose output matches
    the reference packer's by digest, tests/test_packer.py), result against the REFERENCE's own fp32 product stored
    in the fixture.  2048 x 4096 g128 takes the cluster form of the m <= 16 kernel, 1024 x 2048 per-channel too."""
    from test_oracle import big_operands
    g, A, w, _ = big_operands(golden_dir, name)
    gs, s = int(g["groupsize"]), g["s"]
    m, n = int(g["m"]), int(g["n"])
    q = orc.c_quantize(w, s, gs)
    At, Bt, st = pack_problem(A, q, s)
    for sms in (-1, 37):
        C = run_mul(At, Bt, st, m, n, sms=sms)
        check(C, g["C_ref32"], "%s sms=%d" % (name, sms))


def test_linearity_at_full_size():
    """Size-independent property at a benchmark shape: GEMM(a1 + a2) == GEMM(a1) + GEMM(a2) up to fp16
    rounding of the three outputs."""
    m, n, k = 16, 22016, 4096
    A, q, s = orc.make_problem(m, n, k, 128, 21)
    A2 = np.random.default_rng(22).standard_normal((m, k), dtype=np.float32).astype(np.float16)
    A1h = (A.astype(np.float32) * 0.5).astype(np.float16)
    A2h = (A2.astype(np.float32) * 0.5).astype(np.float16)
    Asum = (A1h.astype(np.float32) + A2h.astype(np.float32)).astype(np.float16)
    _, Bt, st = pack_problem(A, q, s)
    C1 = run_mul(to_dev(A1h), Bt, st, m, n).float()
    C2 = run_mul(to_dev(A2h), Bt, st, m, n).float()
    Cs = run_mul(to_dev(Asum), Bt, st, m, n).float()
    # Asum is rounded to fp16 once more than A1h, A2h: allow that rounding through the GEMM
    assert float((Cs - (C1 + C2)).abs().max()) <= 1e-2 * float(Cs.abs().max())


def test_layer_forward_like_reference_module():
    """marlin.Layer: pack() + forward() (marlin.py:60-131) on the device."""
    k, n, gs = 512, 512, 128
    rng = np.random.default_rng(3)
    A, q, s = orc.make_problem(24, n, k, gs, 3)
    ref = orc.np_dequant(q, s, gs)                      # fake-quantised fp16 weights [k, n]
    linear = torch.nn.Linear(k, n, bias=False).half()
    linear.weight.data = torch.from_numpy(np.ascontiguousarray(ref.T))
    layer = pkg.Layer(k, n, groupsize=gs)
    layer.pack(linear, torch.from_numpy(np.ascontiguousarray(s.T)))
    assert np.array_equal(layer.B.numpy(), pkg.pack_weights(q))
    layer = layer.to(DEV)
    out = layer(to_dev(A).view(2, 12, k))
    pkg.device_status(0)
    assert tuple(out.shape) == (2, 12, n)
    check(out.view(24, n), orc.c_gemm(A, q, s, gs))


def test_mul_host_copies_in_and_out():
    """The host-buffer form of the call: pinned A in, pinned C out, one library call."""
    m, n, k, gs = 16, 1024, 2048, 128
    A, q, s = orc.make_problem(m, n, k, gs, 31)
    _, Bt, st = pack_problem(A, q, s)
    hA = torch.from_numpy(A).pin_memory()
    hC = torch.zeros((m, n), dtype=torch.half).pin_memory()
    A_stage = torch.empty((m, k), dtype=torch.half, device=DEV)
    C_stage = torch.empty((m, n), dtype=torch.half, device=DEV)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)
    for _ in range(2):
        pkg.mul_host(hA, Bt, hC, st, ws, A_stage, C_stage)
    pkg.device_status(0)
    want = orc.c_gemm(A, q, s, gs)
    check(hC, want, "mul_host")
    # the same call with its arguments prepared once, on a stream of its own
    side = torch.cuda.Stream(device=DEV)
    hC2 = torch.zeros((m, n), dtype=torch.half).pin_memory()
    op = pkg.HostGemm(hA, Bt, hC2, st, ws, A_stage, C_stage, stream=side)
    for _ in range(3):
        op()
    side.synchronize()
    check(hC2, want, "HostGemm")
    assert torch.equal(hC, hC2)


def test_bounded_wait_runs_out_and_the_stream_survives():
    """Failure detection without a GPU fault: a CTA waits for a partial tile nobody writes; after the limit the
    kernel returns a status instead of hanging, and the next GEMM on the same stream is correct."""
    import ctypes
    import time
    from awesome_cute_b200 import _lib
    m, n, k, gs = 16, 256, 1024, 128
    A, q, s = orc.make_problem(m, n, k, gs, 55)
    At, Bt, st = pack_problem(A, q, s)
    C = torch.zeros((m, n), dtype=torch.half, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(0).cuda_stream)
    run_mul(At, Bt, st, m, n)                     # scratch of this stream exists and is idle
    t0 = time.time()
    rc = _lib.lib.w4a16_selftest_unanswered_wait(p(At), p(Bt), p(C), p(st), m, n, k, gs, 0, stream, 300)
    assert rc == _lib.OK, _lib.last_cuda_error()
    assert _lib.lib.w4a16_device_status(0, stream) == _lib.ERR_TIMEOUT
    assert "timed out at site 4" in _lib.last_cuda_error()
    assert 0.25 < time.time() - t0 < 3.0          # it waited for the limit, not for ever
    assert _lib.lib.w4a16_device_status(0, stream) == _lib.OK      # status is cleared once read
    check(run_mul(At, Bt, st, m, n), orc.c_gemm(A, q, s, gs), "after the timeout")


@pytest.mark.parametrize("m", [16, 256])
def test_dependent_chain_eager_and_graph_replay(m):
    """Consecutive GEMMs on one stream where each one's output is the next one's activations: the next kernel
    may start early (programmatic dependent launch) but must not read its activations, write C or touch the
    scratch before the previous kernel has finished.  Checked eagerly and over several CUDA-graph replays."""
    dims, gs = [1024, 2048, 1024, 512], 128
    rng = np.random.default_rng(91)
    A0 = (rng.standard_normal((m, dims[0]), dtype=np.float32) * 0.5).astype(np.float16)
    layers = []
    for i in range(len(dims) - 1):
        k, n = dims[i], dims[i + 1]
        _, q, s = orc.make_problem(1, n, k, gs, 200 + i)
        layers.append((q, s, to_dev(pkg.pack_weights(q)), to_dev(pkg.permute_scales(s)),
                       torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)))
    acts = [to_dev(A0)] + [torch.zeros((m, n), dtype=torch.half, device=DEV) for n in dims[1:]]

    def chain():
        for i, (q, s, Bt, st, ws) in enumerate(layers):
            pkg.mul(acts[i], Bt, acts[i + 1], st, ws)

    def verify(tag):
        pkg.device_status(0)
        for i, (q, s, Bt, st, ws) in enumerate(layers):
            # each link against the oracle fed with the DEVICE's own input of that link
            check(acts[i + 1], orc.c_gemm(acts[i].cpu().numpy(), q, s, gs), "%s link %d" % (tag, i))

    for rep in range(3):
        for a in acts[1:]:
            a.zero_()
        chain()
        verify("eager %d" % rep)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        chain()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        chain()
        chain()
    for rep in range(4):
        for a in acts[1:]:
            a.zero_()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        verify("graph %d" % rep)


def test_random_shapes_stress():
    """Many small random problems back to back on one stream (different tilings, split counts and scratch
    reuse patterns), each checked against the oracle."""
    rng = np.random.default_rng(123)
    outs = []
    for i in range(40):
        m = int(rng.choice([1, 5, 16, 17, 33, 64, 100, 129, 200]))
        n = 256 * int(rng.integers(1, 9))
        k = 128 * int(rng.integers(1, 25))
        gs = int(rng.choice([128, -1]))
        sms = int(rng.choice([-1, -1, 148, 37, 11]))
        A, q, s = orc.make_problem(m, n, k, gs, 1000 + i)
        At, Bt, st = pack_problem(A, q, s)
        C = torch.zeros((m, n), dtype=torch.half, device=DEV)
        ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)
        pkg.mul(At, Bt, C, st, ws, -1, -1, sms)
        outs.append((C, A, q, s, gs, (m, n, k, gs, sms)))
    pkg.device_status(0)
    for (C, A, q, s, gs, tag) in outs:
        check(C, orc.c_gemm(A, q, s, gs), str(tag))


def test_single_cta_kernels_for_large_batches():
    """W4A16_PAIRS=0 keeps large batches on the single-CTA kernel (128- and 192-row tiles); checked in a child
    process because the switch is read once at load time."""
    import os
    import subprocess
    import sys
    code = (
        "import sys, os; sys.path.insert(0, os.getcwd()); sys.path.insert(0, os.path.join(os.getcwd(), 'tests'))\n"
        "from gpu_common import run_problem\n"
        "for m in (129, 192, 400, 1024):\n"
        "    run_problem(m, 512, 1024, groupsize=128, seed=m)\n"
        "    run_problem(m, 256, 512, 64, 256, groupsize=-1, seed=m + 1, sms=9)\n"
        "print('ok')\n")
    env = dict(os.environ, W4A16_PAIRS="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("sms", [2, 3, 9, 40, 147, 148])
def test_cta_pair_split_counts(sms):
    """The large-batch kernel with every way of cutting 256-column tiles between CTA pairs (sms / 2 pairs)."""
    run_problem(300, 1024, 2048, groupsize=128, seed=sms, sms=sms)
    run_problem(1000, 512, 1024, 64, 256, groupsize=-1, seed=sms + 7, sms=sms)


@pytest.mark.parametrize("sms", [2, 6, 14])
def test_cta_pair_whole_tile_waves_then_stream_k(sms):
    """With two or more 256-column tiles per CTA pair the pairs first take whole tiles round-robin and split only the
    last one or two waves by k-stages: 20 tiles over 1, 3 and 7 pairs (no remainder, 5 waves + 5 split tiles, 1 wave
    + 13 split tiles), group and per-channel scales."""
    run_problem(700, 1280, 2048, groupsize=128, seed=sms, sms=sms)
    run_problem(700, 1280, 2048, groupsize=-1, seed=sms + 3, sms=sms)


def test_cta_pair_waves_on_the_whole_gpu():
    """192 tiles on all pairs of the device (one whole-tile wave, then stream-K); oracle on column windows."""
    m, n, k, gs = 2304, 4096, 4096, 128
    A, q, s = orc.make_problem(m, n, k, gs, 21)
    At, Bt, st = pack_problem(A, q, s)
    C = run_mul(At, Bt, st, m, n)
    for n0 in (0, 1792, 4096 - 256):
        ref = orc.c_gemm(A, np.ascontiguousarray(q[:, n0:n0 + 256]), np.ascontiguousarray(s[:, n0:n0 + 256]), gs)
        check(C[:, n0:n0 + 256], ref, "window %d" % n0)


def test_cta_pair_tile_order_switches():
    """W4A16_MFAST=1 (tile index runs over the batch tiles first) and W4A16_WAVES=0 (contiguous stream-K ranges only)
    are read once at load time: each runs in a child process."""
    import os
    import subprocess
    import sys
    code = (
        "import sys, os; sys.path.insert(0, os.getcwd()); sys.path.insert(0, os.path.join(os.getcwd(), 'tests'))\n"
        "from gpu_common import run_problem\n"
        "for sms in (6, 14):\n"
        "    run_problem(700, 1280, 2048, groupsize=128, seed=sms, sms=sms)\n"
        "    run_problem(700, 1280, 2048, groupsize=-1, seed=sms + 3, sms=sms)\n"
        "print('ok')\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for switch in ({"W4A16_MFAST": "1"}, {"W4A16_WAVES": "0"}):
        r = subprocess.run([sys.executable, "-c", code], cwd=root, env=dict(os.environ, **switch), capture_output=True,
                           text=True, timeout=600)
        assert r.returncode == 0 and "ok" in r.stdout, str(switch) + r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("groupsize", [128, -1])
def test_device_quantize_pack_is_bit_exact(groupsize):
    """Layer.pack on the device against the host packer (itself pinned to the reference packer's golden vectors),
    on raw fp16 weights (every rounding case of round(w / s), clamping included), then through the GEMM."""
    k, n, m = 512, 1024, 16
    rng = np.random.default_rng(61)
    w = (rng.standard_normal((n, k), dtype=np.float32) * 0.06).astype(np.float16)       # [n, k] like nn.Linear.weight
    groups = 1 if groupsize == -1 else k // groupsize
    s = rng.uniform(0.005, 0.02, size=(groups, n)).astype(np.float16)
    B_host, sp_host = pkg.quantize_pack(w, s, groupsize)
    B_dev, sp_dev = pkg.quantize_pack_device(to_dev(w), to_dev(s), groupsize)
    torch.cuda.synchronize()
    assert np.array_equal(B_dev.cpu().numpy(), B_host)
    assert np.array_equal(sp_dev.cpu().numpy().view(np.uint16), sp_host.view(np.uint16))
    A = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    C = run_mul(to_dev(A), B_dev, sp_dev, m, n)
    q = orc.np_quantize(np.ascontiguousarray(w.T), s, groupsize)
    check(C, orc.c_gemm(A, q, s, groupsize), "device-packed")


def test_pair_kernel_dependent_chain_graph_replay():
    """Two large-batch GEMMs (CTA-pair kernel) where the first one's output is the second one's activations,
    eagerly and over CUDA-graph replays; the oracle is evaluated on column windows, fed with the device's own
    activations of each link."""
    m, gs = 1024, 128
    dims = [4096, 8192, 4096]
    rng = np.random.default_rng(17)
    A0 = (rng.standard_normal((m, dims[0]), dtype=np.float32) * 0.25).astype(np.float16)
    layers = []
    for i in range(2):
        k, n = dims[i], dims[i + 1]
        q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
        s = rng.uniform(0.005, 0.02, size=(k // gs, n)).astype(np.float16)
        layers.append((q, s, to_dev(pkg.pack_weights(q)), to_dev(pkg.permute_scales(s)),
                       torch.zeros(n // 128 * 16, dtype=torch.int, device=DEV)))
    acts = [to_dev(A0)] + [torch.zeros((m, n), dtype=torch.half, device=DEV) for n in dims[1:]]

    def chain():
        for i, (q, s, Bt, st, ws) in enumerate(layers):
            pkg.mul(acts[i], Bt, acts[i + 1], st, ws)

    def verify(tag):
        pkg.device_status(0)
        for i, (q, s, Bt, st, ws) in enumerate(layers):
            a_in = acts[i].cpu().numpy()
            for n0 in (0, dims[i + 1] - 256):
                ref = orc.c_gemm(a_in, np.ascontiguousarray(q[:, n0:n0 + 256]), np.ascontiguousarray(s[:, n0:n0 + 256]), gs)
                check(acts[i + 1][:, n0:n0 + 256], ref, "%s link %d window %d" % (tag, i, n0))

    chain()
    verify("eager")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        chain()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        chain()
        chain()
    for rep in range(2):
        for a in acts[1:]:
            a.zero_()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        verify("graph %d" % rep)


@pytest.mark.parametrize("m,nl,k,gs", [(16, 512, 1024, 128), (48, 256, 2048, 128), (200, 512, 512, 128),
                                       (1024, 2048, 4096, 128), (33, 512, 1024, -1), (7, 256, 256, -1),
                                       (1024, 4096, 4096, 128),      # CTA pairs, 128-row tiles
                                       (960, 4096, 4096, -1)])       # CTA pairs, 192-row tiles, per-channel scales
def test_gathering_epilogue_on_one_gpu(m, nl, k, gs):
    """The gathering GEMM with three destinations that all live on this GPU (the kernel only sees pointers): every
    destination receives this rank's columns, bit-identical to the plain GEMM, and nothing else is touched."""
    world, rank = 3, 1
    An, q, sn = orc.make_problem(m, nl, k, gs, m + nl)
    A, Bt, st = pack_problem(An, q, sn)
    ref = orc.c_gemm(An, q, sn, gs)
    ws = torch.zeros(nl // 128 * 16, dtype=torch.int, device=DEV)
    C = torch.zeros((m, nl), dtype=torch.half, device=DEV)
    pkg.mul(A, Bt, C, st, ws)
    dst = [torch.full((m, world * nl), 7.0, dtype=torch.half, device=DEV) for _ in range(world)]
    for _ in range(2):
        pkg.mul_gather(A, Bt, st, ws, [d.data_ptr() for d in dst], rank)
    pkg.device_status(0)
    check(C, ref, "plain")
    for d in dst:
        assert torch.equal(d[:, rank * nl:(rank + 1) * nl], C)
        assert bool((d[:, :rank * nl] == 7.0).all()) and bool((d[:, (rank + 1) * nl:] == 7.0).all())
    assert int(ws.abs().sum()) == 0


def test_gather_buffers_single_rank_and_barrier():
    """GatherBuffers with a world of one (no peers to map): allocation, the torch view of the library's memory,
    the barrier kernel (trivially satisfied) over several epochs, and release."""
    m, n, k = 16, 512, 1024
    An, q, sn = orc.make_problem(m, n, k, 128, 3)
    layer = pkg.ColumnShardedLayer(pkg.pack_weights(q), pkg.permute_scales(sn), 0, 1, DEV)
    bufs = pkg.GatherBuffers(32, n, 0, 1, DEV)
    for _ in range(3):
        out = layer.forward_gathered(to_dev(An), bufs)
    pkg.device_status(0)
    check(out, orc.c_gemm(An, q, sn, 128), "gathered world 1")
    bufs.close()


def test_peer_barrier_gives_up_when_a_rank_never_arrives():
    """A barrier over two ranks of which only this one exists: the flag nothing sets makes the bounded wait run
    out; the status says so and the stream stays usable."""
    import ctypes
    flags = torch.zeros(32, dtype=torch.int, device=DEV)    # two 64-byte flag blocks
    arr = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr() + 64)
    L = pkg._lib.lib
    assert L.w4a16_peer_barrier(arr, 2, 0, 0, torch.cuda.current_stream().cuda_stream, 50) == 0
    with pytest.raises(RuntimeError, match="timed out"):
        pkg.device_status(0)
    pkg.device_status(0)
    test_gather_buffers_single_rank_and_barrier()
