"""Benchmark of the W4A16 (Marlin-layout) GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the decode configuration the metric is quoted on): one STEP is the four Llama-2-7B linear layers
(N,K) = (12288,4096), (4096,4096), (22016,4096), (4096,11008), group size 128, batch M = 16, fp16
activations ~N(0,1), int4 codes uniform with zero-point 8, fp16 scales uniform in [0.005, 0.02]:
four GEMM launches that stream 101 MB of packed weights.  Weights rotate over 3 resident copies
(303 MB > 126 MB L2) so every launch reads its weights from HBM.  The reference's own shape list for these
layers is gemm/marlin_gemm/marlin_test.py:133-142 and gemm/marlin_gemm/marlin_profiling.py:89-94.

metric / value   weight HBM GB/s = packed-weight bytes of all ranks / time.  K steps are captured in one CUDA graph
                 (so the figure is the kernels', not Python's launch path); the graph is replayed R >= 5 times back to
                 back (R chosen so that the timed region is >= 50 ms), every replay between its own pair of CUDA
                 events on the launching stream; ms_per_step = median replay / K per rank, then the max over ranks
e2e              the same metric through the public call `HostGemm` (= `mul_host()` with its arguments prepared once;
                 C ABI w4a16_marlin_gemm_host) with HOST buffers: per GEMM the activations are copied from pinned host
                 memory and the output copied back inside the call, plain launches, no graph; weights stay resident on
                 the device as a layer's parameters do (marlin.py:82-83).  `value`: the step's four layers as independent
                 requests, a stream per layer and request slot, two slots alternating between steps;
                 `value_single_stream`: the same calls in order on one stream
roofline         HBM bound: algorithmic bytes (weights + scales + A + C) per launch / mean launch time
max_err / bound  inside `roofline` and `e2e`: one real packed layer (seeded codes and scales, packed by the shipped
                 packer) run through the same call and compared with the CPU oracle, outside every timed region
cpu_baseline     the CPU oracle (dequantise + fp32 GEMM, all host cores) on one full step
extras           decode sweep M in {1..64}, prefill M in {1024, 4096}, the large-K shape 8192 x 28672
sharded70b       last key of the line: the Llama-2-70B gate-up 57344x8192 and down 8192x28672 layers column-sharded
                 over the N ranks (strong scaling), M in {16, 4096}: plain, + NCCL all-gather, + gathering epilogue
N > 1            `value`: every rank runs the same per-GPU workload on its own column shard of a layer N times as
                 wide (weak scaling, no collective on the data path)
--impl reference the reference has no runnable CPU or sm_100 implementation of this path, so this arm
                 times the CPU restatement of its algorithm (oracle/, kind "port") on rank 0 only, on all host cores
"""
import argparse
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]   # (N, K) of Llama-2-7B linears
LAYERS70 = [("gate_up", 57344, 8192), ("down", 8192, 28672)]          # Llama-2-70B, column-sharded over the ranks
GROUP = 128
M_DECODE = 16
COPIES = 3
METRIC = "w4a16_weight_hbm_gbs_m16"
UNIT = "GB/s"
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from one ncu capture of each of the step's
# four kernels: 26.15, 8.82, 46.68 and 23.64 MB, mean 26.32 MB.  It is a property of the access pattern (every
# weight byte is read once), re-captured whenever the decode kernel's loads change.
NCU_DRAM_BYTES_PER_LAUNCH = 26.32e6
WORKLOAD = "llama2-7b linears (N,K) in {(12288,4096),(4096,4096),(22016,4096),(4096,11008)}, M=16, g128"
# the same for both arms, so that their lines describe one configuration
CONFIG = {
    "workload": WORKLOAD,
    "l2": "weights rotate over %d resident copies (303 MB > 126 MB L2)" % COPIES,
    "timing": "K steps per CUDA graph, >= 5 back-to-back replays (>= 50 ms), median replay, max over ranks",
    "parallelism": "one column shard per GPU, no collective on the data path",
}
MIN_REPLAYS = 5
MIN_TIMED_MS = 50.0


def weight_bytes(shapes):
    return sum(n * k // 2 for n, k in shapes)


def algorithmic_bytes(m, n, k, g=GROUP):
    return n * k // 2 + 2 * (k // g) * n + 2 * m * k + 2 * m * n


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        return {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops": float(pk["bf16_tflops"]),
                "bf16_tflops_sustained": float(pk.get("bf16_tflops_sustained", pk["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while timed regions run (every 20 ms: a timed region is
    at least 50 ms of back-to-back graph replays, and the poll itself stays out of the launch path's way)."""

    PERIOD_S = 0.02

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.active = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            while not self._stop_evt.is_set():
                if self.active.is_set():
                    self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    try:
                        mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    except Exception:
                        mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    for bit, name in names.items():
                        if mask & bit:
                            self.reasons.add(name)
                time.sleep(self.PERIOD_S)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add("nvml_unavailable:%s" % type(e).__name__)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)

    def summary(self):
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------------- reference arm
def cpu_time_step(reps=1):
    """One full step (four GEMMs, M = 16) through the CPU oracle on all host cores; returns (seconds, threads)."""
    from oracle import oracle as orc
    threads = orc.use_all_cores()
    probs = [orc.make_problem(M_DECODE, n, k, GROUP, seed=i) for i, (n, k) in enumerate(SHAPES)]
    orc.c_gemm(*probs[1], GROUP)  # warm the thread pool
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        for (A, q, s) in probs:
            orc.c_gemm(A, q, s, GROUP)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    threads = orc.use_all_cores()    # not the OMP_NUM_THREADS=1 a multi-rank launcher exports
    probs = [orc.make_problem(M_DECODE, n, k, GROUP, seed=i) for i, (n, k) in enumerate(SHAPES)]
    for _ in range(max(args.warmup, 1)):
        orc.c_gemm(*probs[1], GROUP)
    steps = min(args.steps, 20)   # bounded: one step is ~0.1-0.5 s of CPU work
    t0 = time.perf_counter()
    for _ in range(steps):
        for (A, q, s) in probs:
            orc.c_gemm(A, q, s, GROUP)
    dt = (time.perf_counter() - t0) / steps
    val = weight_bytes(SHAPES) / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": CONFIG,
        "note": "CPU restatement of the reference algorithm (dequantise + fp32 GEMM): the reference ships no CPU kernel "
                "and its CUDA kernels do not run on sm_100",
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "%d full steps (4 GEMMs, M=16, 101 MB of packed weights each)" % steps},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------- our arm
class Ctx:
    """Device, ranks, streams and the timing helpers every leg uses."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        import __graft_entry__ as entry
        self.torch, self.dist = torch, dist
        self.pkg = entry.load_package()   # raises if libw4a16.so is missing: there is no fallback
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = load_peaks()
        self.gen = torch.Generator(device=self.dev).manual_seed(1234 + self.rank)
        self.side = torch.cuda.Stream(device=self.dev)
        self.sampler = ClockSampler(self.local)
        self.sampler.start()

    def close(self):
        self.sampler.stop()
        if self.world > 1:
            self.dist.destroy_process_group()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def per_rank(self, x):
        if self.world == 1:
            return [x]
        t = self.torch.zeros(self.world, device=self.dev, dtype=self.torch.float64)
        t[self.rank] = x
        self.dist.all_reduce(t)
        return [float(v) for v in t.tolist()]

    def make_layer(self, n, k, copies):
        """Random packed operands straight on the device: any int32 is a valid packed word (eight
        uniform codes) and the scale permutation of uniform values is uniform."""
        torch = self.torch
        Bs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=self.dev, generator=self.gen)
              for _ in range(copies)]
        ss = [(torch.rand((k // GROUP, n), device=self.dev, generator=self.gen) * 0.015 + 0.005).half() for _ in range(copies)]
        return Bs, ss

    def randn_half(self, m, k):
        return self.torch.randn((m, k), device=self.dev, generator=self.gen).half()

    def capture(self, fn, reps, warm=1):
        """fn(i) for i in range(reps) captured into one CUDA graph (after `warm` eager calls on the capture stream)."""
        torch = self.torch
        with torch.cuda.stream(self.side):
            for i in range(warm):
                fn(i)
        self.side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.side):
            for i in range(reps):
                fn(i)
        return g

    def time_replays(self, graph, reps, min_replays=MIN_REPLAYS, min_ms=MIN_TIMED_MS, max_replays=200):
        """Replays `graph` (reps units each) back to back, each replay between its own pair of events on the launching
        stream.  Returns (median, min) milliseconds per unit on this rank and the number of timed replays."""
        torch = self.torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        graph.replay()                  # untimed: the first replay uploads the graph
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        est = max(a.elapsed_time(b), 1e-3)
        replays = int(min(max_replays, max(min_replays, math.ceil(min_ms / est))))
        if self.world > 1:              # the same count on every rank
            replays = int(self.max_over_ranks(float(replays)))
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
        self.barrier()
        self.sampler.active.set()
        evs[0].record()
        for i in range(replays):
            graph.replay()
            evs[i + 1].record()
        torch.cuda.synchronize()
        self.sampler.active.clear()
        self.barrier()
        ms = sorted(evs[i].elapsed_time(evs[i + 1]) / reps for i in range(replays))
        return ms[len(ms) // 2], ms[0], replays

    def time_graph(self, fn, reps, **kw):
        """An extra's figure: graph of `reps` calls, median replay, max over ranks.  The legs follow one another
        after a short pause, so that a leg that ran the part at its power cap (prefill) does not set the clocks
        and temperatures the next one (HBM-bound) starts from."""
        g = self.capture(fn, reps)
        time.sleep(0.25)
        med, best, _ = self.time_replays(g, reps, **kw)
        return self.max_over_ranks(med)


def parity_case():
    """One real packed layer (seeded codes and scales through the shipped packer) and its oracle result."""
    from oracle import oracle as orc
    m, n, k = M_DECODE, 4096, 4096
    A, q, s = orc.make_problem(m, n, k, GROUP, seed=2024)
    return (m, n, k), A, q, s, orc.c_gemm(A, q, s, GROUP)


def run_ours(args):
    ctx = Ctx()
    torch, pkg, dev, world, rank, peaks = ctx.torch, ctx.pkg, ctx.dev, ctx.world, ctx.rank, ctx.peaks
    warmup = max(args.warmup, 3)

    layers = [ctx.make_layer(n, k, COPIES) for (n, k) in SHAPES]
    acts = [ctx.randn_half(M_DECODE, k) for (_, k) in SHAPES]
    outs = [torch.zeros((M_DECODE, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]
    wss = [torch.zeros(n // 128 * 16, dtype=torch.int, device=dev) for (n, _) in SHAPES]

    def step(i):
        c = i % COPIES
        for li in range(len(SHAPES)):
            pkg.mul(acts[li], layers[li][0][c], outs[li], layers[li][1][c], wss[li])

    # ---- value: K steps captured in one CUDA graph; >= 5 back-to-back replays, each timed with its own events
    graph = ctx.capture(step, args.steps, warm=warmup)
    pkg.device_status(ctx.local)
    med_ms, min_ms, replays = ctx.time_replays(graph, args.steps)
    ms_per_step = ctx.max_over_ranks(med_ms)
    per_rank_med = ctx.per_rank(med_ms)
    per_rank_min = ctx.per_rank(min_ms)
    launches = args.steps * len(SHAPES) * replays
    wbytes = weight_bytes(SHAPES)
    value = world * wbytes / (ms_per_step * 1e-3) / 1e9

    alg = sum(algorithmic_bytes(M_DECODE, n, k) for n, k in SHAPES)
    achieved = alg / (ms_per_step * 1e-3) / 1e9     # per launch == per step here (same 4 launches / same time)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "peak_source": peaks["source"],
                "kernel": "w4a16_decode_kernel<grouped> (tcgen05, m <= 16)", "launch_us": ms_per_step * 1e3 / len(SHAPES),
                "algorithmic_bytes_per_launch": alg / len(SHAPES),
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over the step's four launches",
                "replays": replays, "timed_region_ms": med_ms * args.steps * replays,
                "per_rank_us_per_step_median": [round(v * 1e3, 3) for v in per_rank_med],
                "per_rank_us_per_step_min": [round(v * 1e3, 3) for v in per_rank_min]}

    # ---- parity of the timed call on a real packed layer (outside the timed regions)
    from oracle import oracle as orc
    (pm, pn, pk), pA, pq, ps, pref = parity_case()
    pAt = torch.from_numpy(pA).to(dev)
    pBt = torch.from_numpy(pkg.pack_weights(pq)).to(dev)
    pst = torch.from_numpy(pkg.permute_scales(ps)).to(dev)
    pC = torch.zeros((pm, pn), dtype=torch.half, device=dev)
    pws = torch.zeros(pn // 128 * 16, dtype=torch.int, device=dev)
    pkg.mul(pAt, pBt, pC, pst, pws)
    pkg.device_status(ctx.local)
    ok, err, bound = orc.tolerance_ok(pC.float().cpu().numpy(), pref)
    roofline["max_err"], roofline["bound"], roofline["parity_ok"] = err, bound, bool(ok)

    # ---- e2e: the public call with host buffers, no graph
    # Two request slots per layer, each with its own pinned host buffers, device staging and stream: consecutive
    # steps alternate between them, so that one step's copy back can overlap the next step's copy in and GEMM of the
    # same layer (with one slot per layer: 60 us per step, with two: 50 us).
    E2E_SLOTS = 2
    hA = [[a.cpu().pin_memory() for a in acts] for _ in range(E2E_SLOTS)]
    hC = [[torch.empty((M_DECODE, n), dtype=torch.half).pin_memory() for (n, _) in SHAPES] for _ in range(E2E_SLOTS)]
    dA = [acts] + [[a.clone() for a in acts] for _ in range(E2E_SLOTS - 1)]
    dC = [outs] + [[o.clone() for o in outs] for _ in range(E2E_SLOTS - 1)]
    dW = [wss] + [[w.clone() for w in wss] for _ in range(E2E_SLOTS - 1)]
    lanes = [[torch.cuda.Stream(device=dev) for _ in SHAPES] for _ in range(E2E_SLOTS)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def time_e2e(streams, steps):
        # streams[slot][layer].  One prepared call object per (slot, layer, weight copy): `HostGemm` is `mul_host`
        # with its argument checks and conversions done once, as a layer that runs every decode step would hold it
        nslots = len(streams)
        ops = [[[pkg.HostGemm(hA[sl][li], layers[li][0][c], hC[sl][li], layers[li][1][c], dW[sl][li], dA[sl][li], dC[sl][li],
                              stream=streams[sl][li])
                 for li in range(len(SHAPES))] for c in range(COPIES)] for sl in range(nslots)]
        used = set(st_ for row in streams for st_ in row)

        def e2e_step(i):
            for op in ops[i % nslots][i % COPIES]:   # h2d copy of A, GEMM, d2h copy of C: one public call per GEMM
                op()
        for i in range(6):
            e2e_step(i)
        ctx.barrier()
        ctx.sampler.active.set()
        e0.record()
        for st_ in used:
            st_.wait_event(e0)
        for i in range(steps):
            e2e_step(i)
        for st_ in used:
            torch.cuda.current_stream().wait_stream(st_)
        e1.record()
        torch.cuda.synchronize()
        ctx.sampler.active.clear()
        ctx.barrier()
        return ctx.max_over_ranks(e0.elapsed_time(e1)) / steps

    e2e_steps = max(args.steps, int(MIN_TIMED_MS / 0.05))    # >= 50 ms of plain launches
    e2e_ms = time_e2e(lanes, e2e_steps)
    e2e_single_ms = time_e2e([[lanes[0][0]] * len(SHAPES)], e2e_steps)
    e2e = {"value": world * wbytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": sum(2 * M_DECODE * k for _, k in SHAPES),
           "d2h_bytes_per_step": sum(2 * M_DECODE * n for n, _ in SHAPES), "ms_per_step": e2e_ms, "steps": e2e_steps,
           "streams": "the step's four layers as independent requests: a stream per layer and request slot, two slots "
                      "(own host buffers and staging) alternating between steps",
           "value_single_stream": world * wbytes / (e2e_single_ms * 1e-3) / 1e9, "ms_per_step_single_stream": e2e_single_ms}
    # parity of the host-buffer call
    hpA = torch.from_numpy(pA).pin_memory()
    hpC = torch.empty((pm, pn), dtype=torch.half).pin_memory()
    pC.zero_()
    pkg.mul_host(hpA, pBt, hpC, pst, pws, pAt, pC, stream=lanes[0][0])
    lanes[0][0].synchronize()
    pkg.device_status(ctx.local)
    ok, err, bound = orc.tolerance_ok(hpC.float().numpy(), pref)
    e2e["max_err"], e2e["bound"], e2e["parity_ok"] = err, bound, bool(ok)

    # ---- extras: decode sweep, prefill, large-K (not the headline; same kernels, same timing method)
    extras = {}
    if not args.no_extras:
        sweep = {}
        for m in (1, 2, 4, 8, 16, 32, 64):
            am = [ctx.randn_half(m, k) for (_, k) in SHAPES]
            cm = [torch.zeros((m, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]

            def allfour(i):
                c = i % COPIES
                for li in range(len(SHAPES)):
                    pkg.mul(am[li], layers[li][0][c], cm[li], layers[li][1][c], wss[li])
            ms = ctx.time_graph(allfour, 20, min_ms=10.0)
            sweep["m%d" % m] = {"step_us": round(ms * 1e3, 2), "weight_gbs": round(wbytes / (ms * 1e-3) / 1e9, 1),
                                "frac_of_peak": round(wbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
            if m == M_DECODE:
                per_shape = {}
                for li, (n, k) in enumerate(SHAPES):
                    def one(i, li=li):
                        c = i % COPIES
                        pkg.mul(am[li], layers[li][0][c], cm[li], layers[li][1][c], wss[li])
                    # (a single layer's 3 copies may partly stay in L2: the figure is an upper bound for that shape)
                    t = ctx.time_graph(one, 30, min_ms=10.0)
                    per_shape["%dx%d" % (n, k)] = {"us": round(t * 1e3, 2), "weight_gbs": round(n * k / 2 / (t * 1e-3) / 1e9, 1)}
                sweep["m%d" % m]["per_shape_l2_warmish"] = per_shape
        extras["decode_sweep"] = sweep

        # The same step with its four layers as INDEPENDENT requests: each layer on a stream of its own inside one CUDA
        # graph, each on half of the SMs (the launcher's `sms` argument), nothing joining the streams between steps.
        # One layer's start-up and fix-up then overlap another layer's streaming.  Not the headline: a decoder runs
        # its layers one after the other.
        lanes2 = [torch.cuda.Stream(device=dev) for _ in SHAPES]
        share = max(2, torch.cuda.get_device_properties(dev).multi_processor_count // 2)

        def conc_steps(k_steps):
            for st_ in lanes2:
                st_.wait_stream(torch.cuda.current_stream())
            for i in range(k_steps):
                c = i % COPIES
                for li in range(len(SHAPES)):
                    with torch.cuda.stream(lanes2[li]):
                        pkg.mul(acts[li], layers[li][0][c], outs[li], layers[li][1][c], wss[li], -1, -1, share)
            for st_ in lanes2:
                torch.cuda.current_stream().wait_stream(st_)
        k_conc = 20
        ms = ctx.time_graph(lambda i: conc_steps(k_conc) if i == 0 else None, 1, min_ms=20.0) / k_conc
        extras["independent_layers_side_by_side"] = {
            "step_us": round(ms * 1e3, 2), "weight_gbs": round(world * wbytes / (ms * 1e-3) / 1e9, 1),
            "frac_of_peak": round(wbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
            "how": "four streams inside one CUDA graph, %d CTAs per layer, %d steps per replay" % (share, k_conc)}

        prefill = {}
        for m in (1024, 4096):
            am = [ctx.randn_half(m, k) for (_, k) in SHAPES]
            cm = [torch.zeros((m, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]
            res = {}
            for li, (n, k) in enumerate(SHAPES):
                def one(i, li=li):
                    pkg.mul(am[li], layers[li][0][i % COPIES], cm[li], layers[li][1][i % COPIES], wss[li])
                ms = ctx.time_graph(one, 5, min_ms=20.0)
                tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
                res["%dx%d" % (n, k)] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_peak": round(tf / peaks["bf16_tflops"], 4)}
            tot_flops = sum(2.0 * m * n * k for n, k in SHAPES)
            tot_ms = sum(v["ms"] for v in res.values())
            prefill["m%d" % m] = {"tflops": round(tot_flops / (tot_ms * 1e-3) / 1e12, 1),
                                  "frac_of_peak": round(tot_flops / (tot_ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4),
                                  "frac_of_nominal_2250": round(tot_flops / (tot_ms * 1e-3) / 1e12 / 2250.0, 4), "per_shape": res}
            del am, cm
        extras["prefill"] = prefill

        # skinny batch, large K (N = 8192, K = 28672): every tile is cut between CTAs, so this is the stream-K split
        # and its fix-up; two resident weight copies (235 MB > L2) alternate
        sk_n, sk_k = 8192, 28672
        skB, skS = ctx.make_layer(sk_n, sk_k, 2)
        sk_ws = torch.zeros(sk_n // 128 * 16, dtype=torch.int, device=dev)
        streamk = {}
        for m in (16, 128):
            a_sk = ctx.randn_half(m, sk_k)
            c_sk = torch.zeros((m, sk_n), dtype=torch.half, device=dev)

            def one(i):
                pkg.mul(a_sk, skB[i % 2], c_sk, skS[i % 2], sk_ws)
            ms = ctx.time_graph(one, 20, min_ms=10.0)
            t_hbm = algorithmic_bytes(m, sk_n, sk_k) / (peaks["hbm_gbs"] * 1e9)
            t_tensor = 2.0 * m * sk_n * sk_k / (peaks["bf16_tflops"] * 1e12)
            streamk["m%d" % m] = {"us": round(ms * 1e3, 2), "weight_gbs": round(sk_n * sk_k / 2 / (ms * 1e-3) / 1e9, 1),
                                  "tflops": round(2.0 * m * sk_n * sk_k / (ms * 1e-3) / 1e12, 1),
                                  "roofline_bound": "hbm" if t_hbm >= t_tensor else "tensor",
                                  "frac_of_roofline": round(max(t_hbm, t_tensor) / (ms * 1e-3), 4)}
        del skB, skS
        extras["streamk_8192x28672"] = streamk

    gathered = None
    if world > 1 and not args.no_extras:
        gathered = measure_gathered_step(ctx, args, step, layers, acts, outs, wss)

    # free the 7B layers before the 70B ones are made
    del layers, graph
    torch.cuda.empty_cache()
    sharded = None
    if not args.no_sharded:
        sharded = measure_sharded70b(ctx)

    pkg.device_status(ctx.local)
    clocks = ctx.sampler.summary()
    if rank == 0:
        cpu_s, cpu_threads = cpu_time_step(reps=2) if world == 1 else (None, None)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": CONFIG,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
        }
        if cpu_s is not None:
            line["cpu_baseline"] = {"value": wbytes / cpu_s / 1e9, "unit": UNIT, "cores": cpu_threads, "kind": "port",
                                    "sample": "one full step (4 GEMMs, M=16, 101 MB of packed weights), best of 2"}
        line.update(extras)
        if gathered is not None:
            line["gathered"] = gathered
        line["peaks"] = peaks
        if sharded is not None:
            line["sharded70b"] = sharded      # last: the strong-scaling configuration, compact
        print(json.dumps(line), flush=True)
    ctx.close()


def measure_gathered_step(ctx, args, step, layers, acts, outs, wss):
    """The weak-scaled decode step with the fp16 outputs all-gathered along N after every layer: NCCL, and the
    GEMM's own gathering epilogue + barrier kernel."""
    torch, dist, pkg, dev, world, rank = ctx.torch, ctx.dist, ctx.pkg, ctx.dev, ctx.world, ctx.rank
    wbytes = weight_bytes(SHAPES)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gbufs = [torch.empty((world * M_DECODE, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]
    steps = max(args.steps, 100)

    def gstep(i):
        step(i)
        for li in range(len(SHAPES)):
            dist.all_gather_into_tensor(gbufs[li], outs[li])
    for i in range(3):
        gstep(i)
    ctx.barrier()
    e0.record()
    for i in range(steps):
        gstep(i)
    e1.record()
    torch.cuda.synchronize()
    ctx.barrier()
    gms = ctx.max_over_ranks(e0.elapsed_time(e1)) / steps
    gathered = {"value": world * wbytes / (gms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": gms,
                "note": "eager launches + NCCL all_gather_into_tensor of the fp16 outputs per layer"}
    pbufs, why = None, ""
    try:
        pbufs = [pkg.GatherBuffers(M_DECODE, world * n, rank, world, dev) for (n, _) in SHAPES]
    except Exception as exc:  # e.g. inter-process memory handles not permitted on this host
        why = str(exc)[:200]
    flag = torch.tensor([1 if pbufs is not None else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)     # the arm runs on all ranks or on none
    if int(flag.item()) == 0:
        gathered["fused"] = {"unavailable": why or "a peer rank could not map the gather buffers"}
        if pbufs is not None:
            for b in pbufs:
                b.close()
        return gathered
    try:
        def fstep(i):
            c = i % COPIES
            for li in range(len(SHAPES)):
                pkg.mul_gather(acts[li], layers[li][0][c], layers[li][1][c], wss[li], pbufs[li].dst_ptrs, rank)
                pbufs[li].barrier()
        fgraph = ctx.capture(fstep, args.steps, warm=3)
        med, _, _ = ctx.time_replays(fgraph, args.steps)
        fms = ctx.max_over_ranks(med)
        pkg.device_status(ctx.local)
        step(args.steps - 1)
        torch.cuda.synchronize()
        # (not bit for bit: the plain GEMM may run the cluster form, whose partial tiles are added in another order)
        diff = max(float((pbufs[li].local[:, rank * n:(rank + 1) * n].float() - outs[li].float()).abs().max())
                   for li, (n, _) in enumerate(SHAPES))
        scale = max(float(o.float().abs().max()) for o in outs)
        gathered["fused"] = {"value": world * wbytes / (fms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": fms,
                             "own_columns_vs_plain_gemm_max_abs_diff": ctx.max_over_ranks(diff), "bound": 1e-2 * scale,
                             "note": "graph replays; epilogue stores to all ranks' buffers + barrier kernel per layer, no NCCL"}
    except Exception as exc:
        gathered["fused"] = {"unavailable": str(exc)[:200]}
    for b in pbufs:       # on every rank, whatever happened above: close() holds a collective
        b.close()
    return gathered


def measure_sharded70b(ctx):
    """The Llama-2-70B gate-up (57344 x 8192) and down (8192 x 28672) layers column-sharded over the ranks (strong
    scaling: the layer is fixed, each rank owns N/G columns), M in {16, 4096}: GEMM alone; with N > 1 also + NCCL
    all-gather of the fp16 outputs (graph) and the gathering epilogue + barrier kernel (graph).  Times are us per
    GEMM, max over ranks of each rank's median replay.  On rank 0 a real packed shard is checked against the oracle."""
    torch, dist, pkg, dev, world, rank, peaks = ctx.torch, ctx.dist, ctx.pkg, ctx.dev, ctx.world, ctx.rank, ctx.peaks
    out = {}
    for name, n_full, k in LAYERS70:
        n = n_full // world
        copies = 2 if n * k // 2 > 70e6 else 4
        Bs, ss = ctx.make_layer(n, k, copies)
        ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=dev)
        for m in (16, 4096):
            A = ctx.randn_half(m, k)
            C = torch.zeros((m, n), dtype=torch.half, device=dev)
            reps = 20 if m == 16 else 4

            def one(i):
                pkg.mul(A, Bs[i % copies], C, ss[i % copies], ws)
            ms = ctx.time_graph(one, reps, min_ms=20.0)
            flops = 2.0 * m * n_full * k
            wb = n_full * k / 2
            res = {"us": round(ms * 1e3, 2), "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                   "weight_gbs": round(wb / (ms * 1e-3) / 1e9, 1),
                   "frac_hbm_per_gpu": round(algorithmic_bytes(m, n, k) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                   "frac_tensor_per_gpu": round(flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4)}
            if world > 1:
                try:  # + NCCL all-gather, replayed from a CUDA graph so that both arms are free of host launch cost
                    def nccl_arm(i):
                        one(i)
                        pkg.all_gather_columns(C, world)
                    res["nccl_gather_us"] = round(ctx.time_graph(nccl_arm, reps, min_ms=20.0) * 1e3, 2)
                except Exception as exc:
                    res["nccl_gather_unavailable"] = str(exc)[:120]
                pb, why = None, "a peer rank could not map the gather buffers"
                try:
                    pb = pkg.GatherBuffers(m, n_full, rank, world, dev)
                except Exception as exc:
                    why = str(exc)[:200]
                flag = torch.tensor([1 if pb is not None else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)     # the arm runs on all ranks or on none
                if int(flag.item()) == 1:
                    try:
                        def fused(i):
                            pkg.mul_gather(A, Bs[i % copies], ss[i % copies], ws, pb.dst_ptrs, rank)
                            pb.barrier()
                        fms = ctx.time_graph(fused, reps, min_ms=20.0)
                        pkg.device_status(ctx.local)
                        # the last captured call used copy (reps - 1) % copies: the plain GEMM on it must give this
                        # rank's columns of the gathered buffer (to rounding: the plain GEMM may add partial tiles
                        # in another order)
                        pkg.mul(A, Bs[(reps - 1) % copies], C, ss[(reps - 1) % copies], ws)
                        torch.cuda.synchronize()
                        res["fused_gather_us"] = round(fms * 1e3, 2)
                        own = pb.local[:, rank * n:(rank + 1) * n].float()
                        res["fused_own_columns_max_abs_diff"] = round(ctx.max_over_ranks(float((own - C.float()).abs().max())), 5)
                        res["fused_diff_bound"] = round(1e-2 * float(C.float().abs().max()), 4)
                        # bytes this rank's epilogue sends to the other ranks, against the link rate
                        res["fused_egress_gbs"] = round((world - 1) * 2.0 * m * n / (fms * 1e-3) / 1e9, 1)
                    except Exception as exc:
                        res["fused_gather_unavailable"] = str(exc)[:200]
                    pb.close()     # on every rank, whatever happened above: close() holds a collective
                else:
                    res["fused_gather_unavailable"] = why
                    if pb is not None:
                        pb.close()
            out["%s_m%d" % (name, m)] = res
            del A, C
        del Bs, ss
        torch.cuda.empty_cache()
    out["parity"] = sharded_parity(ctx)
    tf = sum(2.0 * 4096 * nf * k for _, nf, k in LAYERS70) / sum(out["%s_m4096" % nm]["us"] * 1e-6 for nm, _, _ in LAYERS70) / 1e12
    out["aggregate_tflops_m4096"] = round(tf, 1)
    out["n_gpus"] = world
    return out


def sharded_parity(ctx):
    """This rank's shard of a real packed down layer (8192 x 28672 cut with w4a16_shard_columns), M = 16, plain and
    (N > 1) through the gathering epilogue, against the CPU oracle on two column windows.  Max over ranks."""
    torch, dist, pkg, dev, world, rank = ctx.torch, ctx.dist, ctx.pkg, ctx.dev, ctx.world, ctx.rank
    from oracle import oracle as orc
    n_full, k, m = 8192, 28672, 16
    n = n_full // world
    A, q, s = orc.make_problem(m, n_full, k, GROUP, seed=70)      # the same on every rank
    Bf, sf = pkg.pack_weights(q), pkg.permute_scales(s)
    Br, sr = (Bf, sf) if world == 1 else pkg.shard_columns(Bf, sf, rank, world)
    At, Bt, st = (torch.from_numpy(np.ascontiguousarray(x)).to(dev) for x in (A, Br, sr))
    C = torch.zeros((m, n), dtype=torch.half, device=dev)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=dev)
    pkg.mul(At, Bt, C, st, ws)
    pkg.device_status(ctx.local)
    res = {}

    def worst(Cd, col0, width):
        err_max, bound_min, ok_all = 0.0, float("inf"), True
        for w0 in sorted(set([0, width - 256])):
            g0 = col0 + w0
            ref = orc.c_gemm(A, np.ascontiguousarray(q[:, g0:g0 + 256]), np.ascontiguousarray(s[:, g0:g0 + 256]), GROUP)
            ok, err, bound = orc.tolerance_ok(Cd[:, w0:w0 + 256].float().cpu().numpy(), ref)
            err_max, bound_min, ok_all = max(err_max, err), min(bound_min, bound), ok_all and ok
        return err_max, bound_min, ok_all
    err, bound, ok = worst(C, rank * n, n)
    res["plain"] = {"max_err": ctx.max_over_ranks(err), "bound": bound, "ok": bool(ctx.max_over_ranks(0.0 if ok else 1.0) == 0.0)}
    if world > 1:
        pb = None
        try:
            pb = pkg.GatherBuffers(m, n_full, rank, world, dev)
        except Exception:
            pb = None
        flag = torch.tensor([1 if pb is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 1:
            pkg.mul_gather(At, Bt, st, ws, pb.dst_ptrs, rank)
            pb.barrier()
            torch.cuda.synchronize()
            pkg.device_status(ctx.local)
            # the whole gathered row as this rank sees it: its own columns and every peer's
            err, bound, ok = worst(pb.local, 0, n_full)
            nxt = ((rank + 1) % world) * n
            e2, b2, ok2 = worst(pb.local[:, nxt:nxt + n], nxt, n)
            res["fused_gather"] = {"max_err": ctx.max_over_ranks(max(err, e2)), "bound": min(bound, b2),
                                   "ok": bool(ctx.max_over_ranks(0.0 if (ok and ok2) else 1.0) == 0.0)}
            pb.close()
        elif pb is not None:
            pb.close()
    return res


def run_case(args):
    """One shape, per-launch device time; with --eager the command profilers are pointed at.
    --case NxKxM[xG]  e.g. 22016x4096x16  (G = 128 default, -1 per-channel)."""
    import torch

    import __graft_entry__ as entry
    pkg = entry.load_package()
    parts = [int(x) for x in args.case.split("x")]
    n, k, m = parts[:3]
    g = parts[3] if len(parts) > 3 else GROUP
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(7)
    copies = max(2, min(8, int(300e6 // (n * k // 2)) + 1))     # rotate through > 2 x L2 of weights
    if args.copies > 0:
        copies = args.copies                                     # (1: the weights stay in L2, the bound of any prefetch)
    Bs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=dev, generator=gen) for _ in range(copies)]
    groups = 1 if g == -1 else k // g
    ss = [(torch.rand((groups, n), device=dev, generator=gen) * 0.015 + 0.005).half() for _ in range(copies)]
    A = torch.randn((m, k), device=dev, generator=gen).half()
    C = torch.zeros((m, n), dtype=torch.half, device=dev)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=dev)
    if args.eager:
        # plain launches, one event pair each: what a profiler is pointed at (host launch cost included)
        for i in range(args.warmup):
            pkg.mul(A, Bs[i % copies], C, ss[i % copies], ws)
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for i, (a, b) in enumerate(evs):
            a.record()
            pkg.mul(A, Bs[i % copies], C, ss[i % copies], ws)
            b.record()
        torch.cuda.synchronize()
        us = sorted(a.elapsed_time(b) * 1e3 for a, b in evs)
        med, best = us[len(us) // 2], us[0]
    else:
        # the launches replayed from one CUDA graph: device time per launch without the host's launch path
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(side):
            for i in range(max(args.warmup, 1)):
                pkg.mul(A, Bs[i % copies], C, ss[i % copies], ws)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(args.steps):
                pkg.mul(A, Bs[i % copies], C, ss[i % copies], ws)
        g.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3 / args.steps)
        us.sort()
        med, best = us[len(us) // 2], us[0]
    pkg.device_status(0)
    print(json.dumps({"case": args.case, "copies": copies, "mode": "eager" if args.eager else "graph",
                      "launch_us_median": med, "launch_us_min": best,
                      "weight_gbs": n * k / 2 / (med * 1e-6) / 1e9, "tflops": 2.0 * m * n * k / (med * 1e-6) / 1e12}), flush=True)


def run_sharded70b(args):
    """Only the column-sharded Llama-2-70B configuration, as a line of its own."""
    ctx = Ctx()
    out = measure_sharded70b(ctx)
    ctx.pkg.device_status(ctx.local)
    if ctx.rank == 0:
        print(json.dumps({"metric": "w4a16_llama70b_sharded_tflops_m4096", "value": out["aggregate_tflops_m4096"],
                          "unit": "TFLOP/s", "n_gpus": ctx.world, "higher_is_better": True, "scaling": "strong",
                          "dtype": "f16", "data": "synthetic",
                          "config": {"workload": "llama2-70b gate-up 57344x8192 and down 8192x28672, column-sharded, g128, M in {16,4096}"},
                          "clocks": ctx.sampler.summary(), "results": out, "peaks": ctx.peaks}), flush=True)
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the decode sweep, prefill and large-K extras")
    ap.add_argument("--no-sharded", action="store_true", help="skip the column-sharded 70B configuration")
    ap.add_argument("--case", default=None, help="NxKxM[xG]: time one shape only (graph replay; --eager for profilers)")
    ap.add_argument("--eager", action="store_true", help="with --case: plain launches instead of a CUDA graph")
    ap.add_argument("--copies", type=int, default=0,
                    help="with --case: weight copies the launches rotate through (default: enough for > 2 x L2; 1 keeps the weights in L2)")
    ap.add_argument("--workload", default="decode7b", choices=["decode7b", "sharded70b"],
                    help="decode7b: the headline step; sharded70b: only the Llama-2-70B layers column-sharded over the ranks")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "sharded70b":
        run_sharded70b(args)
    elif args.case:
        run_case(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
