"""Benchmark of the W4A16 (Marlin-layout) GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1] at its M = 16 point): one STEP is the four Llama-2-7B linear layers
(N,K) = (12288,4096), (4096,4096), (22016,4096), (4096,11008), group size 128, batch M = 16, fp16
activations ~N(0,1), int4 codes uniform with zero-point 8, fp16 scales uniform in [0.005, 0.02]:
four GEMM launches that stream 101 MB of packed weights.  Weights rotate over 3 resident copies
(303 MB > 126 MB L2) so every launch reads its weights from HBM.

metric / value   weight HBM GB/s = packed-weight bytes of all ranks / time (CUDA events, max over ranks);
                 the K timed steps are replayed from one CUDA graph so the figure is the kernels', not
                 Python's launch path
e2e              the same metric through the public call `mul_host()` (C ABI w4a16_marlin_gemm_host) with HOST
                 buffers: per GEMM the activations are copied from pinned host memory and the output copied
                 back inside the call, plain launches, no graph;
                 weights stay resident on the device as a layer's parameters do (marlin.py:82-83)
roofline         HBM bound: algorithmic bytes (weights + scales + A + C) per launch / mean launch time
cpu_baseline     the CPU oracle (dequantise + fp32 GEMM, all host threads) on one full step
prefill          extra: TFLOP/s at M = 4096 on the same four shapes (BASELINE.json configs[2])
N > 1            every rank runs the same per-GPU workload on its own column shard of a layer N times as
                 wide (weak scaling, no collective on the data path); `gathered` reports the step with
                 an NCCL all-gather of the fp16 outputs added
--impl reference the reference has no runnable CPU or sm_100 implementation of this path, so this arm
                 times the CPU restatement of its algorithm (oracle/, kind "port") on rank 0 only
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]   # (N, K) of Llama-2-7B linears
GROUP = 128
M_DECODE = 16
COPIES = 3
METRIC = "w4a16_weight_hbm_gbs_m16"
UNIT = "GB/s"
# DRAM bytes per launch from one ncu capture of each of the step's four kernels (mean of 26.16, 9.21, 46.68 and
# 23.76 MB); the capture command and the per-shape figures are in profiles/decode_m16_dram_traffic.md.
NCU_DRAM_BYTES_PER_LAUNCH = 26.45e6
WORKLOAD = "llama2-7b linears (N,K) in {(12288,4096),(4096,4096),(22016,4096),(4096,11008)}, M=16, g128"


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
    """Samples SM clock and throttle reasons through NVML while the measurements run."""

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
                time.sleep(0.002)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add("nvml_unavailable:%s" % type(e).__name__)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)

    def summary(self):
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------------- reference arm
def cpu_time_step(threads_note=True, reps=1):
    """One full step (four GEMMs, M = 16) through the CPU oracle; returns (seconds, threads)."""
    from oracle import oracle as orc
    probs = [orc.make_problem(M_DECODE, n, k, GROUP, seed=i) for i, (n, k) in enumerate(SHAPES)]
    orc.c_gemm(*probs[1], GROUP)  # warm the thread pool
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        for (A, q, s) in probs:
            orc.c_gemm(A, q, s, GROUP)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, orc.num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    probs = [orc.make_problem(M_DECODE, n, k, GROUP, seed=i) for i, (n, k) in enumerate(SHAPES)]
    for _ in range(args.warmup):
        orc.c_gemm(*probs[1], GROUP)
    steps = min(args.steps, 20)   # bounded: one step is ~0.5 s of CPU work on 8 cores
    t0 = time.perf_counter()
    for _ in range(steps):
        for (A, q, s) in probs:
            orc.c_gemm(A, q, s, GROUP)
    dt = (time.perf_counter() - t0) / steps
    val = weight_bytes(SHAPES) / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference algorithm (dequantise + fp32 GEMM); "
                   "the reference ships no CPU kernel and its CUDA kernels do not run on sm_100"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                         "sample": "%d full steps (4 GEMMs, M=16, 101 MB of packed weights each)" % steps},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()   # raises if libw4a16.so is missing: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    peaks = load_peaks()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def make_layer(n, k, copies):
        """Random packed operands straight on the device: any int32 is a valid packed word (eight
        uniform codes) and the scale permutation of uniform values is uniform."""
        Bs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=dev, generator=gen)
              for _ in range(copies)]
        ss = [(torch.rand((k // GROUP, n), device=dev, generator=gen) * 0.015 + 0.005).half() for _ in range(copies)]
        return Bs, ss

    layers = [make_layer(n, k, COPIES) for (n, k) in SHAPES]
    acts = [torch.randn((M_DECODE, k), device=dev, generator=gen).half() for (_, k) in SHAPES]
    outs = [torch.zeros((M_DECODE, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]
    wss = [torch.zeros(n // 128 * 16, dtype=torch.int, device=dev) for (n, _) in SHAPES]

    def step(i):
        c = i % COPIES
        for li in range(len(SHAPES)):
            pkg.mul(acts[li], layers[li][0][c], outs[li], layers[li][1][c], wss[li])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    sampler.start()

    # ---- warm-up (eager, on the stream the graph will be captured on)
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        for i in range(max(args.warmup, 3)):
            step(i)
    side.synchronize()
    pkg.device_status(local)

    # ---- value: K steps captured in one CUDA graph, timed with events on the replay stream
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(args.steps):
            step(i)
    graph.replay()               # untimed: first replay uploads the graph
    barrier()
    sampler.active.set()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    ms_mine = e0.elapsed_time(e1)
    ms_total = max_over_ranks(ms_mine)
    ms_per_step = ms_total / args.steps
    per_rank_ms = None
    if world > 1:
        t = torch.zeros(world, device=dev, dtype=torch.float64)
        t[rank] = ms_mine / args.steps
        dist.all_reduce(t)
        per_rank_ms = [round(float(x), 5) for x in t.tolist()]
    launches = args.steps * len(SHAPES)
    wbytes = weight_bytes(SHAPES)
    value = world * wbytes / (ms_per_step * 1e-3) / 1e9

    alg = sum(algorithmic_bytes(M_DECODE, n, k) for n, k in SHAPES)
    achieved = alg / (ms_per_step * 1e-3) / 1e9     # per launch == per step here (same 4 launches / same time)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                "kernel": "w4a16_tc_kernel<16,256,grouped>", "launch_us": ms_total * 1e3 / launches,
                "algorithmic_bytes_per_launch": alg / len(SHAPES)}
    roofline["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH
    roofline["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over the step's four launches (profiles/decode_m16_dram_traffic.md)"

    # ---- e2e: the public call with host buffers, no graph
    hA = [a.cpu().pin_memory() for a in acts]
    hC = [torch.empty((M_DECODE, n), dtype=torch.half).pin_memory() for (n, _) in SHAPES]

    # the step's four GEMMs are independent layers: each is issued on its own stream so that one layer's
    # host<->device copies overlap another layer's kernel (each stream has its own library scratch)
    lanes = [torch.cuda.Stream(device=dev) for _ in SHAPES]

    def e2e_step(i):
        c = i % COPIES
        for li in range(len(SHAPES)):   # h2d copy of A, GEMM, d2h copy of C: one public call per GEMM
            pkg.mul_host(hA[li], layers[li][0][c], hC[li], layers[li][1][c], wss[li], acts[li], outs[li], stream=lanes[li])

    for i in range(3):
        e2e_step(i)
    barrier()
    e0.record()
    for st_ in lanes:
        st_.wait_event(e0)
    for i in range(args.steps):
        e2e_step(i)
    for st_ in lanes:
        torch.cuda.current_stream().wait_stream(st_)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    e2e = {"value": world * wbytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": sum(2 * M_DECODE * k for _, k in SHAPES),
           "d2h_bytes_per_step": sum(2 * M_DECODE * n for n, _ in SHAPES), "ms_per_step": e2e_ms}

    # ---- extras: decode sweep and prefill (not the headline; same kernels, same timing method)
    extras = {}
    if not args.no_extras:
        def time_graph(fn, reps):
            with torch.cuda.stream(side):
                fn(0)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(reps):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        sweep = {}
        for m in (1, 2, 4, 8, 16, 32, 64):
            am = [torch.randn((m, k), device=dev, generator=gen).half() for (_, k) in SHAPES]
            cm = [torch.zeros((m, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]
            per_shape = {}
            for li, (n, k) in enumerate(SHAPES):
                def one(i, li=li):
                    c = i % COPIES
                    pkg.mul(am[li], layers[li][0][c], cm[li], layers[li][1][c], wss[li])
                # a single layer's 3 copies may fit in L2: pad the rotation with the other layers' traffic
                ms = time_graph(one, 30)
                per_shape["%dx%d" % (n, k)] = {"us": ms * 1e3, "weight_gbs": n * k / 2 / (ms * 1e-3) / 1e9}
            def allfour(i):
                c = i % COPIES
                for li in range(len(SHAPES)):
                    pkg.mul(am[li], layers[li][0][c], cm[li], layers[li][1][c], wss[li])
            ms = time_graph(allfour, 20)
            sweep["m%d" % m] = {"step_us": ms * 1e3, "weight_gbs": wbytes / (ms * 1e-3) / 1e9,
                                "frac_of_peak": wbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "per_shape_l2_warmish": per_shape}
        extras["decode_sweep"] = sweep

        prefill = {}
        for m in (1024, 4096):
            am = [torch.randn((m, k), device=dev, generator=gen).half() for (_, k) in SHAPES]
            cm = [torch.zeros((m, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]
            res = {}
            for li, (n, k) in enumerate(SHAPES):
                def one(i, li=li):
                    pkg.mul(am[li], layers[li][0][i % COPIES], cm[li], layers[li][1][i % COPIES], wss[li])
                ms = time_graph(one, 5)
                tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
                res["%dx%d" % (n, k)] = {"ms": ms, "tflops": tf, "frac_of_peak": tf / peaks["bf16_tflops"]}
            tot_flops = sum(2.0 * m * n * k for n, k in SHAPES)
            tot_ms = sum(v["ms"] for v in res.values())
            prefill["m%d" % m] = {"tflops": tot_flops / (tot_ms * 1e-3) / 1e12,
                                  "frac_of_peak": tot_flops / (tot_ms * 1e-3) / 1e12 / peaks["bf16_tflops"], "per_shape": res}
            del am, cm
        extras["prefill"] = prefill

        # skinny batch, large K (N = 8192, K = 28672): every tile is cut between CTAs, so this is the stream-K split
        # and its fix-up; two resident weight copies (235 MB > L2) alternate
        sk_n, sk_k = 8192, 28672
        skB, skS = make_layer(sk_n, sk_k, 2)
        sk_ws = torch.zeros(sk_n // 128 * 16, dtype=torch.int, device=dev)
        streamk = {}
        for m in (16, 128):
            a_sk = torch.randn((m, sk_k), device=dev, generator=gen).half()
            c_sk = torch.zeros((m, sk_n), dtype=torch.half, device=dev)
            def one(i):
                pkg.mul(a_sk, skB[i % 2], c_sk, skS[i % 2], sk_ws)
            ms = time_graph(one, 20)
            t_hbm = algorithmic_bytes(m, sk_n, sk_k) / (peaks["hbm_gbs"] * 1e9)
            t_tensor = 2.0 * m * sk_n * sk_k / (peaks["bf16_tflops"] * 1e12)
            streamk["m%d" % m] = {"us": ms * 1e3, "weight_gbs": sk_n * sk_k / 2 / (ms * 1e-3) / 1e9,
                                  "tflops": 2.0 * m * sk_n * sk_k / (ms * 1e-3) / 1e12,
                                  "roofline_bound": "hbm" if t_hbm >= t_tensor else "tensor",
                                  "frac_of_roofline": max(t_hbm, t_tensor) / (ms * 1e-3)}
        del skB, skS
        extras["streamk_8192x28672"] = streamk
        extras["peaks"] = peaks

    gathered = None
    if world > 1:
        # the step with the fp16 outputs all-gathered along N (only where a caller asks for the full row)
        gbufs = [torch.empty((world * M_DECODE, n), dtype=torch.half, device=dev) for (n, _) in SHAPES]

        def gstep(i):
            step(i)
            for li in range(len(SHAPES)):
                dist.all_gather_into_tensor(gbufs[li], outs[li])
        for i in range(3):
            gstep(i)
        barrier()
        e0.record()
        for i in range(args.steps):
            gstep(i)
        e1.record()
        torch.cuda.synchronize()
        barrier()
        gms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
        gathered = {"value": world * wbytes / (gms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": gms,
                    "note": "eager launches + NCCL all_gather_into_tensor of the fp16 outputs per layer"}
        # the same step with the gathering epilogue: the GEMM stores its tiles into every rank's output buffer over
        # peer-mapped memory; a one-warp barrier kernel per layer takes the place of the collective
        pbufs, why = None, ""
        try:
            pbufs = [pkg.GatherBuffers(M_DECODE, world * n, rank, world, dev) for (n, _) in SHAPES]
        except Exception as exc:  # e.g. inter-process memory handles not permitted on this host
            why = str(exc)[:200]
        flag = torch.tensor([1 if pbufs is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)     # the arm runs on all ranks or on none
        if int(flag.item()) == 0:
            gathered["fused"] = {"unavailable": why or "a peer rank could not map the gather buffers"}
            pbufs = None
        try:
            if pbufs is None:
                raise StopIteration

            def fstep(i):
                c = i % COPIES
                for li in range(len(SHAPES)):
                    pkg.mul_gather(acts[li], layers[li][0][c], layers[li][1][c], wss[li], pbufs[li].dst_ptrs, rank)
                    pbufs[li].barrier()
            for i in range(3):
                fstep(i)
            barrier()
            e0.record()
            for i in range(args.steps):
                fstep(i)
            e1.record()
            torch.cuda.synchronize()
            barrier()
            fms_eager = max_over_ranks(e0.elapsed_time(e1)) / args.steps
            # and replayed from one CUDA graph, like `value` (the barrier's epoch counter lives on the device)
            with torch.cuda.stream(side):
                fstep(0)
            side.synchronize()
            fgraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(fgraph, stream=side):
                for i in range(args.steps):
                    fstep(i)
            fgraph.replay()
            barrier()
            e0.record()
            fgraph.replay()
            e1.record()
            torch.cuda.synchronize()
            barrier()
            fms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
            pkg.device_status(local)
            same = all(torch.equal(pbufs[li].local[:, rank * n:(rank + 1) * n], outs[li]) for li, (n, _) in enumerate(SHAPES))
            gathered["fused"] = {"value": world * wbytes / (fms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": fms,
                                 "ms_per_step_eager": fms_eager, "own_columns_match_plain_gemm": bool(same),
                                 "note": "K steps replayed from one CUDA graph; epilogue stores to all ranks' buffers + barrier kernel per layer, no NCCL"}
        except StopIteration:
            pass
        except Exception as exc:
            gathered["fused"] = {"unavailable": str(exc)[:200]}
        if pbufs is not None:       # on every rank, whatever happened above: close() holds a collective
            for b in pbufs:
                b.close()

    sampler.active.clear()
    sampler.stop()
    pkg.device_status(local)

    if rank == 0:
        cpu_s, cpu_threads = cpu_time_step(reps=2) if world == 1 else (None, None)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "weights rotate over %d resident copies (%.0f MB > 126 MB L2)"
                       % (COPIES, COPIES * wbytes / 1e6), "launch": "K steps replayed from one CUDA graph",
                       "parallelism": "column shards, one per GPU, no collective" if world > 1 else "single GPU"},
            "clocks": sampler.summary(), "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
        }
        if cpu_s is not None:
            line["cpu_baseline"] = {"value": wbytes / cpu_s / 1e9, "unit": UNIT, "cores": cpu_threads, "kind": "port",
                                    "sample": "one full step (4 GEMMs, M=16, 101 MB of packed weights), best of 2"}
        if gathered is not None:
            line["gathered"] = gathered
        if per_rank_ms is not None:
            line["per_rank_ms_per_step"] = per_rank_ms
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    """BASELINE.json configs[4]: Llama-2-70B layers column-sharded over the ranks (strong scaling: the layer is
    fixed, each rank owns N/G columns), M in {16, 4096}, with and without the NCCL all-gather of the fp16 outputs.
    One JSON line; `value` is the aggregate TFLOP/s at M = 4096 without the gather."""
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    gen = torch.Generator(device=dev).manual_seed(99 + rank)
    layers70 = [("gate_up", 57344, 8192), ("down", 8192, 28672)]
    side = torch.cuda.Stream(device=dev)
    out = {}
    for name, n_full, k in layers70:
        n = n_full // world
        copies = 2 if n * k // 2 > 70e6 else 4
        Bs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=dev, generator=gen) for _ in range(copies)]
        ss = [(torch.rand((k // GROUP, n), device=dev, generator=gen) * 0.015 + 0.005).half() for _ in range(copies)]
        ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=dev)
        for m in (16, 4096):
            A = torch.randn((m, k), device=dev, generator=gen).half()
            C = torch.zeros((m, n), dtype=torch.half, device=dev)
            reps = 20 if m == 16 else 4

            def one(i):
                pkg.mul(A, Bs[i % copies], C, ss[i % copies], ws)
            with torch.cuda.stream(side):
                one(0)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(reps):
                    one(i)
            g.replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / reps
            gms = None
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
                for _ in range(2):
                    one(0)
                    full = pkg.all_gather_columns(C, world)
                torch.cuda.synchronize()
                dist.barrier()
                a.record()
                for i in range(reps):
                    one(i)
                    full = pkg.all_gather_columns(C, world)
                b.record()
                torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b) / reps], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                gms = float(t.item())
                del full
                ggms = None
                try:  # the NCCL variant replayed from a CUDA graph as well, so that both arms are free of host launch cost
                    ng = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(ng, stream=side):
                        for i in range(reps):
                            one(i)
                            full = pkg.all_gather_columns(C, world)
                    ng.replay()
                    torch.cuda.synchronize()
                    dist.barrier()
                    a.record()
                    ng.replay()
                    b.record()
                    torch.cuda.synchronize()
                    t = torch.tensor([a.elapsed_time(b) / reps], device=dev, dtype=torch.float64)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    ggms = float(t.item())
                    del ng, full
                except Exception:
                    ggms = None
                pb, why = None, "a peer rank could not map the gather buffers"
                try:
                    pb = pkg.GatherBuffers(m, n_full, rank, world, dev)
                except Exception as exc:
                    why = str(exc)[:200]
                flag = torch.tensor([1 if pb is not None else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)     # the arm runs on all ranks or on none
                try:  # gathering epilogue + barrier kernel instead of the collective
                    if int(flag.item()) == 0:
                        raise RuntimeError(why)

                    def fused(i):
                        pkg.mul_gather(A, Bs[i % copies], ss[i % copies], ws, pb.dst_ptrs, rank)
                        pb.barrier()
                    with torch.cuda.stream(side):
                        for i in range(2):
                            fused(i)
                    side.synchronize()
                    fg = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(fg, stream=side):
                        for i in range(reps):
                            fused(i)
                    fg.replay()
                    torch.cuda.synchronize()
                    dist.barrier()
                    a.record()
                    fg.replay()
                    b.record()
                    torch.cuda.synchronize()
                    t = torch.tensor([a.elapsed_time(b) / reps], device=dev, dtype=torch.float64)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    fms = float(t.item())
                    pkg.device_status(local)
                    pkg.mul(A, Bs[(reps - 1) % copies], C, ss[(reps - 1) % copies], ws)
                    torch.cuda.synchronize()
                    fused_ok = bool(torch.equal(pb.local[:, rank * n:(rank + 1) * n], C))
                except Exception as exc:
                    fms, fused_ok = None, str(exc)[:200]
                if int(flag.item()) == 1:   # on every rank, whatever happened above: close() holds a collective
                    pb.close()
            flops = 2.0 * m * n_full * k
            wb = n_full * k / 2
            res = {"us": ms * 1e3, "tflops": flops / (ms * 1e-3) / 1e12, "weight_gbs": wb / (ms * 1e-3) / 1e9,
                   "frac_hbm_per_gpu": wb / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                   "frac_tensor_per_gpu": flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
            if gms is not None:
                res["gathered_us"] = gms * 1e3
                res["gathered_tflops"] = flops / (gms * 1e-3) / 1e12
                if ggms is not None:
                    res["gathered_graph_us"] = ggms * 1e3
                if fms is not None:
                    res["fused_gather_us"] = fms * 1e3
                    res["fused_gather_tflops"] = flops / (fms * 1e-3) / 1e12
                    res["fused_gather_own_columns_match"] = fused_ok
                else:
                    res["fused_gather_unavailable"] = fused_ok
            out["%s_m%d" % (name, m)] = res
            del A, C
        del Bs, ss
        torch.cuda.empty_cache()
    pkg.device_status(local)
    if rank == 0:
        tf = sum(2.0 * 4096 * nf * k for _, nf, k in layers70) / sum(out["%s_m4096" % nm]["us"] * 1e-6 for nm, _, _ in layers70) / 1e12
        print(json.dumps({"metric": "w4a16_llama70b_sharded_tflops_m4096", "value": tf, "unit": "TFLOP/s", "n_gpus": world,
                          "higher_is_better": True, "scaling": "strong", "dtype": "f16", "data": "synthetic",
                          "config": {"workload": "llama2-70b gate-up 57344x8192 and down 8192x28672, column-sharded, g128, M in {16,4096}"},
                          "results": out, "peaks": peaks}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the decode sweep and prefill extras")
    ap.add_argument("--case", default=None, help="NxKxM[xG]: time one shape only (graph replay; --eager for profilers)")
    ap.add_argument("--eager", action="store_true", help="with --case: plain launches instead of a CUDA graph")
    ap.add_argument("--workload", default="decode7b", choices=["decode7b", "sharded70b"],
                    help="decode7b: the headline step; sharded70b: Llama-2-70B layers column-sharded over the ranks")
    args = ap.parse_args()
    if args.workload == "sharded70b":
        run_sharded70b(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
