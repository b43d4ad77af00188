"""Phase timeline of one GEMM launch, from the kernels' own time stamps.

    python awesome-cute_b200/phase_trace.py 4096x4096x16 22016x4096x16 [NxKxM[xSMS] ...]

Builds a trace twin of the library (the shipped sources with -DW4A16_TRACE: lane 0 of one warp per role stores
%globaltimer at each phase and sums the clocks it spent waiting) next to the shipped one, runs each shape a few
times eagerly on cuda:0 with rotating weight copies, and prints per phase the min / median / max over the CTAs of
the last launch, relative to the first CTA's entry, plus per-role wait and work clocks per k-stage.  Reading
%globaltimer costs a few hundred nanoseconds, so consecutive stamps of one warp are never closer than that.
A debugging aid: nothing printed here is a benchmark figure, and the shipped library carries none of the stamps.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libw4a16_trace.so")
SRC = ["w4a16_gemm.cu", "w4a16_quant.cu", "w4a16_pack.cpp", "w4a16_blob.cpp"]
PHASES = ["entry", "prologue done", "first stage landed", "first operand tile in TMEM", "last dequant (set 0)",
          "first accumulator folded", "last accumulator folded", "other CTAs' partial tiles seen", "epilogue done",
          "first ring-full of loads issued", "last TMA issued", "first MMA issued", "last MMA issued (issuer 0)", "TMEM freed",
          "first fix-up poll came back", "CTA-wide sync passed"]
BUCKETS = {0: "producer: wait for a free stage", 1: "producer: issue", 4: "dequant warp 0: wait for the stage",
           5: "dequant warp 0: wait for the operand buffer", 6: "dequant warp 0: wait + work",
           9: "MMA issuer 0: wait for the operand", 10: "MMA issuer 0: issue", 11: "MMA issuer 0: wait for the accumulator"}


def build():
    csrc = os.path.join(HERE, "csrc")
    newest = max(os.path.getmtime(os.path.join(csrc, f)) for f in os.listdir(csrc))
    if os.path.exists(SO) and os.path.getmtime(SO) >= newest:
        return
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC",
           "-DW4A16_TRACE", "-shared", "-o", SO] + [os.path.join(csrc, f) for f in SRC]
    subprocess.run(cmd, check=True)


def run(lib, n, k, m, sms=-1, group=128, reps=5):
    dev = torch.device("cuda:0")
    vp = ctypes.c_void_p
    gen = torch.Generator(device=dev).manual_seed(1)
    copies = 6
    Bs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), dtype=torch.int32, device=dev, generator=gen) for _ in range(copies)]
    ss = [(torch.rand((k // group, n), device=dev, generator=gen) * 0.015 + 0.005).half() for _ in range(copies)]
    A = torch.randn((m, k), device=dev, generator=gen).half()
    C = torch.zeros((m, n), dtype=torch.half, device=dev)
    ws = torch.zeros(n // 128 * 16, dtype=torch.int, device=dev)
    tr = torch.zeros((2 * 256 * 16,), dtype=torch.int64, device=dev)
    lib.w4a16_debug_set_trace(vp(tr.data_ptr()))
    stream = vp(torch.cuda.current_stream().cuda_stream)
    for i in range(reps):
        tr.zero_()
        rc = lib.w4a16_marlin_gemm(vp(A.data_ptr()), vp(Bs[i % copies].data_ptr()), vp(C.data_ptr()), vp(ss[i % copies].data_ptr()),
                                   m, n, k, vp(ws.data_ptr()), group, 0, stream, -1, -1, sms, 16)
        torch.cuda.synchronize()
        assert rc == 0, rc
    full = tr.cpu().numpy().astype(np.int64)
    t, bk = full[:4096].reshape(256, 16), full[4096:].reshape(256, 16)
    used = t[:, 0] > 0
    t0 = t[used][:, 0].min()
    steps = np.maximum(bk[used][:, 3], 1)
    print("n=%d k=%d m=%d sms=%d: %d CTAs, %d k-stages per CTA (median)" % (n, k, m, sms, used.sum(), np.median(steps)))
    for i, name in enumerate(PHASES):
        col = t[used][:, i]
        col = col[col > 0]
        if len(col):
            print("  %-34s min %7.2f  med %7.2f  max %7.2f us  (%d CTAs)" % (name, (col.min() - t0) / 1e3, (np.median(col) - t0) / 1e3,
                                                                             (col.max() - t0) / 1e3, len(col)))
    for i, name in BUCKETS.items():
        col = bk[used][:, i].astype(float)
        print("  %-46s %7.0f clocks per k-stage of the CTA" % (name, np.median(col / steps)))


def main():
    build()
    lib = ctypes.CDLL(SO)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.w4a16_marlin_gemm.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp, ci, ci, vp, ci, ci, ci, ci]
    for case in sys.argv[1:] or ["4096x4096x16", "22016x4096x16", "8192x28672x16"]:
        parts = [int(x) for x in case.split("x")]
        run(lib, parts[0], parts[1], parts[2], parts[3] if len(parts) > 3 else -1)


if __name__ == "__main__":
    main()
