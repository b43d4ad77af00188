"""Generate the golden vectors under tests/golden/ from the REFERENCE's own Python.

Run where a checkout of the reference project is at hand and pass its path:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It imports gemm/marlin_gemm/marlin.py (its missing ``marlin_lib`` extension is tolerated by the
module itself, marlin.py:5-8) and follows ``gen_quant4`` of gemm/marlin_gemm/marlin_test.py:18-55 on
the CPU: random fp16 weights -> scales -> codes -> fake-quantised ``ref`` -> ``Layer.pack`` -> packed
``B`` and permuted ``s``; then ``C_ref = matmul(A, ref)`` (marlin_test.py:64) in fp32 and in fp16.
Everything the oracle must reproduce is stored: inputs, intermediate codes, packed outputs, C_ref, and
the three permutation tables of ``_get_perms``.
"""
import os
import sys

import numpy as np
import torch
import torch.nn as nn

if len(sys.argv) != 2:
    sys.exit("usage: make_golden.py /path/to/reference")
REF = sys.argv[1]
sys.dont_write_bytecode = True
sys.path.insert(0, os.path.join(REF, "gemm", "marlin_gemm"))
import marlin  # noqa: E402  (the reference module)

OUT = os.path.dirname(os.path.abspath(__file__))
DEV = torch.device("cpu")


def gen_quant4(k, n, groupsize, gen):
    """marlin_test.py:18-55 with DEV = cpu and an explicit generator (m there == k here)."""
    maxq = 2 ** 4 - 1
    w = torch.randn((k, n), dtype=torch.float32, generator=gen).half()
    w_in = w.clone()
    if groupsize != -1:
        w = w.reshape((-1, groupsize, n)).permute(1, 0, 2).reshape((groupsize, -1))
    s = torch.max(torch.abs(w), 0, keepdim=True)[0]
    s *= 2 / maxq
    w = torch.round(w / s).int()
    w += (maxq + 1) // 2
    w = torch.clamp(w, 0, maxq)
    ref = (w - (maxq + 1) // 2).half() * s
    if groupsize != -1:
        def reshape(x):
            return x.reshape((groupsize, -1, n)).permute(1, 0, 2).reshape((k, n)).contiguous()
        ref = reshape(ref)
        w = reshape(w)
    s = s.reshape((-1, n)).contiguous()
    linear = nn.Linear(k, n)
    linear.weight.data = ref.t()
    layer = marlin.Layer(256, 256, groupsize=groupsize, cute_version=False)
    gs = k if groupsize == -1 else groupsize
    layer.k, layer.n, layer.groupsize = k, n, gs
    layer.B = torch.empty((k // 16, n * 16 // 8), dtype=torch.int, device=DEV)
    layer.s = torch.empty((k // gs, n), dtype=torch.half, device=DEV)
    layer.pack(linear, s.t())
    return w_in, w.to(torch.uint8), s, ref, layer.B, layer.s


def case(name, m, n, k, groupsize, seed):
    gen = torch.Generator().manual_seed(seed)
    A = torch.randn((m, k), dtype=torch.float32, generator=gen).half()
    w_in, q, s, ref, B, s_packed = gen_quant4(k, n, groupsize, gen)
    C_ref32 = torch.matmul(A.float(), ref.float())
    C_ref16 = torch.matmul(A, ref)
    np.savez_compressed(
        os.path.join(OUT, name + ".npz"),
        m=m, n=n, k=k, groupsize=groupsize, seed=seed,
        A=A.numpy(), w_in=w_in.numpy(), q=q.numpy(), s=s.numpy(), ref=ref.numpy(),
        B=B.numpy(), s_packed=s_packed.numpy(), C_ref32=C_ref32.numpy(), C_ref16=C_ref16.numpy(),
    )
    print(name, "B", tuple(B.shape), "s", tuple(s_packed.shape))


def main():
    perm, sp, sps = marlin._perm.numpy(), np.array(marlin._scale_perm), np.array(marlin._scale_perm_single)
    np.savez_compressed(os.path.join(OUT, "perms.npz"), perm=perm, scale_perm=sp, scale_perm_single=sps)
    # shapes taken from the reference's own test lists (marlin_test.py:78-131), kept small
    case("g128_m16_n256_k512", 16, 256, 512, 128, seed=0)      # test_groups
    case("gm1_m16_n256_k512", 16, 256, 512, -1, seed=1)        # test_groups, per-channel
    case("gm1_m3_n512_k192", 3, 512, 192, -1, seed=2)          # test_tiles m=3 / test_very_few_stages k=192
    case("g128_m12_n256_k128", 12, 256, 128, 128, seed=3)      # one group == k: single-scale permutation


if __name__ == "__main__":
    main()
