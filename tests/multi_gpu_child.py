"""Child process of test_gpu_multi.py: one rank of a column-sharded layer with the gathering epilogue.

Launched by torch.distributed.run, one process per GPU.  The process group (gloo: it only carries the 64-byte memory
handles and the final verdict) never touches the data path; the outputs cross NVLink through the GEMM kernel's own
stores and the ranks are ordered by the library's barrier kernel.  Exits non-zero on any mismatch.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as entry  # noqa: E402
from oracle import oracle as orc  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo")
    pkg = entry.load_package()
    n, k, gs = 512 * world, 1024, 128
    bufs = [pkg.GatherBuffers(1024, n, rank, world, dev) for _ in range(2)]     # alternate: no write-after-read hazard
    bad = 0
    for it, m in enumerate((16, 300, 1024, 16)):
        A, q, s = orc.make_problem(m, n, k, gs, 100 + it)                      # same on every rank
        layer = pkg.ColumnShardedLayer(pkg.pack_weights(q), pkg.permute_scales(s), rank, world, dev)
        out = layer.forward_gathered(torch.from_numpy(A).to(dev), bufs[it % 2])
        pkg.device_status(rank)
        ref = orc.c_gemm(A, q, s, gs)
        ok, err, bound = orc.tolerance_ok(out.float().cpu().numpy(), ref)
        # every rank must hold bit-identical rows: compare checksums of the gathered result over the ranks
        digest = torch.tensor([float(out.float().sum()), float(out.float().abs().sum())], dtype=torch.float64)
        lo, hi = digest.clone(), digest.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if not ok or not torch.equal(lo, hi):
            print("rank %d m=%d: ok=%s err=%g bound=%g digests %s %s" % (rank, m, ok, err, bound, lo, hi), flush=True)
            bad += 1
    for b in bufs:
        b.close()
    verdict = torch.tensor([bad])
    dist.all_reduce(verdict)
    dist.destroy_process_group()
    sys.exit(1 if int(verdict) else 0)


if __name__ == "__main__":
    main()
