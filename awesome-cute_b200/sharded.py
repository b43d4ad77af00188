"""Column-sharded W4A16 layers: each rank of a process group owns N/G output columns of a packed layer.

The reference is single-GPU; this is the only multi-GPU piece.  A column shard is a pure slice of the
packed operands (both Marlin permutations are local to 64-column blocks, gemm/marlin_gemm/marlin.py:29-57),
so every rank runs the unchanged GEMM on its slice and there is no reduction between GPUs.  The one
exchange step, used only when the caller asks for the full output row, is an all-gather of the fp16
outputs along N (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
import numpy as np
import torch
import torch.distributed as dist

from . import marlin


class ColumnShardedLayer:
    """Rank-local shard of a packed layer.

    B, s_packed: the FULL packed layer on the host (numpy), as produced by pack_weights/permute_scales or
    Layer.pack.  Only this rank's slice is kept (and moved to `device`)."""

    def __init__(self, B, s_packed, rank, world, device, max_par=16):
        if world < 1 or not (0 <= rank < world):
            raise ValueError("bad rank %d of %d" % (rank, world))
        self.rank, self.world = rank, world
        self.k = B.shape[0] * 16
        self.n = B.shape[1] // 2
        if self.n % world or (self.n // world) % 256:
            # the reference's operator wants n % 256 == 0 for m > 16 (marlin_cute_kernel.cu:39-58); keep that per shard
            raise ValueError("n=%d does not split into %d column shards that are multiples of 256" % (self.n, world))
        self.n_local = self.n // world
        Bs, ss = marlin.shard_columns(B, s_packed, rank, world)
        self.groupsize = -1 if ss.shape[0] == 1 else self.k // ss.shape[0]
        self.device = torch.device(device)
        self.B = torch.from_numpy(Bs).to(self.device)
        self.s = torch.from_numpy(ss).to(self.device)
        self.workspace = torch.zeros(self.n_local // 128 * max_par, dtype=torch.int, device=self.device)

    def forward(self, A, gather=False, group=None, gemm=None):
        """A: fp16 [m, k] replicated on every rank.  Returns this rank's columns [m, n/G], or with
        gather=True the full [m, n] on every rank.  `gemm(A, B, C, s, workspace)` defaults to the CUDA
        operator; the CPU tests pass a stand-in, since there is no CPU implementation of the operator."""
        m = A.shape[0]
        C = torch.empty((m, self.n_local), dtype=torch.half, device=A.device)
        (gemm or marlin.mul)(A, self.B, C, self.s, self.workspace)
        if not gather:
            return C
        return all_gather_columns(C, self.world, group)


def all_gather_columns(C_local, world, group=None):
    """[m, n/G] per rank -> [m, n] on every rank (rank r's columns at r*n/G)."""
    if world == 1:
        return C_local
    m, nl = C_local.shape
    stacked = torch.empty((world * m, nl), dtype=C_local.dtype, device=C_local.device)   # rank-major rows
    dist.all_gather_into_tensor(stacked, C_local.contiguous(), group=group)
    return stacked.view(world, m, nl).permute(1, 0, 2).reshape(m, world * nl)
