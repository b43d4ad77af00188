"""Column-sharded W4A16 layers: each rank of a process group owns N/G output columns of a packed layer.

The reference is single-GPU; this is the only multi-GPU piece.  A column shard is a pure slice of the
packed operands (both Marlin permutations are local to 64-column blocks, gemm/marlin_gemm/marlin.py:29-57),
so every rank runs the unchanged GEMM on its slice and there is no reduction between GPUs.  The one
exchange step, used only when the caller asks for the full output row, is an all-gather of the fp16
outputs along N.  Two forms: a plain all-gather (NCCL over NVLink on GPUs, gloo in the CPU tests), and the
gathering epilogue, where the GEMM kernel itself stores every finished tile into all ranks' output buffers
over peer-mapped memory (`GatherBuffers`, `ColumnShardedLayer.forward_gathered`), followed by a one-warp
barrier kernel instead of a collective.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import _lib, marlin

_L = _lib.lib


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

    def forward_gathered(self, A, bufs, barrier=True):
        """Full [m, n] output on every rank without a collective: the GEMM's epilogue stores this rank's columns
        into every rank's buffer of `bufs` (a GatherBuffers), then the barrier kernel orders the ranks.  The
        returned tensor is a view of bufs.local; it is overwritten by the next call with the same `bufs`, which
        must not be issued before every rank has consumed this result (barrier, or alternate two GatherBuffers)."""
        m = A.shape[0]
        if m > bufs.m_max or bufs.n != self.n or bufs.world != self.world:
            raise ValueError("GatherBuffers do not fit this layer / batch")
        marlin.mul_gather(A, self.B, self.s, self.workspace, bufs.dst_ptrs, self.rank)
        if barrier:
            bufs.barrier()
        return bufs.local[:m]


class _RawDeviceArray:
    """Lets torch view device memory that this library allocated (CUDA array interface, version 2)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}


class GatherBuffers:
    """One fp16 [m_max, n] output buffer per rank, each mapped into every other rank's process, plus the flag
    blocks of the barrier.  Collective over `group` (handles travel by all_gather_object); the rank's device must
    be current.  `local` is this rank's buffer as a torch tensor; after `barrier()` it holds all ranks' columns."""

    def __init__(self, m_max, n, rank, world, device, group=None):
        self.rank, self.world, self.m_max, self.n = rank, world, m_max, n
        self.device = torch.device(device)
        self.dev = self.device.index if self.device.index is not None else (torch.cuda.current_device() if torch.cuda.is_available() else 0)
        data_bytes = (m_max * n * 2 + 255) // 256 * 256
        self._bytes = data_bytes + 64
        base = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        err = _L.w4a16_peer_alloc(self._bytes, ctypes.byref(base), handle)
        self._own = base.value if not err else None
        self._opened = []
        handles = [None] * world
        if world > 1:   # every rank takes part in the exchange, also one whose allocation failed
            dist.all_gather_object(handles, None if err else handle.raw, group=group)
        self._check(err, "w4a16_peer_alloc")
        if any(h is None for r, h in enumerate(handles) if r != rank):
            _L.w4a16_peer_free(self._own)
            self._own = None
            raise RuntimeError("a peer rank could not allocate its gather buffer")
        bases = []
        for r in range(world):
            if r == rank:
                bases.append(self._own)
                continue
            p = ctypes.c_void_p()
            self._check(_L.w4a16_peer_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(p)),
                        "w4a16_peer_open")
            self._opened.append(p.value)
            bases.append(p.value)
        self.dst_ptrs = bases
        self._flags = (ctypes.c_void_p * world)(*[b + data_bytes for b in bases])
        self.local = torch.as_tensor(_RawDeviceArray(self._own, (m_max, n), "<f2"), device=self.device)

    @staticmethod
    def _check(err, what):
        if err:
            raise RuntimeError("%s failed with code %d: %s" % (what, err, _lib.last_cuda_error()))

    def barrier(self, limit_ms=2000):
        """Enqueue the cross-GPU barrier on the current stream (w4a16_peer_barrier)."""
        self._check(_L.w4a16_peer_barrier(self._flags, self.world, self.rank, self.dev,
                                          torch.cuda.current_stream(self.dev).cuda_stream, limit_ms),
                    "w4a16_peer_barrier")

    def close(self, group=None):
        """Unmap the peers' buffers, then (after every rank has unmapped) free the own one."""
        torch.cuda.synchronize(self.dev)
        for p in self._opened:
            _L.w4a16_peer_close(p)
        self._opened = []
        if self.world > 1:
            dist.barrier(group=group)
        if self._own:
            self.local = None
            _L.w4a16_peer_free(self._own)
            self._own = None


def all_gather_columns(C_local, world, group=None):
    """[m, n/G] per rank -> [m, n] on every rank (rank r's columns at r*n/G)."""
    if world == 1:
        return C_local
    m, nl = C_local.shape
    stacked = torch.empty((world * m, nl), dtype=C_local.dtype, device=C_local.device)   # rank-major rows
    dist.all_gather_into_tensor(stacked, C_local.contiguous(), group=group)
    return stacked.view(world, m, nl).permute(1, 0, 2).reshape(m, world * nl)
