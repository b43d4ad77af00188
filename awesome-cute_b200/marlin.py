"""Host-side mirror of the reference's Python surface for the W4A16 path
(gemm/marlin_gemm/marlin.py: ``mul`` :11-24, ``Layer`` :60-131) on top of the C ABI.

Same names, argument meaning and error behaviour; torch is used only to hold device memory and to
name the current stream.  The arithmetic is in libw4a16.so: the sm_100a kernel for ``mul``, the C++
packer for ``Layer.pack``.
"""
import ctypes

import numpy as np
import torch
import torch.nn as nn

from . import _lib

_L = _lib.lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _check(err, prob_m, prob_n, prob_k, thread_k, thread_n, groupsize):
    # the messages of gemm/marlin_gemm/marlin_gemm.cpp:48-55
    if err == _lib.ERR_PROB_SHAPE:
        raise RuntimeError("Problem (m=%d, n=%d, k=%d) not compatible with thread_k=%d, thread_n=%d."
                           % (prob_m, prob_n, prob_k, thread_k, thread_n))
    if err == _lib.ERR_KERN_SHAPE:
        raise RuntimeError("No kernel implementation for thread_k=%d, thread_n=%d, groupsize=%d."
                           % (thread_k, thread_n, groupsize))
    if err != _lib.OK:
        raise RuntimeError("w4a16_marlin_gemm failed with code %d: %s" % (err, _lib.last_cuda_error()))


def mul(A, B, C, s, workspace, thread_k=-1, thread_n=-1, sms=-1, max_par=16, cute_version=True, _entry=None):
    """Marlin FP16xINT4 multiply (reference: marlin.py:11-24 -> marlin_gemm.cpp:19-56).
    @A: `torch.half` input matrix of shape `(m, k)` in standard row-major layout
    @B: `torch.int` weight matrix of original shape `(k, n)` in Marlin format; see `Layer.pack()`
    @C: `torch.half` out matrix of shape `(m, n)` in standard row-major layout
    @s: `torch.half` scales of shape `(k / groupsize, n)`
    @workspace: `torch.int` tensor with at least `n / 128 * max_par` entries that are all zero
    @thread_k, @thread_n, @sms, @max_par: as in the reference; -1 = automatic
    @cute_version: accepted for signature compatibility; there is one kernel here
    """
    prob_m, prob_k = A.shape[0], A.shape[1]
    prob_n = C.shape[1]
    groupsize = -1 if s.shape[0] == 1 else prob_k // s.shape[0]
    if groupsize != -1 and groupsize * s.shape[0] != prob_k:
        raise RuntimeError("k=%d not compatible with %d groups." % (prob_k, s.shape[0]))
    need = prob_n // 128 * max_par      # w4a16_workspace_ints, computed here to keep the call path short
    if workspace.numel() < need:
        raise RuntimeError("workspace must be of size at least %d." % need)
    if not A.is_cuda:
        raise RuntimeError("mul() needs CUDA tensors; there is no CPU implementation of this operator.")
    dev = A.get_device()
    fn = _entry or _L.w4a16_marlin_gemm
    if torch.cuda.current_device() == dev:
        err = fn(A.data_ptr(), B.data_ptr(), C.data_ptr(), s.data_ptr(), prob_m, prob_n, prob_k, workspace.data_ptr(),
                 groupsize, dev, torch.cuda.current_stream(dev).cuda_stream, thread_k, thread_n, sms, max_par)
    else:
        with torch.cuda.device(dev):
            err = fn(A.data_ptr(), B.data_ptr(), C.data_ptr(), s.data_ptr(), prob_m, prob_n, prob_k,
                     workspace.data_ptr(), groupsize, dev, torch.cuda.current_stream(dev).cuda_stream, thread_k,
                     thread_n, sms, max_par)
    if err:
        _check(err, prob_m, prob_n, prob_k, thread_k, thread_n, groupsize)


def mul_host(A_host, B, C_host, s, workspace, A_stage, C_stage, stream=None):
    """`mul` for HOST activations / outputs (pinned torch tensors): copy in, multiply, copy out, all enqueued
    on `stream` (a torch.cuda.Stream; default: the current stream of B's device) by one call into the library.  A_stage [m, k] and C_stage [m, n] are
    device staging tensors owned by the caller; B, s, workspace are device tensors as for `mul`.  Synchronise
    the stream before reading C_host."""
    prob_m, prob_k = A_host.shape
    prob_n = C_host.shape[1]
    groupsize = -1 if s.shape[0] == 1 else prob_k // s.shape[0]
    if groupsize != -1 and groupsize * s.shape[0] != prob_k:
        raise RuntimeError("k=%d not compatible with %d groups." % (prob_k, s.shape[0]))
    if workspace.numel() < prob_n // 128 * 16:
        raise RuntimeError("workspace must be of size at least %d." % (prob_n // 128 * 16))
    if A_host.is_cuda or C_host.is_cuda or not B.is_cuda:
        raise RuntimeError("mul_host() takes host activations/outputs and device weights.")
    dev = B.get_device()
    if torch.cuda.current_device() != dev:
        raise RuntimeError("device %d must be current" % dev)
    err = _L.w4a16_marlin_gemm_host(A_host.data_ptr(), B.data_ptr(), C_host.data_ptr(), s.data_ptr(), prob_m, prob_n,
                                    prob_k, workspace.data_ptr(), groupsize, dev,
                                    (stream if stream is not None else torch.cuda.current_stream(dev)).cuda_stream,
                                    A_stage.data_ptr(), C_stage.data_ptr())
    if err:
        _check(err, prob_m, prob_n, prob_k, -1, -1, groupsize)


class HostGemm:
    """`mul_host` with its arguments checked and converted once: a layer that is called every decode step with the
    same pinned host buffers pays the library call only (the checks and conversions of `mul_host` cost about as much
    as the call itself).  `op = HostGemm(A_host, B, C_host, s, workspace, A_stage, C_stage, stream)`, then `op()` per
    step: enqueues the copy of A_host to the device, the GEMM and the copy of the result into C_host on `stream`.
    The tensors must stay alive and in place while the object is used."""

    def __init__(self, A_host, B, C_host, s, workspace, A_stage, C_stage, stream=None):
        prob_m, prob_k = A_host.shape
        prob_n = C_host.shape[1]
        groupsize = -1 if s.shape[0] == 1 else prob_k // s.shape[0]
        if groupsize != -1 and groupsize * s.shape[0] != prob_k:
            raise RuntimeError("k=%d not compatible with %d groups." % (prob_k, s.shape[0]))
        if workspace.numel() < prob_n // 128 * 16:
            raise RuntimeError("workspace must be of size at least %d." % (prob_n // 128 * 16))
        if A_host.is_cuda or C_host.is_cuda or not B.is_cuda:
            raise RuntimeError("HostGemm takes host activations/outputs and device weights.")
        dev = B.get_device()
        st = stream if stream is not None else torch.cuda.current_stream(dev)
        self._keep = (A_host, B, C_host, s, workspace, A_stage, C_stage, st)
        self._shape = (prob_m, prob_n, prob_k, groupsize)
        self._dev = dev
        vp, ci = ctypes.c_void_p, ctypes.c_int
        self._args = (vp(A_host.data_ptr()), vp(B.data_ptr()), vp(C_host.data_ptr()), vp(s.data_ptr()), ci(prob_m), ci(prob_n),
                      ci(prob_k), vp(workspace.data_ptr()), ci(groupsize), ci(dev), vp(st.cuda_stream), vp(A_stage.data_ptr()),
                      vp(C_stage.data_ptr()))

    def __call__(self):
        err = _L.w4a16_marlin_gemm_host(*self._args)     # the library checks that the device is current
        if err:
            _check(err, self._shape[0], self._shape[1], self._shape[2], -1, -1, self._shape[3])


def mul_gather(A, B, s, workspace, dst_ptrs, rank):
    """Column-shard GEMM whose epilogue writes this rank's columns into every rank's [m, world * n_local] buffer
    (w4a16_marlin_gemm_gather).  dst_ptrs: device addresses of the `world` destination buffers as seen from this
    process (own buffer at index `rank`, peer-mapped ones elsewhere).  No counterpart in the reference."""
    prob_m, prob_k = A.shape
    n_local = B.shape[1] // 2
    groupsize = -1 if s.shape[0] == 1 else prob_k // s.shape[0]
    world = len(dst_ptrs)
    dev = A.get_device()
    if torch.cuda.current_device() != dev:
        raise RuntimeError("device %d must be current" % dev)
    arr = (ctypes.c_void_p * world)(*[int(p) for p in dst_ptrs])
    err = _L.w4a16_marlin_gemm_gather(A.data_ptr(), B.data_ptr(), s.data_ptr(), prob_m, n_local, prob_k,
                                      workspace.data_ptr(), groupsize, dev, torch.cuda.current_stream(dev).cuda_stream,
                                      arr, world, rank)
    if err:
        _check(err, prob_m, n_local, prob_k, -1, -1, groupsize)


def mul_simt(A, B, C, s, workspace, thread_k=-1, thread_n=-1, sms=-1, max_par=16):
    """Same call through the diagnostic CUDA-core kernel (tests only)."""
    mul(A, B, C, s, workspace, thread_k, thread_n, sms, max_par, _entry=_L.w4a16_marlin_gemm_simt)


def device_status(dev=None):
    """Synchronise the current stream of `dev`; raise if a kernel gave up a bounded wait."""
    dev = torch.cuda.current_device() if dev is None else dev
    err = _L.w4a16_device_status(dev, ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if err != _lib.OK:
        raise RuntimeError("w4a16 device status %d: %s" % (err, _lib.last_cuda_error()))


# ----------------------------------------------------------------------------- host packer (numpy in, numpy out)
def _np(a, dt):
    a = np.ascontiguousarray(a)
    if a.dtype != dt:
        raise TypeError("expected %s, got %s" % (dt, a.dtype))
    return a


def _vp(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def pack_weights(q):
    """uint8 codes [k, n] -> int32 [k/16, 2n] (marlin.py:119-129)."""
    q = _np(q, np.uint8)
    k, n = q.shape
    B = np.empty((k // 16, 2 * n), np.int32)
    err = _L.w4a16_pack_weights(_vp(q), k, n, _vp(B))
    if err:
        raise ValueError("w4a16_pack_weights: code %d" % err)
    return B


def unpack_weights(B, k, n):
    B = _np(B, np.int32)
    q = np.empty((k, n), np.uint8)
    err = _L.w4a16_unpack_weights(_vp(B), k, n, _vp(q))
    if err:
        raise ValueError("w4a16_unpack_weights: code %d" % err)
    return q


def permute_scales(s):
    """fp16 [groups, n] natural order -> kernel order (marlin.py:111-118)."""
    s = _np(s, np.float16)
    out = np.empty_like(s)
    err = _L.w4a16_permute_scales(_vp(s), s.shape[0], s.shape[1], _vp(out))
    if err:
        raise ValueError("w4a16_permute_scales: code %d" % err)
    return out


def unpermute_scales(sp):
    sp = _np(sp, np.float16)
    out = np.empty_like(sp)
    err = _L.w4a16_unpermute_scales(_vp(sp), sp.shape[0], sp.shape[1], _vp(out))
    if err:
        raise ValueError("w4a16_unpermute_scales: code %d" % err)
    return out


def quantize_pack(weight_nk, scales, groupsize):
    """All of Layer.pack on host arrays: weight fp16 [n, k] (nn.Linear layout), scales fp16 [groups, n]."""
    w = _np(weight_nk, np.float16)
    s = _np(scales, np.float16)
    n, k = w.shape
    groups = 1 if groupsize == -1 else k // groupsize
    B = np.empty((k // 16, 2 * n), np.int32)
    sp = np.empty((groups, n), np.float16)
    err = _L.w4a16_quantize_pack(_vp(w), _vp(s), k, n, groupsize, _vp(B), _vp(sp))
    if err:
        raise ValueError("w4a16_quantize_pack: code %d" % err)
    return B, sp


def shard_columns(B, s_packed, rank, world):
    """Column shard `rank` of `world` of a packed layer (B int32 [k/16, 2n], s_packed fp16 [groups, n])."""
    B = _np(B, np.int32)
    sp = _np(s_packed, np.float16)
    k, n = B.shape[0] * 16, B.shape[1] // 2
    groups = sp.shape[0]
    if world < 1 or n % world:
        raise ValueError("n=%d does not split over %d ranks" % (n, world))
    Bs = np.empty((k // 16, 2 * n // world), np.int32)
    ss = np.empty((groups, n // world), np.float16)
    err = _L.w4a16_shard_columns(_vp(B), _vp(sp), k, n, groups, rank, world, _vp(Bs), _vp(ss))
    if err:
        raise ValueError("w4a16_shard_columns: code %d" % err)
    return Bs, ss


class Layer(nn.Module):
    """4-bit (symmetric grouped) linear layer without bias (reference: marlin.py:60-131)."""

    def __init__(self, infeatures, outfeatures, groupsize=-1, cute_version=True):
        super().__init__()
        if groupsize not in [-1, 128]:
            raise ValueError('Only groupsize -1 and 128 are supported.')
        if infeatures % 128 != 0 or outfeatures % 256 != 0:
            raise ValueError('`infeatures` must be divisible by 128 and `outfeatures` by 256.')
        if groupsize == -1:
            groupsize = infeatures
        if infeatures % groupsize != 0:
            raise ValueError('`infeatures` must be divisible by `groupsize`.')
        self.k = infeatures
        self.n = outfeatures
        self.groupsize = groupsize
        self.cute_version = cute_version
        self.register_buffer('B', torch.empty((self.k // 16, self.n * 16 // 8), dtype=torch.int))
        self.register_buffer('s', torch.empty((self.k // groupsize, self.n), dtype=torch.half))
        self.register_buffer('workspace', torch.zeros(self.n // 128 * 16, dtype=torch.int), persistent=False)

    def forward(self, A):
        C = torch.empty(A.shape[:-1] + (self.s.shape[1],), dtype=A.dtype, device=A.device)
        mul(A.view((-1, A.shape[-1])), self.B, C.view((-1, C.shape[-1])), self.s, self.workspace)
        return C

    def pack(self, linear, scales):
        """Pack a fake-quantized linear layer (reference: marlin.py:92-131).
        @linear: fake-quantized `torch.nn.Linear` layer to convert (must be of type `torch.half`)
        @scales: corresponding quantization scales of shape `(infeatures, groups)`
        """
        if linear.weight.dtype != torch.half:
            raise ValueError('Only `torch.half` weights are supported.')
        w = linear.weight.data.detach().cpu().contiguous().numpy()          # [n, k]
        s = scales.detach().t().cpu().contiguous().numpy()                   # [groups, n]
        gs = -1 if self.groupsize == self.k else self.groupsize
        B, sp = quantize_pack(w, s, gs)
        self.B[:, :] = torch.from_numpy(B).to(self.B.device)
        self.s[:, :] = torch.from_numpy(sp).to(self.s.device)


# ----------------------------------------------------------------------------- device-side pack, files
def quantize_pack_device(weight_nk, scales, groupsize):
    """Layer.pack on the device: weight fp16 [n, k] (CUDA), scales fp16 [groups, n] (CUDA) -> (B int32 [k/16, 2n],
    s_packed fp16 [groups, n]) on the same device.  Bit-exact with quantize_pack()."""
    if not (weight_nk.is_cuda and scales.is_cuda):
        raise RuntimeError("quantize_pack_device() needs CUDA tensors")
    if weight_nk.dtype != torch.half or scales.dtype != torch.half:
        raise ValueError('Only `torch.half` weights and scales are supported.')
    weight_nk, scales = weight_nk.contiguous(), scales.contiguous()
    n, k = weight_nk.shape
    groups = 1 if groupsize == -1 else k // groupsize
    B = torch.empty((k // 16, 2 * n), dtype=torch.int, device=weight_nk.device)
    sp = torch.empty((groups, n), dtype=torch.half, device=weight_nk.device)
    dev = weight_nk.get_device()
    with torch.cuda.device(dev):
        err = _L.w4a16_quantize_pack_device(weight_nk.data_ptr(), scales.data_ptr(), k, n, groupsize, B.data_ptr(),
                                            sp.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    if err:
        raise ValueError("w4a16_quantize_pack_device: code %d" % err)
    return B, sp


def save_packed(path, B, s_packed):
    """Write a packed layer (numpy B int32 [k/16, 2n], s_packed fp16 [groups, n]) to a file."""
    B, sp = _np(B, np.int32), _np(s_packed, np.float16)
    k, n = B.shape[0] * 16, B.shape[1] // 2
    groupsize = -1 if sp.shape[0] == 1 else k // sp.shape[0]
    err = _L.w4a16_blob_write(str(path).encode(), _vp(B), _vp(sp), k, n, groupsize)
    if err:
        raise ValueError("w4a16_blob_write: code %d" % err)


def load_packed(path, rank=0, world=1):
    """Read a packed layer, or column shard `rank` of `world` of it, from a file -> (B, s_packed, groupsize)."""
    k, n, gs, groups = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    err = _L.w4a16_blob_info(str(path).encode(), ctypes.byref(k), ctypes.byref(n), ctypes.byref(gs), ctypes.byref(groups))
    if err:
        raise ValueError("w4a16_blob_info: code %d" % err)
    if world < 1 or n.value % world:
        raise ValueError("n=%d does not split over %d ranks" % (n.value, world))
    B = np.empty((k.value // 16, 2 * n.value // world), np.int32)
    sp = np.empty((groups.value, n.value // world), np.float16)
    err = _L.w4a16_blob_read(str(path).encode(), rank, world, _vp(B), _vp(sp))
    if err:
        raise ValueError("w4a16_blob_read: code %d" % err)
    return B, sp, gs.value
