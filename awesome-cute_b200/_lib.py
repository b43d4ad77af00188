"""ctypes door onto libw4a16.so (the C ABI declared in include/w4a16.h).

There is no Python or CPU implementation behind this module: if the shared library has not been
built (``python -c "import __graft_entry__ as g; g.build()"`` or ``make -C awesome-cute_b200/csrc``)
importing it raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("W4A16_LIB") or os.path.join(_HERE, "libw4a16.so")   # W4A16_LIB: debugging override

OK, ERR_PROB_SHAPE, ERR_KERN_SHAPE, ERR_CUDA, ERR_TIMEOUT, ERR_ARG = 0, 1, 2, 3, 4, 5

# every symbol include/w4a16.h declares: name -> (restype, argtypes)
_vp, _i = ctypes.c_void_p, ctypes.c_int
_GEMM_ARGS = [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _i, _i, _i]
SYMBOLS = {
    "w4a16_marlin_gemm": (_i, _GEMM_ARGS),
    "w4a16_marlin_gemm_simt": (_i, _GEMM_ARGS),
    "w4a16_marlin_gemm_builtin_scratch": (_i, _GEMM_ARGS),
    "w4a16_marlin_gemm_host": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp]),
    "w4a16_workspace_ints": (_i, [_i, _i]),
    "w4a16_device_status": (_i, [_i, _vp]),
    "w4a16_release_stream": (_i, [_i, _vp]),
    "w4a16_plan": (_i, [_i, _i, _i, _i, _i, _i, _vp]),
    "w4a16_selftest_unanswered_wait": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i]),
    "w4a16_last_cuda_error": (ctypes.c_char_p, []),
    "w4a16_pack_weights": (_i, [_vp, _i, _i, _vp]),
    "w4a16_unpack_weights": (_i, [_vp, _i, _i, _vp]),
    "w4a16_permute_scales": (_i, [_vp, _i, _i, _vp]),
    "w4a16_unpermute_scales": (_i, [_vp, _i, _i, _vp]),
    "w4a16_quantize_pack": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "w4a16_shard_columns": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "w4a16_quantize_pack_device": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "w4a16_blob_write": (_i, [ctypes.c_char_p, _vp, _vp, _i, _i, _i]),
    "w4a16_blob_info": (_i, [ctypes.c_char_p, ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "w4a16_blob_read": (_i, [ctypes.c_char_p, _i, _i, _vp, _vp]),
    "w4a16_marlin_gemm_gather": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _vp, ctypes.POINTER(_vp), _i, _i]),
    "w4a16_peer_alloc": (_i, [ctypes.c_size_t, ctypes.POINTER(_vp), _vp]),
    "w4a16_peer_open": (_i, [_vp, ctypes.POINTER(_vp)]),
    "w4a16_peer_close": (_i, [_vp]),
    "w4a16_peer_free": (_i, [_vp]),
    "w4a16_peer_barrier": (_i, [ctypes.POINTER(_vp), _i, _i, _i, _vp, _i]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libw4a16.so is not built (%s). Build it with `make -C awesome-cute_b200/csrc`; "
            "there is no fallback implementation." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError here means the library does not match the header
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class Plan(ctypes.Structure):
    """w4a16_plan_t of include/w4a16.h"""
    _fields_ = [(n, _i) for n in ("kernel", "tile_rows", "k_per_stage", "workers", "ctas_per_worker", "whole_tile_waves",
                                  "stages_per_worker")]


KERNEL_NAMES = {0: "none", 1: "single", 2: "pairs", 3: "decode", 4: "decode_cluster"}


def plan(m, n, k, groupsize=128, sms=-1, device_sms=148):
    """Which kernel `mul` would launch for these sizes on a device of `device_sms` SMs and how the work is cut
    (w4a16_plan: host arithmetic only, works without a GPU).  Returns (return code, dict)."""
    out = Plan()
    rc = lib.w4a16_plan(m, n, k, groupsize, sms, device_sms, ctypes.byref(out))
    d = {f: getattr(out, f) for f, _ in Plan._fields_}
    d["kernel"] = KERNEL_NAMES.get(d["kernel"], d["kernel"])
    return rc, d


def last_cuda_error():
    return lib.w4a16_last_cuda_error().decode()
