"""ctypes binding of ``lib/libffb200.so`` (the sm_100a kernels).

The library is plain C ABI: raw device pointers, sizes and a stream handle.  It
is loaded lazily; on a machine with a GPU a missing or stale library is an
error (the CUDA path must never silently degrade to PyTorch composites), on a
CPU-only machine the ops use their PyTorch reference implementations and this
module is never asked for the library.
"""
import ctypes
import os
import threading

import torch

from .. import _build

_lock = threading.Lock()
_lib = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float

ACT_NONE, ACT_RELU, ACT_SIGMOID = 0, 1, 2
OUT_BF16, OUT_F32, OUT_F32_ATOMIC = 0, 1, 2


class GemmArgs(ctypes.Structure):
    """Mirror of ``struct GemmArgs`` in csrc/gemm_api.h."""
    _fields_ = [
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("splits", c_int), ("kblocks_per_split", c_int),
        ("out_mode", c_int), ("trans_out", c_int), ("act", c_int), ("glu", c_int),
        ("dm_div", c_int), ("dm_mod", c_int), ("a_zmul", c_int), ("b_zmul", c_int),
        ("alpha", c_float),
        ("C", c_void_p), ("ldc", c_ll), ("c_bstride", c_ll),
        ("bias", c_void_p),
        ("rowscale", c_void_p), ("rs_bstride", c_ll),
        ("mul", c_void_p), ("ldmul", c_ll), ("mul_bstride", c_ll),
        ("dmask", c_void_p), ("lddm", c_ll),
        ("resid", c_void_p), ("ldres", c_ll), ("res_bstride", c_ll),
        ("peer_slab", c_int),
        ("cq", c_int), ("cq_mdiv", c_int), ("cq_sr2", c_ll), ("cq_sr1", c_ll), ("cq_sc1", c_ll),
    ]


def _declare(lib):
    P, I, L, F = c_void_p, c_int, c_ll, c_float
    sig = {
        "ffb_gemm_bf16": [P, P, I, I, L, L, L, L, I, I, ctypes.POINTER(GemmArgs), P],
        "ffb_gemm_bf16_peer": [P, P, I, I, L, L, L, L, I, ctypes.POINTER(GemmArgs), I, ctypes.POINTER(c_void_p), I, P],
        "ffb_read_status": [ctypes.POINTER(c_int), I],
        "ffb_attention_fwd": [P, P, P, L, L, L, L, P, P, L, P, L, L, P, I, I, I, I, I, F, P],
        "ffb_attention_bwd": [P, P, P, L, L, L, L, P, P, L, P, P, P, P, P, I, I, I, I, I, F, P],
        "ffb_attention_bwd_strided": [P, P, P, L, L, L, L, P, P, L, P, P, L, L, P, P, P, P, L, L, L, L, P, I, I, I, I, I, F, P],
        "ffb_layernorm_fwd": [P, P, P, P, P, P, L, I, F, I, P],
        "ffb_layernorm_bwd": [P, P, P, P, P, P, P, I, P, P, L, I, I, P],
        "ffb_layernorm_bwd_acc": [P, P, P, P, P, P, P, I, P, P, L, I, P],
        "ffb_layernorm_fwd_transposed": [P, P, P, P, P, P, L, I, F, P],
        "ffb_layernorm_bwd_transposed": [P, P, P, P, P, P, P, P, P, L, I, P],
        "ffb_layernorm_bwd_transposed_acc": [P, P, P, P, P, P, P, P, P, L, I, P],
        "ffb_glu_mask_t_fwd": [P, P, P, I, L, P],
        "ffb_glu_mask_t_bwd": [P, P, P, P, I, L, P],
        "ffb_global_attention_fwd": [P, P, P, P, P, P, L, I, I, I, P],
        "ffb_recycle_pair_embed": [P, P, P, P, P, P, P, P, I, I, I, I, I, F, F, P],
        "ffb_softmax_fwd": [P, P, P, P, L, L, L, L, I, I, P],
        "ffb_softmax_bwd": [P, P, P, L, I, I, P],
        "ffb_bias_sigmoid_mul_fwd": [P, P, P, P, L, I, P],
        "ffb_bias_sigmoid_mul_bwd": [P, P, P, P, P, P, L, I, P],
        "ffb_bias_dropout_add_fwd": [P, P, P, P, P, L, I, I, I, P],
        "ffb_mask_mul": [P, P, P, L, I, I, I, P],
        "ffb_bias_ele_dropout_res_fwd": [P, P, P, P, P, P, L, I, I, I, P],
        "ffb_bias_ele_dropout_res_bwd": [P, P, P, P, P, P, P, L, I, I, I, P],
        "ffb_glu_mask_fwd": [P, P, P, P, L, I, P],
        "ffb_glu_mask_bwd": [P, P, P, P, P, P, L, I, P],
        "ffb_act_bwd": [P, P, P, L, I, I, P],
        "ffb_colsum": [P, P, L, I, P],
        "ffb_adam": [P, P, P, P, P, L, P, F, F, F, F, P],
    }
    for name, argtypes in sig.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
    return lib


def lib_path():
    return _build.lib_path()


def available():
    return os.path.exists(lib_path())


def get():
    """Returns the loaded library, building it first when a compiler is at hand."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not available():
                try:
                    _build.build(verbose=False)
                except Exception as e:  # no nvcc on the box
                    raise RuntimeError(
                        "fastfold_b200: native library %s is missing and could not be built (%s). "
                        "Run `python -m fastfold_b200._build` on a machine with nvcc." % (lib_path(), e))
            _lib = _declare(ctypes.CDLL(lib_path()))
    return _lib


def has(name):
    return hasattr(get(), name)


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def dtype_code(dt):
    return _DT[dt]


LAUNCHES = [0]   # number of native launcher calls made through this module (bench.py reports it)


def check(code, what):
    LAUNCHES[0] += 1
    if code != 0:
        raise RuntimeError("fastfold_b200 kernel launch failed: %s returned %d" % (what, code))


def read_status(clear=True):
    """Device status word: ``[code, blockIdx.x, blockIdx.y, blockIdx.z, detail, ...]``.

    ``code != 0`` means a kernel gave up on a bounded wait (see csrc/common.cuh).
    Synchronises the device.
    """
    out = (c_int * 8)()
    check(get().ffb_read_status(out, 1 if clear else 0), "ffb_read_status")
    return list(out)


def raise_on_status():
    st = read_status()
    if st[0] != 0:
        raise RuntimeError("fastfold_b200 device status %s (code, block x/y/z, detail)" % st[:5])
