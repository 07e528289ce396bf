"""ctypes binding of libornith_cuda.so.

The library is the product; this module only declares its C ABI
(include/ornith_cuda.h) to Python.  Loading fails loudly when the shared object
is missing — there is no Python or CPU stand-in for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libornith_cuda.so")

ORNITH_OK = 0
ORNITH_ERR_BACKEND = 6
ACT_F32, ACT_BF16 = 0, 1
KV_F32, KV_INT8_HEAD, KV_Q8_0 = 0, 1, 2
HEADMAP_TILED, HEADMAP_GROUPED = 0, 1

f32p = C.POINTER(C.c_float)
i8p = C.POINTER(C.c_int8)
vp = C.c_void_p


class KvCache(C.Structure):                 # ornith_kv_cache (tier 1)
    _fields_ = [("K", f32p), ("V", f32p), ("Kq", i8p), ("Vq", i8p), ("Ks", f32p), ("Vs", f32p),
                ("quantized", C.c_int), ("capacity", C.c_int), ("len", C.c_int),
                ("n_kv_heads", C.c_int), ("head_dim", C.c_int)]


class DeltaState(C.Structure):              # ornith_delta_state
    _fields_ = [("S", f32p), ("dk", C.c_int), ("dv", C.c_int)]


class ConvState(C.Structure):               # ornith_conv_state
    _fields_ = [("buf", f32p), ("K", C.c_int), ("C", C.c_int)]


class CudaQproj(C.Structure):
    """ornith_cuda_qproj: one projection of a grouped launch."""
    _fields_ = [("wtype", C.c_int), ("W", C.c_void_p), ("n_out", C.c_int), ("y", C.c_void_p)]


class CudaKv(C.Structure):                  # ornith_cuda_kv
    _fields_ = [("mode", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("n_seq", C.c_int32),
                ("K", vp), ("V", vp), ("Ks", vp), ("Vs", vp), ("seq_off", vp)]


class CudaFullLayer(C.Structure):           # ornith_cuda_full_layer
    _fields_ = [("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("rope_dim", C.c_int32), ("gated", C.c_int32), ("eps", C.c_float), ("scale", C.c_float),
                ("q_norm_w", vp), ("k_norm_w", vp), ("rope_inv_freq", vp)]


class CudaLinearLayer(C.Structure):         # ornith_cuda_linear_layer
    _fields_ = [("nk", C.c_int32), ("nv", C.c_int32), ("dk", C.c_int32), ("dv", C.c_int32),
                ("conv_k", C.c_int32), ("head_map", C.c_int32), ("out_scale", C.c_float), ("eps", C.c_float),
                ("conv_w", vp), ("conv_b", vp), ("a_coef", vp), ("dt_bias", vp), ("norm_w", vp)]


class CudaShard(C.Structure):               # ornith_cuda_shard
    _fields_ = [(n, C.c_int32) for n in ("rank", "world", "v_head0", "n_v_heads", "k_head0", "n_k_heads",
                                          "q_head0", "n_q_heads", "kv_head0", "n_kv_heads")]


class CudaLinearState(C.Structure):         # ornith_cuda_linear_state
    _fields_ = [("S", vp), ("conv", vp), ("S_seq_stride", C.c_int64), ("conv_seq_stride", C.c_int64)]


# every symbol include/ornith_cuda.h declares: name -> (restype, argtypes)
_I, _F, _SZ = C.c_int, C.c_float, C.c_size_t
SYMBOLS = {
    "ornith_backend_cuda_available": (_I, []),
    "ornith_last_error": (C.c_char_p, []),
    "ornith_set_error": (None, None),
    # tier 1
    "ornith_kv_init": (_I, [vp, _I, _I, _I]),
    "ornith_kv_init_ex": (_I, [vp, _I, _I, _I, _I]),
    "ornith_kv_bytes_per_token": (_SZ, [_I, _I, _I]),
    "ornith_kv_free": (None, [vp]),
    "ornith_kv_reset": (None, [vp]),
    "ornith_gqa_step": (None, [vp, f32p, f32p, f32p, _I, f32p, _F]),
    "ornith_gqa_reference": (None, [f32p, f32p, f32p, _I, _I, _I, _I, f32p, _F]),
    "ornith_delta_init": (_I, [vp, _I, _I]),
    "ornith_delta_free": (None, [vp]),
    "ornith_delta_reset": (None, [vp]),
    "ornith_delta_step": (None, [vp, f32p, f32p, f32p, _F, _F, f32p]),
    "ornith_delta_prefill": (None, [vp, f32p, f32p, f32p, f32p, f32p, _I, _I, f32p]),
    "ornith_conv_init": (_I, [vp, _I, _I]),
    "ornith_conv_free": (None, [vp]),
    "ornith_conv_reset": (None, [vp]),
    "ornith_conv_step": (None, [vp, f32p, f32p, f32p, f32p]),
    "ornith_conv_prefill": (None, [vp, f32p, f32p, f32p, _I, f32p]),
    # tier 2
    "ornith_cuda_last_error": (C.c_char_p, []),
    "ornith_cuda_set_device": (_I, [_I]),
    "ornith_cuda_malloc": (_I, [C.POINTER(vp), _SZ]),
    "ornith_cuda_free": (_I, [vp]),
    "ornith_cuda_memset": (_I, [vp, _I, _SZ]),
    "ornith_cuda_h2d": (_I, [vp, vp, _SZ]),
    "ornith_cuda_d2h": (_I, [vp, vp, _SZ]),
    "ornith_cuda_sync": (_I, [vp]),
    "ornith_cuda_poll_status": (_I, []),
    "ornith_cuda_selftest_wait_timeout": (_I, [_I]),
    "ornith_cuda_set_alloc_hook": (None, [vp, vp]),
    "ornith_cuda_stream_release": (_I, [vp, _I]),
    "ornith_cuda_rope_inv_freq": (None, [_F, _I, f32p]),
    "ornith_cuda_q8_0_encode": (_I, [vp, vp, _SZ, vp]),
    "ornith_cuda_q8_0_decode": (_I, [vp, vp, _SZ, vp]),
    "ornith_cuda_full_attn_step_scratch": (_SZ, [vp, _I, _I]),
    "ornith_cuda_full_attn_step": (_I, [vp, vp, vp, vp, vp, vp, vp, vp, _I, _I, vp, _SZ, vp]),
    "ornith_cuda_full_attn_step_static": (_I, [vp, vp, vp, vp, vp, vp, vp, vp, _I, _I, vp]),
    "ornith_cuda_full_attn_prefill_scratch": (_SZ, [vp, _I, _I, _I]),
    "ornith_cuda_full_attn_prefill": (_I, [vp, vp, vp, vp, vp, vp, vp, vp, _I, _I, _I, vp, _SZ, vp]),
    "ornith_cuda_kv_append": (_I, [vp, vp, vp, vp, vp, vp, _I, _I, vp]),
    "ornith_cuda_advance": (_I, [vp, _I, _I, vp]),
    "ornith_cuda_head_shard": (_I, [_I, _I, _I, _I, _I, _I, vp]),
    "ornith_cuda_gather_layout": (_I, [vp, vp, _I, _SZ, _I, _I, vp]),
    "ornith_cuda_qproj_scratch": (_SZ, [_I, _I]),
    "ornith_cuda_q8k_quantize": (_I, [vp, _I, _I, _I, vp, vp, _SZ, vp]),
    "ornith_cuda_matmul_q8_0": (_I, [vp, _I, _I, vp, _I, _I, vp, _I, vp, _SZ, vp]),
    "ornith_cuda_matmul_q_scratch": (_SZ, [_I, _I, _I]),
    "ornith_cuda_matmul_q": (_I, [_I, vp, _I, _I, vp, _I, _I, vp, _I, vp, _SZ, vp]),
    "ornith_cuda_q8k_image": (_I, [vp, _I, _I, _I, vp, _SZ, vp]),
    "ornith_cuda_matmul_q_image": (_I, [_I, vp, _I, _I, vp, _I, vp, _I, vp]),
    "ornith_cuda_matmul_q_group": (_I, [vp, _I, _I, vp, _I, _I, vp]),
    "ornith_cuda_engine_new": (vp, [_I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I, _I, _I, _I]),
    "ornith_cuda_engine_free": (None, [vp]),
    "ornith_cuda_engine_full_layer": (_I, [vp, _I, vp, vp]),
    "ornith_cuda_engine_linear_layer": (_I, [vp, _I, vp, vp, vp, vp]),
    "ornith_cuda_engine_full_attn": (_I, [vp, _I, _I, _I, vp, vp, vp, vp]),
    "ornith_cuda_engine_linear_attn": (_I, [vp, _I, _I, _I, vp, vp, vp, vp, vp]),
    "ornith_cuda_engine_record_bytes": (_SZ, [vp, _I, _I]),
    "ornith_cuda_engine_export": (_I, [vp, _I, _I, vp, _SZ]),
    "ornith_cuda_engine_import": (_I, [vp, _I, _I, vp, _SZ]),
    "ornith_cuda_kv_record_bytes": (_SZ, [vp, _I]),
    "ornith_cuda_kv_export": (_I, [vp, _I, _I, vp, _SZ, vp]),
    "ornith_cuda_kv_import": (_I, [vp, _I, vp, _SZ, vp, vp, vp]),
    "ornith_cuda_linear_record_bytes": (_SZ, [vp]),
    "ornith_cuda_linear_export": (_I, [vp, vp, _I, _I, vp, _SZ, vp]),
    "ornith_cuda_linear_import": (_I, [vp, vp, _I, _I, vp, _SZ, vp]),
    "ornith_cuda_linear_attn_step": (_I, [vp, vp, vp, vp, vp, vp, vp, vp, _I, _I, vp]),
    "ornith_cuda_linear_attn_prefill_scratch": (_SZ, [vp, _I, _I]),
    "ornith_cuda_linear_attn_prefill": (_I, [vp, vp, vp, vp, vp, vp, vp, vp, _I, _I, _I, _I, vp, _SZ, vp]),
    "ornith_cuda_conv_export": (_I, [vp, _I, _I, _I, vp, vp]),
    "ornith_cuda_conv_import": (_I, [vp, _I, _I, _I, vp, vp]),
    "ornith_cuda_delta_step": (_I, [vp, _I, _I, _I, vp, vp, vp, vp, vp, vp, vp]),
    "ornith_cuda_delta_prefill": (_I, [vp, _I, _I, vp, vp, vp, vp, vp, _I, _I, vp, vp]),
    "ornith_cuda_conv_image": (_I, [vp, _I, _I, vp, vp, vp, _I, vp, vp]),
}

_lib = None


class BackendError(RuntimeError):
    pass


def load() -> C.CDLL:
    """Load libornith_cuda.so and declare its ABI.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BackendError(
            f"{LIB_PATH} is missing: build it with `python -m ornithology_b200.build`. "
            "There is no CPU fallback for the attention path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)             # AttributeError = ABI drift, let it surface
        fn.restype = res
        if args is not None:
            fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str = "") -> None:
    if status != ORNITH_OK:
        msg = load().ornith_cuda_last_error().decode(errors="replace")
        raise BackendError(f"{what or 'ornith_cuda call'} failed with status {status}: {msg}")
