"""ctypes front-end to the CPU checkers (TEST INFRASTRUCTURE ONLY).

Two libraries are wrapped:

* ``liboracle.so``  — the restatement in ``ornith_oracle.c`` (class :class:`Oracle`);
* ``_ref/libornith_ref.so`` — the reference's own objects, when they were built
  from a reference checkout (class :class:`Ref`).  It mirrors the C structs of the
  reference's ``src/ornith_attn.h:57-136`` so the reference functions can be
  driven directly.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libornith_ref.so")

KV_F32, KV_INT8_HEAD, KV_Q8_0 = 0, 1, 2
HEADMAP_TILED, HEADMAP_GROUPED = 0, 1
# weight types with an integer dot against Q8_K activations (ids as in the GGUF file, src/ornith_gguf.h:24-30)
GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 8, 12, 14
QROW_BYTES = {GGML_Q8_0: lambda n: n // 32 * 34, GGML_Q4_K: lambda n: n // 256 * 144, GGML_Q6_K: lambda n: n // 256 * 210}

_f32p = C.POINTER(C.c_float)


def _fp(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(_f32p)


def build(force: bool = False) -> None:
    """Compile liboracle.so (and _ref when a reference checkout is present)."""
    if force or not os.path.exists(ORACLE_SO) or \
            os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(_HERE, "ornith_oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)
    ref = os.environ.get("ORNITH_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"))
    if os.path.isdir(os.path.join(ref, "src")) and (force or not os.path.exists(REF_SO)):
        subprocess.check_call(["make", "-C", _HERE, "ref", f"REF={ref}"], stdout=subprocess.DEVNULL)


class _KV(C.Structure):
    _fields_ = [("mode", C.c_int), ("capacity", C.c_int), ("len", C.c_int),
                ("n_kv_heads", C.c_int), ("head_dim", C.c_int),
                ("K", _f32p), ("V", _f32p),
                ("Kq", C.POINTER(C.c_int8)), ("Vq", C.POINTER(C.c_int8)),
                ("Ks", _f32p), ("Vs", _f32p),
                ("Kb", C.POINTER(C.c_uint8)), ("Vb", C.POINTER(C.c_uint8))]


class _LinearParams(C.Structure):
    _fields_ = [("nk", C.c_int), ("nv", C.c_int), ("dk", C.c_int), ("dv", C.c_int),
                ("conv_k", C.c_int), ("head_map", C.c_int),
                ("out_scale", C.c_float), ("eps", C.c_float),
                ("conv_w", _f32p), ("conv_b", _f32p), ("a_coef", _f32p),
                ("dt_bias", _f32p), ("norm_w", _f32p)]


class _FullParams(C.Structure):
    _fields_ = [("nh", C.c_int), ("nkv", C.c_int), ("hd", C.c_int), ("rope_dim", C.c_int),
                ("theta", C.c_float), ("eps", C.c_float),
                ("q_norm_w", _f32p), ("k_norm_w", _f32p)]


class LinearLayer:
    """Host-side description of one gated delta-net layer (weights as float32 arrays)."""

    def __init__(self, nk, nv, dk, dv, conv_w, a_coef, dt_bias, norm_w, conv_b=None,
                 conv_k=4, head_map=HEADMAP_TILED, out_scale=None, eps=1e-6):
        self.nk, self.nv, self.dk, self.dv, self.conv_k = nk, nv, dk, dv, conv_k
        self.head_map, self.eps = head_map, eps
        self.out_scale = float(np.float32(1.0) / np.sqrt(np.float32(dk))) if out_scale is None else out_scale
        self.conv_w = np.ascontiguousarray(conv_w, np.float32)
        self.conv_b = None if conv_b is None else np.ascontiguousarray(conv_b, np.float32)
        self.a_coef = np.ascontiguousarray(a_coef, np.float32)
        self.dt_bias = np.ascontiguousarray(dt_bias, np.float32)
        self.norm_w = np.ascontiguousarray(norm_w, np.float32)
        self.qd, self.vd = nk * dk, nv * dv
        self.cc = 2 * self.qd + self.vd
        assert self.conv_w.shape == (self.cc, conv_k)

    def c_struct(self):
        return _LinearParams(self.nk, self.nv, self.dk, self.dv, self.conv_k, self.head_map,
                             self.out_scale, self.eps, _fp(self.conv_w), _fp(self.conv_b),
                             _fp(self.a_coef), _fp(self.dt_bias), _fp(self.norm_w))


class FullLayer:
    """Host-side description of one full-attention layer."""

    def __init__(self, nh, nkv, hd, q_norm_w, k_norm_w, rope_dim=64, theta=1e7, eps=1e-6):
        self.nh, self.nkv, self.hd, self.rope_dim = nh, nkv, hd, rope_dim
        self.theta, self.eps = theta, eps
        self.q_norm_w = np.ascontiguousarray(q_norm_w, np.float32)
        self.k_norm_w = np.ascontiguousarray(k_norm_w, np.float32)

    def c_struct(self):
        return _FullParams(self.nh, self.nkv, self.hd, self.rope_dim, self.theta, self.eps,
                           _fp(self.q_norm_w), _fp(self.k_norm_w))


class OracleKV:
    """A KV cache held by the oracle (f32, int8-per-head or Q8_0 rows)."""

    def __init__(self, lib, capacity, nkv, hd, mode):
        self._lib = lib
        self.c = _KV()
        if lib.orc_kv_init(C.byref(self.c), capacity, nkv, hd, mode) != 0:
            raise MemoryError("orc_kv_init failed")
        self.capacity, self.nkv, self.hd, self.mode = capacity, nkv, hd, mode

    @property
    def len(self):
        return self.c.len

    def _arr(self, ptr, shape, dtype):
        n = int(np.prod(shape))
        if n == 0:
            return np.zeros(shape, dtype)
        buf = (C.c_char * (n * np.dtype(dtype).itemsize)).from_address(C.addressof(ptr.contents))
        return np.frombuffer(buf, dtype=dtype).reshape(shape).copy()

    def rows_f32(self):
        """(K, V) rows attention reads, [len][nkv][hd] (F32 and Q8_0 modes)."""
        s = (self.len, self.nkv, self.hd)
        return self._arr(self.c.K, s, np.float32), self._arr(self.c.V, s, np.float32)

    def rows_q8_0(self):
        s = (self.len, self.nkv, self.hd // 32 * 34)
        return self._arr(self.c.Kb, s, np.uint8), self._arr(self.c.Vb, s, np.uint8)

    def rows_int8(self):
        s = (self.len, self.nkv, self.hd)
        t = (self.len, self.nkv)
        return (self._arr(self.c.Kq, s, np.int8), self._arr(self.c.Vq, s, np.int8),
                self._arr(self.c.Ks, t, np.float32), self._arr(self.c.Vs, t, np.float32))

    def free(self):
        self._lib.orc_kv_free(C.byref(self.c))

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Oracle:
    """numpy wrappers over liboracle.so."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = L = C.CDLL(path)
        L.orc_dot.restype = C.c_float
        L.orc_sigmoid.restype = C.c_float
        L.orc_silu.restype = C.c_float
        L.orc_softplus.restype = C.c_float
        for f in (L.orc_sigmoid, L.orc_silu, L.orc_softplus):
            f.argtypes = [C.c_float]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_kv_int8_encode.restype = C.c_float
        L.orc_rng_uniform.restype = C.c_float
        L.orc_rng_uniform.argtypes = [C.c_void_p, C.c_float, C.c_float]
        L.orc_rng_fill.argtypes = [C.c_void_p, _f32p, C.c_int64, C.c_float, C.c_float]
        L.orc_kv_bytes_per_token.restype = C.c_size_t
        L.orc_q8_0_encode.argtypes = [_f32p, C.c_void_p, C.c_size_t]
        L.orc_q8_0_decode.argtypes = [C.c_void_p, _f32p, C.c_size_t]
        L.orc_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_float]
        L.orc_l2norm_eps.argtypes = [_f32p, _f32p, C.c_int, C.c_float]
        L.orc_rope_partial.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_gqa_step.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, C.c_int, _f32p, C.c_float]
        L.orc_gqa_reference.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                        _f32p, C.c_float]
        L.orc_delta_step.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p,
                                     C.c_float, C.c_float, _f32p]
        L.orc_delta_prefill.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p,
                                        C.c_int, C.c_int, _f32p]
        L.orc_conv_step.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, _f32p]
        L.orc_conv_prefill.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, C.c_int, _f32p]
        L.orc_linear_attn_step.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.orc_linear_attn_prefill.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p,
                                              C.c_int, C.c_int, _f32p]
        L.orc_full_attn_step.argtypes = [C.c_void_p, C.c_void_p, C.c_int, _f32p, _f32p, _f32p, _f32p]
        L.orc_full_attn_prefill.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                            _f32p, _f32p, _f32p, _f32p]

    # -- rng -------------------------------------------------------------
    def rng_fill(self, seed, n, lo, hi, state=None):
        """n uniforms from the reference's splitmix64 stream; returns (array, state)."""
        st = C.c_uint64(seed) if state is None else state
        out = np.empty(n, np.float32)
        self.lib.orc_rng_fill(C.byref(st), _fp(out), n, lo, hi)
        return out, st

    # -- scalars / vectors -------------------------------------------------
    def sigmoid(self, x): return self.lib.orc_sigmoid(float(x))
    def silu(self, x): return self.lib.orc_silu(float(x))
    def softplus(self, x): return self.lib.orc_softplus(float(x))
    def f32_to_f16(self, x): return self.lib.orc_f32_to_f16(float(x))
    def f16_to_f32(self, h): return self.lib.orc_f16_to_f32(int(h))

    def rmsnorm(self, x, w, eps):
        x = np.ascontiguousarray(x, np.float32); out = np.empty_like(x)
        self.lib.orc_rmsnorm(_fp(x), _fp(w), _fp(out), x.size, eps)
        return out

    def l2norm_eps(self, x, eps):
        x = np.ascontiguousarray(x, np.float32); out = np.empty_like(x)
        self.lib.orc_l2norm_eps(_fp(x), _fp(out), x.size, eps)
        return out

    def softmax(self, x):
        x = np.array(x, np.float32)
        self.lib.orc_softmax(_fp(x), x.size)
        return x

    def rope_partial(self, v, rotary_dim, pos, theta):
        v = np.array(v, np.float32)
        self.lib.orc_rope_partial(_fp(v), v.size, rotary_dim, pos, theta)
        return v

    # -- quantised projections ----------------------------------------------
    def q8k_quantize(self, x):
        """f32 [..., k] (k a multiple of 256) -> Q8_K blocks as bytes [..., k/256, 292]."""
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[:-1] + (x.shape[-1] // 256, 292), np.uint8)
        self.lib.orc_q8k_quantize.argtypes = [_f32p, C.c_void_p, C.c_int64]
        self.lib.orc_q8k_quantize(_fp(x), out.ctypes.data, x.size)
        return out

    def matmul_q8_0(self, W, n_in, X):
        """Y [T][out] = X [T][n_in] through Q8_0 weight rows W (bytes [out][n_in/32*34]), the engine's integer path."""
        W = np.ascontiguousarray(W, np.uint8)
        X = np.ascontiguousarray(X, np.float32).reshape(-1, n_in)
        n_out = W.size // (n_in // 32 * 34)
        Y = np.empty((X.shape[0], n_out), np.float32)
        self.lib.orc_matmul_q8_0.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
        if self.lib.orc_matmul_q8_0(W.ctypes.data, n_in, n_out, _fp(X), X.shape[0], _fp(Y)) != 0:
            raise ValueError("the input width must be a multiple of 256")
        return Y

    def matmul_q(self, wtype, W, n_in, X):
        """The same for any weight type with an integer path: GGML_Q8_0, GGML_Q4_K, GGML_Q6_K."""
        W = np.ascontiguousarray(W, np.uint8)
        X = np.ascontiguousarray(X, np.float32).reshape(-1, n_in)
        self.lib.orc_qrow_bytes.restype = C.c_size_t
        rb = self.lib.orc_qrow_bytes(wtype, n_in)
        if rb == 0 or n_in % 256:
            raise ValueError("no integer path for this weight type / width")
        n_out = W.size // rb
        Y = np.empty((X.shape[0], n_out), np.float32)
        self.lib.orc_matmul_q.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
        assert self.lib.orc_matmul_q(wtype, W.ctypes.data, n_in, n_out, _fp(X), X.shape[0], _fp(Y)) == 0
        return Y

    # -- codecs ----------------------------------------------------------
    def q8_0_encode(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.size // 32 * 34, np.uint8)
        if self.lib.orc_q8_0_encode(_fp(x), out.ctypes.data, x.size) != 0:
            raise ValueError("Q8_0 needs a multiple of 32 elements")
        return out

    def q8_0_decode(self, b):
        b = np.ascontiguousarray(b, np.uint8)
        n = b.size // 34 * 32
        out = np.empty(n, np.float32)
        self.lib.orc_q8_0_decode(b.ctypes.data, _fp(out), n)
        return out

    def kv_int8_encode(self, x):
        x = np.ascontiguousarray(x, np.float32)
        q = np.empty(x.size, np.int8)
        s = self.lib.orc_kv_int8_encode(_fp(x), x.size, q.ctypes.data_as(C.POINTER(C.c_int8)))
        return q, np.float32(s)

    # -- attention core --------------------------------------------------
    def kv(self, capacity, nkv, hd, mode=KV_F32):
        return OracleKV(self.lib, capacity, nkv, hd, mode)

    def gqa_step(self, kv, q, k_new, v_new, n_heads, scale=0.0):
        out = np.zeros(n_heads * kv.hd, np.float32)
        self.lib.orc_gqa_step(C.byref(kv.c), _fp(q), _fp(k_new), _fp(v_new), n_heads, _fp(out), scale)
        return out

    def gqa_reference(self, Q, K, V, T, nh, nkv, hd, scale=0.0):
        O = np.zeros((T, nh * hd), np.float32)
        self.lib.orc_gqa_reference(_fp(Q), _fp(K), _fp(V), T, nh, nkv, hd, _fp(O), scale)
        return O

    def delta_step(self, S, q, k, v, alpha, beta):
        dv, dk = S.shape
        o = np.empty(dv, np.float32)
        self.lib.orc_delta_step(_fp(S), dk, dv, _fp(q), _fp(k), _fp(v), alpha, beta, _fp(o))
        return o

    def delta_prefill(self, S, Q, K, V, alpha, beta, chunk):
        dv, dk = S.shape
        T = alpha.size
        O = np.empty((T, dv), np.float32)
        self.lib.orc_delta_prefill(_fp(S), dk, dv, _fp(Q), _fp(K), _fp(V), _fp(alpha), _fp(beta),
                                   T, chunk, _fp(O))
        return O

    def conv_step(self, buf, K, x, w, bias=None):
        out = np.empty_like(x)
        self.lib.orc_conv_step(_fp(buf), K, x.size, _fp(x), _fp(w), _fp(bias), _fp(out))
        return out

    def conv_prefill(self, buf, K, X, w, bias=None):
        T, Cn = X.shape
        OUT = np.empty_like(X)
        self.lib.orc_conv_prefill(_fp(buf), K, Cn, _fp(X), _fp(w), _fp(bias), T, _fp(OUT))
        return OUT

    # -- layers ----------------------------------------------------------
    def linear_attn_step(self, layer: LinearLayer, S, conv_buf, qkv, a, b, z):
        out = np.empty(layer.vd, np.float32)
        p = layer.c_struct()
        self.lib.orc_linear_attn_step(C.byref(p), _fp(S), _fp(conv_buf), _fp(qkv), _fp(a), _fp(b),
                                      _fp(z), _fp(out))
        return out

    def linear_attn_prefill(self, layer: LinearLayer, S, conv_buf, QKV, A, B, Z, chunk=32):
        T = QKV.shape[0]
        OUT = np.empty((T, layer.vd), np.float32)
        p = layer.c_struct()
        self.lib.orc_linear_attn_prefill(C.byref(p), _fp(S), _fp(conv_buf), _fp(QKV), _fp(A), _fp(B),
                                         _fp(Z), T, chunk, _fp(OUT))
        return OUT

    def full_attn_step(self, layer: FullLayer, kv, pos, qproj, k, v):
        out = np.zeros(layer.nh * layer.hd, np.float32)
        p = layer.c_struct()
        self.lib.orc_full_attn_step(C.byref(p), C.byref(kv.c), pos, _fp(qproj), _fp(k), _fp(v), _fp(out))
        return out

    def full_attn_prefill(self, layer: FullLayer, kv, base, QP, K, V):
        T = QP.shape[0]
        OUT = np.zeros((T, layer.nh * layer.hd), np.float32)
        p = layer.c_struct()
        self.lib.orc_full_attn_prefill(C.byref(p), C.byref(kv.c), base, T, _fp(QP), _fp(K), _fp(V), _fp(OUT))
        return OUT


# ---------------------------------------------------------------------------
# The reference's own objects
# ---------------------------------------------------------------------------

class _RefKV(C.Structure):          # src/ornith_attn.h:57-69
    _fields_ = [("K", _f32p), ("V", _f32p),
                ("Kq", C.POINTER(C.c_int8)), ("Vq", C.POINTER(C.c_int8)),
                ("Ks", _f32p), ("Vs", _f32p),
                ("quantized", C.c_int), ("capacity", C.c_int), ("len", C.c_int),
                ("n_kv_heads", C.c_int), ("head_dim", C.c_int)]


class _RefDelta(C.Structure):       # src/ornith_attn.h:104-107
    _fields_ = [("S", _f32p), ("dk", C.c_int), ("dv", C.c_int)]


class _RefConv(C.Structure):        # src/ornith_attn.h:129-132
    _fields_ = [("buf", _f32p), ("K", C.c_int), ("C", C.c_int)]


OGGML_Q8_0 = 8                      # src/ornith_gguf.h:24


class Ref:
    """The reference's own compiled attention path (present only where it was built)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self, path: str = REF_SO):
        self.lib = L = C.CDLL(path)
        L.ot_dot.restype = C.c_float
        for n in ("ot_sigmoid", "ot_silu1", "ot_softplus"):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_float]
        L.ot_rng_uniform.restype = C.c_float
        L.ot_rng_uniform.argtypes = [C.c_void_p, C.c_float, C.c_float]
        L.ot_rng_fill.argtypes = [C.c_void_p, _f32p, C.c_int64, C.c_float, C.c_float]
        L.oq_f32_to_f16.restype = C.c_uint16
        L.oq_f32_to_f16.argtypes = [C.c_float]
        L.oq_f16_to_f32.restype = C.c_float
        L.oq_f16_to_f32.argtypes = [C.c_uint16]
        L.oq_quantize.argtypes = [C.c_uint32, _f32p, C.c_void_p, C.c_size_t]
        L.oq_dequantize.argtypes = [C.c_uint32, C.c_void_p, _f32p, C.c_size_t]
        L.ornith_kv_bytes_per_token.restype = C.c_size_t
        L.ot_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_float]
        L.ot_l2norm_eps.argtypes = [_f32p, _f32p, C.c_int, C.c_float]
        L.ot_rope_partial.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.ot_softmax.argtypes = [_f32p, C.c_int]
        L.ornith_gqa_step.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, C.c_int, _f32p, C.c_float]
        L.ornith_gqa_reference.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                           _f32p, C.c_float]
        L.ornith_delta_step.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, C.c_float, C.c_float, _f32p]
        L.ornith_delta_prefill.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, _f32p, _f32p,
                                           C.c_int, C.c_int, _f32p]
        L.ornith_conv_step.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, _f32p]
        L.ornith_conv_prefill.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, C.c_int, _f32p]

    def rng_fill(self, seed, n, lo, hi, state=None):
        st = C.c_uint64(seed) if state is None else state
        out = np.empty(n, np.float32)
        self.lib.ot_rng_fill(C.byref(st), _fp(out), n, lo, hi)
        return out, st

    def q8_0_encode(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.size // 32 * 34, np.uint8)
        assert self.lib.oq_quantize(OGGML_Q8_0, _fp(x), out.ctypes.data, x.size) == 0
        return out

    def q8k_quantize(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[:-1] + (x.shape[-1] // 256, 292), np.uint8)
        self.lib.refdrv_q8k_quantize.argtypes = [_f32p, C.c_void_p, C.c_longlong]
        self.lib.refdrv_q8k_quantize(_fp(x), out.ctypes.data, x.size)
        return out

    def matmul_q8_0(self, W, n_in, X):
        W = np.ascontiguousarray(W, np.uint8)
        X = np.ascontiguousarray(X, np.float32).reshape(-1, n_in)
        n_out = W.size // (n_in // 32 * 34)
        Y = np.empty((X.shape[0], n_out), np.float32)
        self.lib.refdrv_matmul_q8_0.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
        assert self.lib.refdrv_matmul_q8_0(W.ctypes.data, n_in, n_out, _fp(X), X.shape[0], _fp(Y)) == 0
        return Y

    def matmul_q(self, wtype, W, n_in, X):
        W = np.ascontiguousarray(W, np.uint8)
        X = np.ascontiguousarray(X, np.float32).reshape(-1, n_in)
        n_out = W.size // QROW_BYTES[wtype](n_in)
        Y = np.empty((X.shape[0], n_out), np.float32)
        self.lib.refdrv_matmul_q.argtypes = [C.c_uint, C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
        assert self.lib.refdrv_matmul_q(wtype, W.ctypes.data, n_in, n_out, _fp(X), X.shape[0], _fp(Y)) == 0
        return Y

    def quantize_rows(self, wtype, x):
        """f32 [rows][n] -> the reference encoder's bytes [rows][row bytes] (Q8_0, Q4_K, Q6_K)."""
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[:-1] + (QROW_BYTES[wtype](x.shape[-1]),), np.uint8)
        self.lib.refdrv_quantize_rows.argtypes = [C.c_uint, _f32p, C.c_void_p, C.c_longlong]
        self.lib.refdrv_quantize_rows.restype = C.c_longlong
        assert self.lib.refdrv_quantize_rows(wtype, _fp(x), out.ctypes.data, x.size) == out.size
        return out

    def q8_0_decode(self, b):
        n = b.size // 34 * 32
        out = np.empty(n, np.float32)
        assert self.lib.oq_dequantize(OGGML_Q8_0, b.ctypes.data, _fp(out), n) == 0
        return out

    def kv_init(self, capacity, nkv, hd, quantized):
        c = _RefKV()
        assert self.lib.ornith_kv_init_ex(C.byref(c), capacity, nkv, hd, quantized) == 0
        return c

    def kv_free(self, c):
        self.lib.ornith_kv_free(C.byref(c))

    def gqa_step(self, c, q, k_new, v_new, n_heads, scale=0.0):
        out = np.zeros(n_heads * c.head_dim, np.float32)
        self.lib.ornith_gqa_step(C.byref(c), _fp(q), _fp(k_new), _fp(v_new), n_heads, _fp(out), scale)
        return out

    def gqa_reference(self, Q, K, V, T, nh, nkv, hd, scale=0.0):
        O = np.zeros((T, nh * hd), np.float32)
        self.lib.ornith_gqa_reference(_fp(Q), _fp(K), _fp(V), T, nh, nkv, hd, _fp(O), scale)
        return O

    def delta_step(self, S, q, k, v, alpha, beta):
        dv, dk = S.shape
        st = _RefDelta(_fp(S), dk, dv)
        o = np.empty(dv, np.float32)
        self.lib.ornith_delta_step(C.byref(st), _fp(q), _fp(k), _fp(v), alpha, beta, _fp(o))
        return o

    def delta_prefill(self, S, Q, K, V, alpha, beta, chunk):
        dv, dk = S.shape
        T = alpha.size
        st = _RefDelta(_fp(S), dk, dv)
        O = np.empty((T, dv), np.float32)
        self.lib.ornith_delta_prefill(C.byref(st), _fp(Q), _fp(K), _fp(V), _fp(alpha), _fp(beta),
                                      T, chunk, _fp(O))
        return O

    def conv_step(self, buf, K, x, w, bias=None):
        cs = _RefConv(_fp(buf), K, x.size)
        out = np.empty_like(x)
        self.lib.ornith_conv_step(C.byref(cs), _fp(x), _fp(w), _fp(bias), _fp(out))
        return out

    def conv_prefill(self, buf, K, X, w, bias=None):
        T, Cn = X.shape
        cs = _RefConv(_fp(buf), K, Cn)
        OUT = np.empty_like(X)
        self.lib.ornith_conv_prefill(C.byref(cs), _fp(X), _fp(w), _fp(bias), T, _fp(OUT))
        return OUT


# ---- the reference's functions driven through whole layer steps (ref_driver.c) -----------
class _RefDrvLinear(C.Structure):
    _fields_ = [("nk", C.c_int), ("nv", C.c_int), ("dk", C.c_int), ("dv", C.c_int), ("conv_k", C.c_int),
                ("eps", C.c_float), ("conv_w", _f32p), ("a_coef", _f32p), ("dt_bias", _f32p), ("norm_w", _f32p)]


class _RefDrvFull(C.Structure):
    _fields_ = [("nh", C.c_int), ("nkv", C.c_int), ("hd", C.c_int), ("rope_dim", C.c_int),
                ("theta", C.c_float), ("eps", C.c_float), ("q_norm_w", _f32p), ("k_norm_w", _f32p),
                ("q8_0", C.c_int)]


def ref_linear_step(ref: "Ref", layer: LinearLayer, S, conv_buf, qkv, a, b, z):
    """One token of a delta-net layer through the reference's own functions
    (real-weights conventions: tiled head map, no conv bias, 1/sqrt(dk) scale)."""
    assert layer.head_map == HEADMAP_TILED and layer.conv_b is None
    p = _RefDrvLinear(layer.nk, layer.nv, layer.dk, layer.dv, layer.conv_k, layer.eps,
                      _fp(layer.conv_w), _fp(layer.a_coef), _fp(layer.dt_bias), _fp(layer.norm_w))
    out = np.empty(layer.vd, np.float32)
    ref.lib.refdrv_linear_step(C.byref(p), _fp(S), _fp(conv_buf), _fp(qkv), _fp(a), _fp(b), _fp(z), _fp(out))
    return out


def ref_full_step(ref: "Ref", layer: FullLayer, kv_struct, pos, qproj, k, v, q8_0=False):
    """One token of a full-attention layer through the reference's own functions over
    its f32 cache; q8_0 passes the appended rows through the reference's Q8_0 codec."""
    p = _RefDrvFull(layer.nh, layer.nkv, layer.hd, layer.rope_dim, layer.theta, layer.eps,
                    _fp(layer.q_norm_w), _fp(layer.k_norm_w), int(q8_0))
    out = np.zeros(layer.nh * layer.hd, np.float32)
    ref.lib.refdrv_full_step(C.byref(p), C.byref(kv_struct), int(pos), _fp(qproj), _fp(k), _fp(v), _fp(out))
    return out
