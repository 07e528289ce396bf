"""Host-side mirror of the engine's attention header over the CUDA drop-in (tier 1).

Same names, argument meaning and error behaviour as the engine's C functions
(reference: src/ornith_attn.h:71-147), with numpy float32 arrays standing in for
the host pointers.  Every call goes through libornith_cuda.so; nothing is
computed in Python.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import ConvState, DeltaState, KvCache, f32p


def _p(a):
    if a is None:
        return None
    assert isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(f32p)


def backend_cuda_available() -> bool:
    return bool(_lib.load().ornith_backend_cuda_available())


def last_error() -> str:
    return _lib.load().ornith_last_error().decode(errors="replace")


# ---- KV cache + GQA ---------------------------------------------------------------
def kv_init_ex(capacity, n_kv_heads, head_dim, quantized=0) -> KvCache:
    c = KvCache()
    st = _lib.load().ornith_kv_init_ex(C.byref(c), capacity, n_kv_heads, head_dim, quantized)
    if st != 0:
        raise MemoryError(last_error())
    return c


def kv_init(capacity, n_kv_heads, head_dim) -> KvCache:
    return kv_init_ex(capacity, n_kv_heads, head_dim, 0)


def kv_bytes_per_token(n_kv_heads, head_dim, quantized) -> int:
    return _lib.load().ornith_kv_bytes_per_token(n_kv_heads, head_dim, quantized)


def kv_free(c: KvCache) -> None:
    _lib.load().ornith_kv_free(C.byref(c))


def kv_reset(c: KvCache) -> None:
    _lib.load().ornith_kv_reset(C.byref(c))


def gqa_step(c: KvCache, q, k_new, v_new, n_heads, out=None, scale=0.0):
    if out is None:
        out = np.zeros(n_heads * c.head_dim, np.float32)
    _lib.load().ornith_gqa_step(C.byref(c), _p(q), _p(k_new), _p(v_new), n_heads, _p(out), scale)
    return out


def gqa_reference(Q, K, V, T, n_heads, n_kv_heads, head_dim, scale=0.0):
    O = np.zeros((T, n_heads * head_dim), np.float32)
    _lib.load().ornith_gqa_reference(_p(Q), _p(K), _p(V), T, n_heads, n_kv_heads, head_dim, _p(O), scale)
    return O


def kv_host_rows(c: KvCache):
    """The caller-visible host images of the cache, first `len` positions."""
    n = c.len * c.n_kv_heads * c.head_dim
    shape = (c.len, c.n_kv_heads, c.head_dim)
    if c.quantized:
        s = c.len * c.n_kv_heads
        return (np.ctypeslib.as_array(c.Kq, (n,)).copy().reshape(shape),
                np.ctypeslib.as_array(c.Vq, (n,)).copy().reshape(shape),
                np.ctypeslib.as_array(c.Ks, (s,)).copy().reshape(shape[:2]),
                np.ctypeslib.as_array(c.Vs, (s,)).copy().reshape(shape[:2]))
    return (np.ctypeslib.as_array(c.K, (n,)).copy().reshape(shape),
            np.ctypeslib.as_array(c.V, (n,)).copy().reshape(shape))


# ---- gated delta rule -------------------------------------------------------------
def delta_view(S: np.ndarray) -> DeltaState:
    """A state view over caller memory, the way the engine builds them
    (reference: src/ornith_rforward.c:494)."""
    dv, dk = S.shape
    return DeltaState(_p(S), dk, dv)


def delta_step(S: np.ndarray, q, k, v, alpha, beta):
    st = delta_view(S)
    o = np.zeros(S.shape[0], np.float32)
    _lib.load().ornith_delta_step(C.byref(st), _p(q), _p(k), _p(v), alpha, beta, _p(o))
    return o


def delta_prefill(S: np.ndarray, Q, K, V, alpha, beta, chunk):
    st = delta_view(S)
    T = alpha.size
    O = np.zeros((T, S.shape[0]), np.float32)
    _lib.load().ornith_delta_prefill(C.byref(st), _p(Q), _p(K), _p(V), _p(alpha), _p(beta), T, chunk, _p(O))
    return O


# ---- causal conv --------------------------------------------------------------------
def conv_step(buf: np.ndarray, K, x, w, bias=None):
    cs = ConvState(_p(buf), K, x.size)
    out = np.zeros_like(x)
    _lib.load().ornith_conv_step(C.byref(cs), _p(x), _p(w), _p(bias), _p(out))
    return out


def conv_prefill(buf: np.ndarray, K, X, w, bias=None):
    T, Cn = X.shape
    cs = ConvState(_p(buf), K, Cn)
    OUT = np.zeros_like(X)
    _lib.load().ornith_conv_prefill(C.byref(cs), _p(X), _p(w), _p(bias), T, _p(OUT))
    return OUT
