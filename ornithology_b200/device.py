"""Python face of the device-resident C ABI (tier 2 of include/ornith_cuda.h).

torch is used for what it is good at here — owning device memory and streams.
Every computation is a call into libornith_cuda.so with raw device pointers.
The classes mirror the engine's objects: a full-attention layer with its KV
cache (reference: src/ornith_rforward.c:419-455, src/ornith_attn.h:57-69) and a
gated delta-net layer with its recurrent state and conv history
(reference: src/ornith_rforward.c:457-503, :212-274).
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _lib
from ._lib import (ACT_BF16, ACT_F32, HEADMAP_GROUPED, HEADMAP_TILED, KV_F32, KV_INT8_HEAD, KV_Q8_0,
                   CudaFullLayer, CudaKv, CudaLinearLayer, CudaLinearState, check)

__all__ = ["FullLayer", "KvBatch", "LinearLayer", "LinearState", "full_attn_step", "full_attn_prefill", "kv_append",
           "linear_attn_step", "linear_attn_prefill", "advance", "q8_0_encode", "q8_0_decode",
           "ACT_F32", "ACT_BF16", "KV_F32", "KV_INT8_HEAD", "KV_Q8_0", "HEADMAP_TILED", "HEADMAP_GROUPED"]


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _act(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return ACT_F32
    if t.dtype == torch.bfloat16:
        return ACT_BF16
    raise TypeError(f"activations must be float32 or bfloat16, got {t.dtype}")


def _dev_f32(a, device):
    return None if a is None else torch.as_tensor(np.ascontiguousarray(a, np.float32)).to(device)


class _Scratch:
    def __init__(self):
        self.buf = None

    def get(self, nbytes: int, device):
        if self.buf is None or self.buf.numel() < nbytes or self.buf.device != torch.device(device):
            self.buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        return self.buf


class FullLayer:
    """Weights and shape of one full-attention layer, resident on the device."""

    def __init__(self, nh, nkv, hd, q_norm_w=None, k_norm_w=None, rope_dim=64, theta=1e7, eps=1e-6,
                 gated=True, scale=0.0, device="cuda:0"):
        lib = _lib.load()
        self.nh, self.nkv, self.hd, self.rope_dim, self.gated = nh, nkv, hd, rope_dim, bool(gated)
        self.device = torch.device(device)
        self.q_norm_w = _dev_f32(q_norm_w, device)
        self.k_norm_w = _dev_f32(k_norm_w, device)
        self.inv_freq = None
        if rope_dim > 0:
            tab = np.empty(rope_dim // 2, np.float32)
            lib.ornith_cuda_rope_inv_freq(theta, rope_dim, tab.ctypes.data_as(_lib.f32p))
            self.inv_freq = torch.from_numpy(tab).to(device)
        self.c = CudaFullLayer(nh, nkv, hd, rope_dim, int(self.gated), eps, scale,
                               _ptr(self.q_norm_w), _ptr(self.k_norm_w), _ptr(self.inv_freq))
        self.scratch = _Scratch()

    @property
    def qproj_width(self):
        return self.nh * self.hd * (2 if self.gated else 1)


class KvBatch:
    """One layer's KV cache for a batch of sequences with individual capacities."""

    def __init__(self, mode, nkv, hd, capacities, device="cuda:0"):
        self.mode, self.nkv, self.hd = mode, nkv, hd
        self.capacities = [int(c) for c in capacities]
        self.n_seq = len(self.capacities)
        self.device = torch.device(device)
        off = np.zeros(self.n_seq + 1, np.int64)
        off[1:] = np.cumsum(self.capacities)
        self.seq_off_host = off
        self.seq_off = torch.from_numpy(off).to(device)
        total = int(off[-1])
        self.row_bytes = {KV_F32: hd * 4, KV_INT8_HEAD: hd, KV_Q8_0: hd // 32 * 34}[mode]
        self.K = torch.zeros(max(total * nkv * self.row_bytes, 16), dtype=torch.uint8, device=device)
        self.V = torch.zeros_like(self.K)
        self.Ks = self.Vs = None
        if mode == KV_INT8_HEAD:
            self.Ks = torch.zeros(max(total * nkv, 1), dtype=torch.float32, device=device)
            self.Vs = torch.zeros_like(self.Ks)
        self.c = CudaKv(mode, nkv, hd, self.n_seq, _ptr(self.K), _ptr(self.V), _ptr(self.Ks), _ptr(self.Vs),
                        _ptr(self.seq_off))

    def bytes_per_token(self):
        extra = 8 * self.nkv if self.mode == KV_INT8_HEAD else 0
        return 2 * self.nkv * self.row_bytes + extra

    def rows(self, seq, n):
        """Host copy of the first n stored rows of sequence `seq`: (K, V[, Ks, Vs])."""
        o = int(self.seq_off_host[seq])
        rb = self.nkv * self.row_bytes
        Kb = self.K[o * rb:(o + n) * rb].cpu().numpy()
        Vb = self.V[o * rb:(o + n) * rb].cpu().numpy()
        if self.mode == KV_F32:
            return Kb.view(np.float32).reshape(n, self.nkv, self.hd), Vb.view(np.float32).reshape(n, self.nkv, self.hd)
        if self.mode == KV_Q8_0:
            return Kb.reshape(n, self.nkv, -1), Vb.reshape(n, self.nkv, -1)
        return (Kb.view(np.int8).reshape(n, self.nkv, self.hd), Vb.view(np.int8).reshape(n, self.nkv, self.hd),
                self.Ks[o * self.nkv:(o + n) * self.nkv].cpu().numpy().reshape(n, self.nkv),
                self.Vs[o * self.nkv:(o + n) * self.nkv].cpu().numpy().reshape(n, self.nkv))


class Q8_0Weight:
    """A projection weight on the device as the GGUF tensor's Q8_0 rows, [n_out][n_in/32][34] bytes."""

    def __init__(self, rows_bytes, n_in, device="cuda:0"):
        rows = np.ascontiguousarray(rows_bytes, np.uint8).reshape(-1)
        self.n_in = int(n_in)
        self.n_out = rows.size // (self.n_in // 32 * 34)
        self.bytes = torch.from_numpy(rows).to(device)
        self._scratch = None

    def scratch(self, T):
        need = _lib.load().ornith_cuda_qproj_scratch(int(T), self.n_in)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.uint8, device=self.bytes.device)
        return self._scratch


def q8k_quantize(x, n_in):
    """x [T][n_in] on the device -> the engine's Q8_K blocks, [T][n_in/256][292] bytes (host array)."""
    lib = _lib.load()
    T = x.numel() // n_in
    blocks = torch.empty(T * (n_in // 256) * 292, dtype=torch.uint8, device=x.device)
    need = lib.ornith_cuda_qproj_scratch(T, n_in)
    scr = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib.ornith_cuda_q8k_quantize(_ptr(x), _act(x), T, n_in, _ptr(blocks), _ptr(scr), need, _stream()), "q8k_quantize")
    return blocks.cpu().numpy().reshape(T, n_in // 256, 292)


def matmul_q8_0(w: Q8_0Weight, x, out=None):
    """y [T][n_out] = x [T][n_in] through Q8_0 weight rows (the engine's quantised projection)."""
    lib = _lib.load()
    T = x.numel() // w.n_in
    if out is None:
        out = torch.empty(T, w.n_out, dtype=x.dtype, device=x.device)
    scr = w.scratch(T)
    check(lib.ornith_cuda_matmul_q8_0(_ptr(w.bytes), w.n_in, w.n_out, _ptr(x), _act(x), T, _ptr(out), _act(out), _ptr(scr),
                                      scr.numel(), _stream()), "matmul_q8_0")
    return out


GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 8, 12, 14          # GGUF tensor type ids (reference: src/ornith_gguf.h:24-30)
_QROW_BYTES = {GGML_Q8_0: lambda n: n // 32 * 34, GGML_Q4_K: lambda n: n // 256 * 144, GGML_Q6_K: lambda n: n // 256 * 210}


class QWeight:
    """A projection weight on the device as the GGUF tensor's bytes: [n_out] rows of Q8_0, Q4_K or Q6_K blocks."""

    def __init__(self, wtype, rows_bytes, n_in, device="cuda:0"):
        rows = np.ascontiguousarray(rows_bytes, np.uint8).reshape(-1)
        self.wtype, self.n_in = int(wtype), int(n_in)
        self.n_out = rows.size // _QROW_BYTES[self.wtype](self.n_in)
        self.bytes = torch.from_numpy(rows).to(device)
        self._scratch = None

    def scratch(self, T):
        need = _lib.load().ornith_cuda_matmul_q_scratch(self.wtype, int(T), self.n_in)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.uint8, device=self.bytes.device)
        return self._scratch


def q8k_image(x, n_in, image=None):
    """x [T][n_in] -> the Q8_K image the integer products read; one image serves every projection of the same input."""
    lib = _lib.load()
    T = x.numel() // n_in
    need = lib.ornith_cuda_matmul_q_scratch(GGML_Q8_0, T, n_in)
    if image is None or image.numel() < need:
        image = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib.ornith_cuda_q8k_image(_ptr(x), _act(x), T, n_in, _ptr(image), image.numel(), _stream()), "q8k_image")
    return image


def matmul_q(w: QWeight, x, out=None, image=None, T=None, out_dtype=None):
    """y [T][n_out] = x [T][n_in] through quantised weight rows: the engine's integer path, bit for bit.
    With image= (from q8k_image) and T=, x is not read again."""
    lib = _lib.load()
    if image is not None:
        if out is None:
            out = torch.empty(T, w.n_out, dtype=out_dtype or torch.float32, device=image.device)
        check(lib.ornith_cuda_matmul_q_image(w.wtype, _ptr(w.bytes), w.n_in, w.n_out, _ptr(image), int(T), _ptr(out), _act(out),
                                             _stream()), "matmul_q_image")
        return out
    T = x.numel() // w.n_in
    if out is None:
        out = torch.empty(T, w.n_out, dtype=x.dtype, device=x.device)
    scr = w.scratch(T)
    check(lib.ornith_cuda_matmul_q(w.wtype, _ptr(w.bytes), w.n_in, w.n_out, _ptr(x), _act(x), T, _ptr(out), _act(out),
                                   _ptr(scr), scr.numel(), _stream()), "matmul_q")
    return out


def matmul_q_group(ws, image, T, outs=None, out_dtype=None):
    """Several projections of the same (already quantised) input in one launch per weight type; returns the outputs."""
    lib = _lib.load()
    if outs is None:
        outs = [torch.empty(T, w.n_out, dtype=out_dtype or torch.float32, device=image.device) for w in ws]
    arr = (_lib.CudaQproj * len(ws))()
    for i, (w, o) in enumerate(zip(ws, outs)):
        arr[i].wtype, arr[i].W, arr[i].n_out, arr[i].y = w.wtype, _ptr(w.bytes), w.n_out, _ptr(o)
    check(lib.ornith_cuda_matmul_q_group(C.cast(arr, C.c_void_p), len(ws), ws[0].n_in, _ptr(image), int(T), _act(outs[0]), _stream()),
          "matmul_q_group")
    return outs


def kv_export(kv: KvBatch, seq, length):
    """Session record of the first `length` positions of sequence `seq` (bytes, the engine's layer record)."""
    lib = _lib.load()
    n = lib.ornith_cuda_kv_record_bytes(C.byref(kv.c), int(length))
    buf = np.zeros(n, np.uint8)
    check(lib.ornith_cuda_kv_export(C.byref(kv.c), int(seq), int(length), buf.ctypes.data_as(C.c_void_p), n, _stream()),
          "kv_export")
    return buf


def kv_import(kv: KvBatch, seq, record, kv_len=None):
    """Load a session record into sequence `seq`; returns its position count (and sets kv_len[seq] if given)."""
    lib = _lib.load()
    rec = np.ascontiguousarray(record, np.uint8)
    n = C.c_int32(0)
    check(lib.ornith_cuda_kv_import(C.byref(kv.c), int(seq), rec.ctypes.data_as(C.c_void_p), rec.size, C.byref(n),
                                    _ptr(kv_len), _stream()), "kv_import")
    return n.value


class LinearLayer:
    """Weights and shape of one gated delta-net layer, resident on the device."""

    def __init__(self, nk, nv, dk, dv, conv_w, a_coef, dt_bias, norm_w, conv_b=None, conv_k=4,
                 head_map=HEADMAP_TILED, out_scale=None, eps=1e-6, device="cuda:0"):
        _lib.load()
        self.nk, self.nv, self.dk, self.dv, self.conv_k, self.head_map = nk, nv, dk, dv, conv_k, head_map
        self.qd, self.vd = nk * dk, nv * dv
        self.cc = 2 * self.qd + self.vd
        self.device = torch.device(device)
        if out_scale is None:
            out_scale = float(np.float32(1.0) / np.sqrt(np.float32(dk)))
        self.conv_w = _dev_f32(conv_w, device)
        self.conv_b = _dev_f32(conv_b, device)
        self.a_coef = _dev_f32(a_coef, device)
        self.dt_bias = _dev_f32(dt_bias, device)
        self.norm_w = _dev_f32(norm_w, device)
        assert tuple(self.conv_w.shape) == (self.cc, conv_k)
        self.c = CudaLinearLayer(nk, nv, dk, dv, conv_k, head_map, out_scale, eps, _ptr(self.conv_w),
                                 _ptr(self.conv_b), _ptr(self.a_coef), _ptr(self.dt_bias), _ptr(self.norm_w))
        self.scratch = _Scratch()


class LinearState:
    """Recurrent state S [n_seq][nv][dv][dk] and conv ring [n_seq][conv_k][Cc] of one layer."""

    def __init__(self, layer: LinearLayer, n_seq, device=None):
        device = device or layer.device
        self.layer, self.n_seq = layer, n_seq
        self.S = torch.zeros(n_seq, layer.nv, layer.dv, layer.dk, dtype=torch.float32, device=device)
        self.conv = torch.zeros(n_seq, layer.conv_k, layer.cc, dtype=torch.float32, device=device)
        self.c = CudaLinearState(_ptr(self.S), _ptr(self.conv), layer.nv * layer.dv * layer.dk,
                                 layer.conv_k * layer.cc)

    def conv_image(self, seq, pos):
        """The engine's history image [(conv_k-1)][Cc], oldest first, for sequence `seq`."""
        L = self.layer
        img = torch.empty(L.conv_k - 1, L.cc, dtype=torch.float32, device=self.conv.device)
        check(_lib.load().ornith_cuda_conv_export(_ptr(self.conv[seq]), L.conv_k, L.cc, int(pos), _ptr(img),
                                                  _stream()), "conv_export")
        return img

    def export_record(self, seq, pos):
        """Session record of sequence `seq` after `pos` tokens: S, conv_k, Cc, history image (bytes)."""
        lib = _lib.load()
        n = lib.ornith_cuda_linear_record_bytes(C.byref(self.layer.c))
        buf = np.zeros(n, np.uint8)
        check(lib.ornith_cuda_linear_export(C.byref(self.layer.c), C.byref(self.c), int(seq), int(pos),
                                            buf.ctypes.data_as(C.c_void_p), n, _stream()), "linear_export")
        return buf

    def import_record(self, seq, pos, record):
        lib = _lib.load()
        rec = np.ascontiguousarray(record, np.uint8)
        check(lib.ornith_cuda_linear_import(C.byref(self.layer.c), C.byref(self.c), int(seq), int(pos),
                                            rec.ctypes.data_as(C.c_void_p), rec.size, _stream()), "linear_import")

    def load_conv_image(self, seq, pos, image):
        L = self.layer
        img = torch.as_tensor(np.ascontiguousarray(image, np.float32)).to(self.conv.device)
        check(_lib.load().ornith_cuda_conv_import(_ptr(self.conv[seq]), L.conv_k, L.cc, int(pos), _ptr(img),
                                                  _stream()), "conv_import")


def full_attn_step(layer: FullLayer, kv: KvBatch, kv_len, qproj, k, v, out=None, rope_pos=None, max_len=None):
    """One decode token per sequence through a full-attention layer (between the projections)."""
    lib = _lib.load()
    B = kv.n_seq
    act = _act(qproj)
    if out is None:
        out = torch.empty(B, layer.nh * layer.hd, dtype=qproj.dtype, device=qproj.device)
    if max_len is None:
        max_len = int(kv_len.max().item()) + 1
    need = lib.ornith_cuda_full_attn_step_scratch(C.byref(layer.c), B, int(max_len))
    scr = layer.scratch.get(need, qproj.device)
    check(lib.ornith_cuda_full_attn_step(C.byref(layer.c), C.byref(kv.c), _ptr(kv_len), _ptr(rope_pos),
                                         _ptr(qproj), _ptr(k), _ptr(v), _ptr(out), act, int(max_len),
                                         _ptr(scr), scr.numel(), _stream()), "full_attn_step")
    return out


def full_attn_prefill(layer: FullLayer, kv: KvBatch, kv_len, qproj, k, v, T, out=None, rope_pos=None, max_len=None):
    """T new tokens per sequence; `max_len` bounds kv_len[b] + T (default: the largest capacity)."""
    lib = _lib.load()
    if max_len is None:
        max_len = max(kv.capacities)
    B = kv.n_seq
    act = _act(qproj)
    if out is None:
        out = torch.empty(B, T, layer.nh * layer.hd, dtype=qproj.dtype, device=qproj.device)
    need = lib.ornith_cuda_full_attn_prefill_scratch(C.byref(layer.c), B, int(T), int(max_len))
    scr = layer.scratch.get(need, qproj.device)
    check(lib.ornith_cuda_full_attn_prefill(C.byref(layer.c), C.byref(kv.c), _ptr(kv_len), _ptr(rope_pos),
                                            _ptr(qproj), _ptr(k), _ptr(v), _ptr(out), act, int(T), int(max_len),
                                            _ptr(scr), scr.numel(), _stream()), "full_attn_prefill")
    return out


def kv_append(layer: FullLayer, kv: KvBatch, kv_len, k, v, T=1, rope_pos=None):
    """Normalise + rotate k and encode k, v into the cache at kv_len[b].. (no attention)."""
    check(_lib.load().ornith_cuda_kv_append(C.byref(layer.c), C.byref(kv.c), _ptr(kv_len), _ptr(rope_pos),
                                            _ptr(k), _ptr(v), _act(k), int(T), _stream()), "kv_append")


def linear_attn_step(layer: LinearLayer, st: LinearState, pos, qkv, a, b, z, out=None):
    """One decode token per sequence through a gated delta-net layer (between the projections)."""
    lib = _lib.load()
    act = _act(qkv)
    B = st.n_seq
    if out is None:
        out = torch.empty(B, layer.vd, dtype=qkv.dtype, device=qkv.device)
    check(lib.ornith_cuda_linear_attn_step(C.byref(layer.c), C.byref(st.c), _ptr(pos), _ptr(qkv), _ptr(a),
                                           _ptr(b), _ptr(z), _ptr(out), act, B, _stream()), "linear_attn_step")
    return out


def linear_attn_prefill(layer: LinearLayer, st: LinearState, pos, qkv, a, b, z, T, chunk=32, out=None):
    lib = _lib.load()
    act = _act(qkv)
    B = st.n_seq
    if out is None:
        out = torch.empty(B, T, layer.vd, dtype=qkv.dtype, device=qkv.device)
    need = lib.ornith_cuda_linear_attn_prefill_scratch(C.byref(layer.c), B, int(T))
    scr = layer.scratch.get(need, qkv.device)
    check(lib.ornith_cuda_linear_attn_prefill(C.byref(layer.c), C.byref(st.c), _ptr(pos), _ptr(qkv), _ptr(a),
                                              _ptr(b), _ptr(z), _ptr(out), act, B, int(T), int(chunk),
                                              _ptr(scr), scr.numel(), _stream()), "linear_attn_prefill")
    return out


def advance(counters: torch.Tensor, delta=1):
    check(_lib.load().ornith_cuda_advance(_ptr(counters), counters.numel(), int(delta), _stream()), "advance")


def q8_0_encode(x: torch.Tensor) -> torch.Tensor:
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = torch.empty(x.numel() // 32 * 34, dtype=torch.uint8, device=x.device)
    check(_lib.load().ornith_cuda_q8_0_encode(_ptr(x), _ptr(out), x.numel(), _stream()), "q8_0_encode")
    return out


def q8_0_decode(b: torch.Tensor) -> torch.Tensor:
    n = b.numel() // 34 * 32
    out = torch.empty(n, dtype=torch.float32, device=b.device)
    check(_lib.load().ornith_cuda_q8_0_decode(_ptr(b), _ptr(out), n, _stream()), "q8_0_decode")
    return out
