"""Generate the golden fixtures in this directory from the reference's own code.

Run where the reference checkout is mounted (it is compiled, unmodified, into
oracle/_ref/libornith_ref.so by oracle/Makefile):

    python tests/golden/make_golden.py

Every array below is produced by calling the reference's functions
(src/ornith_attn.c, src/ornith_tensor.c, src/ornith_quant.c, src/ornith_qdot.c) through ctypes; the
seeds and shapes of the first four files are those of the reference's
tests/test_attn.c (:28-192).  The layer-level files compose the reference
primitives exactly as src/ornith_rforward.c:419-503 / src/ornith_forward.c:277-399
do, minus the projections.
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle.oracle import Ref, _fp, build  # noqa: E402

build()
r = Ref()
L = r.lib


def save(name, **kw):
    np.savez_compressed(os.path.join(HERE, name), **kw)
    print(name, {k: getattr(v, "shape", v) for k, v in kw.items()})


def silu(x):
    return np.array([L.ot_silu1(float(v)) for v in x.ravel()], np.float32).reshape(x.shape)


def sigmoid(x):
    return np.float32(L.ot_sigmoid(float(x)))


def rmsnorm(x, w, eps):
    out = np.empty_like(x)
    L.ot_rmsnorm(_fp(np.ascontiguousarray(x)), _fp(w), _fp(out), x.size, eps)
    return out


def l2norm(x):
    out = np.empty_like(x)
    L.ot_l2norm_eps(_fp(np.ascontiguousarray(x)), _fp(out), x.size, 1e-6)
    return out


def rope(v, rot, pos, theta):
    v = np.array(v, np.float32)
    L.ot_rope_partial(_fp(v), v.size, rot, pos, theta)
    return v


# ---- tests/test_attn.c:28-83 -------------------------------------------------
def delta_parity():
    dk, dv, T = 6, 5, 17
    st = C.c_uint64(0xABCDEF)
    Q, _ = r.rng_fill(0, T * dk, -1, 1, st)
    K, _ = r.rng_fill(0, T * dk, -1, 1, st)
    V, _ = r.rng_fill(0, T * dv, -1, 1, st)
    al = np.empty(T, np.float32); be = np.empty(T, np.float32)
    for t in range(T):
        al[t] = L.ot_rng_uniform(C.byref(st), 0.85, 0.999)
        be[t] = L.ot_rng_uniform(C.byref(st), 0.1, 0.9)
    Q, K, V = Q.reshape(T, dk), K.reshape(T, dk), V.reshape(T, dv)
    S = np.zeros((dv, dk), np.float32)
    O = np.stack([r.delta_step(S, Q[t], K[t], V[t], al[t], be[t]) for t in range(T)])
    save("attn_delta_parity.npz", Q=Q, K=K, V=V, alpha=al, beta=be, O_step=O, S_final=S)


# ---- tests/test_attn.c:87-119 ------------------------------------------------
def gqa(seed, nh, nkv, hd, T, name, quantized):
    st = C.c_uint64(seed)
    Q, _ = r.rng_fill(0, T * nh * hd, -1, 1, st)
    K, _ = r.rng_fill(0, T * nkv * hd, -1, 1, st)
    V, _ = r.rng_fill(0, T * nkv * hd, -1, 1, st)
    Q, K, V = Q.reshape(T, -1), K.reshape(T, -1), V.reshape(T, -1)
    O_ref = r.gqa_reference(Q, K, V, T, nh, nkv, hd)
    c = r.kv_init(T, nkv, hd, quantized)
    O_step = np.stack([r.gqa_step(c, Q[t], K[t], V[t], nh) for t in range(T)])
    kw = dict(Q=Q, K=K, V=V, O_naive=O_ref, O_step=O_step, nh=nh, nkv=nkv, hd=hd)
    if quantized:
        n = T * nkv * hd
        kw["Kq"] = np.ctypeslib.as_array(c.Kq, (n,)).copy().reshape(T, nkv, hd)
        kw["Vq"] = np.ctypeslib.as_array(c.Vq, (n,)).copy().reshape(T, nkv, hd)
        kw["Ks"] = np.ctypeslib.as_array(c.Ks, (T * nkv,)).copy().reshape(T, nkv)
        kw["Vs"] = np.ctypeslib.as_array(c.Vs, (T * nkv,)).copy().reshape(T, nkv)
    r.kv_free(c)
    save(name, **kw)


# ---- tests/test_attn.c:162-192 -----------------------------------------------
def conv():
    K, Cn, T = 4, 3, 9
    st = C.c_uint64(7)
    X, _ = r.rng_fill(0, T * Cn, -1, 1, st)
    w, _ = r.rng_fill(0, Cn * K, -1, 1, st)
    b, _ = r.rng_fill(0, Cn, -0.2, 0.2, st)
    X = X.reshape(T, Cn); w = w.reshape(Cn, K)
    buf = np.zeros((K - 1) * Cn + 1, np.float32)
    OUT = r.conv_prefill(buf, K, X, w, b)
    save("attn_conv.npz", X=X, w=w, b=b, OUT=OUT, buf_final=buf[:-1].reshape(K - 1, Cn))


# ---- Q8_0 + f16 known answers (src/ornith_quant.c:14-65, :155-184) -----------
def codecs():
    g = np.random.default_rng(2024)
    blocks = [np.zeros(32), np.full(32, 1e-9), np.full(32, 6e-6),       # zero / f16-subnormal scales
              np.arange(32) - 15.5, (np.arange(32) - 16) * 0.5,         # exact .5 ties after scaling
              np.r_[127.0, (np.arange(31) + 0.5)], np.r_[-127.0, -(np.arange(31) + 0.5)],
              np.r_[1e30, g.standard_normal(31) * 1e29], np.r_[70000.0 * 127, np.ones(31)],
              np.sin(np.arange(32) * 0.3) * 5.0, np.sin((np.arange(32) + 32) * 0.3) * 5.0]
    blocks += [g.standard_normal(32) * s for s in (1e-3, 1.0, 1.0, 30.0, 1e4) for _ in range(40)]
    x = np.concatenate(blocks).astype(np.float32)
    b = r.q8_0_encode(x)
    save("q8_0_vectors.npz", x=x, bytes=b, decoded=r.q8_0_decode(b))
    f = np.concatenate([g.standard_normal(3000) * 10.0 ** g.integers(-9, 6, 3000),
                        [0.0, -0.0, 1.0, -0.5, 65504.0, 65519.9, 65520.0, 1e9, 5.96e-8, 2.98e-8,
                         2.9802322e-8, 3e-8, 6.1e-5, 6.09e-5, np.inf, -np.inf]]).astype(np.float32)
    h = np.array([L.oq_f32_to_f16(float(v)) for v in f], np.uint16)
    allh = np.arange(65536, dtype=np.uint16)
    back = np.array([L.oq_f16_to_f32(int(v)) for v in allh], np.float32)
    save("f16_vectors.npz", f=f, h=h, all_h_to_f32_bits=back.view(np.uint32))
    # the reference's per-head int8 KV code (src/ornith_attn.c:65-77), via its cache
    hd = 64
    rows = np.stack([g.standard_normal(hd) * s for s in (1e-3, 1, 1, 50)] +
                    [np.zeros(hd), (np.arange(hd) - 31.5) / 31.5 * 127 / 127]).astype(np.float32)
    c = r.kv_init(len(rows), 1, hd, 1)
    for row in rows:
        r.gqa_step(c, np.zeros(hd, np.float32), row, row, 1)
    save("kv_int8_vectors.npz", x=rows,
         codes=np.ctypeslib.as_array(c.Kq, (rows.size,)).copy().reshape(rows.shape),
         scales=np.ctypeslib.as_array(c.Ks, (len(rows),)).copy())
    r.kv_free(c)


# ---- one 35B-shaped value head, step path ------------------------------------
def delta_head128():
    g = np.random.default_rng(5)
    dk = dv = 128; T = 24
    Q = np.stack([l2norm(v) for v in g.standard_normal((T, dk)).astype(np.float32)])
    K = np.stack([l2norm(v) for v in g.standard_normal((T, dk)).astype(np.float32)])
    V = g.standard_normal((T, dv)).astype(np.float32)
    al = g.uniform(0.4, 0.999, T).astype(np.float32); be = g.uniform(0.05, 0.95, T).astype(np.float32)
    S = np.zeros((dv, dk), np.float32)
    O = np.stack([r.delta_step(S, Q[t], K[t], V[t], al[t], be[t]) for t in range(T)])
    S2 = np.zeros((dv, dk), np.float32)
    O2 = r.delta_prefill(S2, Q, K, V, al, be, 8)
    save("delta_head128.npz", Q=Q, K=K, V=V, alpha=al, beta=be, O_step=O, S_final=S,
         O_chunk8=O2, S_chunk8=S2)


# ---- layer wiring: linear layer (src/ornith_rforward.c:457-503, :300-314) ----
def linear_layer(name, head_map, with_bias, scaled, seed):
    g = np.random.default_rng(seed)
    nk, nv, dk, dv, K, T = 2, 4, 32, 32, 4, 12
    qd, vd = nk * dk, nv * dv; Cc = 2 * qd + vd
    conv_w = g.uniform(-0.2, 0.2, (Cc, K)).astype(np.float32)
    conv_b = g.uniform(-0.1, 0.1, Cc).astype(np.float32) if with_bias else None
    a_coef = g.uniform(-0.8, -0.2, nv).astype(np.float32)
    dt_bias = g.uniform(-0.05, 0.05, nv).astype(np.float32)
    norm_w = g.uniform(0.9, 1.1, dv).astype(np.float32)
    QKV = g.standard_normal((T, Cc)).astype(np.float32)
    A = g.standard_normal((T, nv)).astype(np.float32); B = g.standard_normal((T, nv)).astype(np.float32)
    Z = g.standard_normal((T, vd)).astype(np.float32)
    buf = np.zeros((K - 1) * Cc + 1, np.float32)
    S = np.zeros((nv, dv, dk), np.float32)
    OUT = np.empty((T, vd), np.float32)
    scale = np.float32(1.0) / np.sqrt(np.float32(dk))
    for t in range(T):
        conv = silu(r.conv_step(buf, K, QKV[t], conv_w, conv_b))
        q, k, v = conv[:qd], conv[qd:2 * qd], conv[2 * qd:]
        o_all = np.empty(vd, np.float32)
        for hv in range(nv):
            kh = hv % nk if head_map == 0 else hv // (nv // nk)
            qn = l2norm(q[kh * dk:(kh + 1) * dk]); kn = l2norm(k[kh * dk:(kh + 1) * dk])
            sp = np.float32(L.ot_softplus(float(np.float32(A[t, hv] + dt_bias[hv]))))
            # expf through libm, like the reference (src/ornith_rforward.c:282-284)
            alpha = np.float32(_expf(np.float32(a_coef[hv] * sp)))
            o_all[hv * dv:(hv + 1) * dv] = r.delta_step(S[hv], qn, kn, np.ascontiguousarray(v[hv * dv:(hv + 1) * dv]),
                                                        alpha, sigmoid(B[t, hv]))
        if scaled:
            o_all = (o_all * scale).astype(np.float32)
        o = np.concatenate([rmsnorm(o_all[h * dv:(h + 1) * dv], norm_w, 1e-6) for h in range(nv)])
        OUT[t] = o * silu(Z[t])
    save(name, nk=nk, nv=nv, dk=dk, dv=dv, head_map=head_map, scaled=int(scaled),
         conv_w=conv_w, conv_b=(conv_b if with_bias else np.zeros(0, np.float32)),
         a_coef=a_coef, dt_bias=dt_bias, norm_w=norm_w, QKV=QKV, A=A, B=B, Z=Z,
         OUT=OUT, S_final=S, conv_final=buf[:-1].reshape(K - 1, Cc))


_libm = C.CDLL("libm.so.6")
_libm.expf.restype = C.c_float
_libm.expf.argtypes = [C.c_float]


def _expf(x):
    return _libm.expf(float(x))


# ---- layer wiring: full layer (src/ornith_rforward.c:419-455) ----------------
def full_layer(name, quantized, seed):
    g = np.random.default_rng(seed)
    nh, nkv, hd, rot, T, theta = 4, 2, 64, 16, 10, 1e7
    qw = g.uniform(0.9, 1.1, hd).astype(np.float32); kw_ = g.uniform(0.9, 1.1, hd).astype(np.float32)
    QP = g.standard_normal((T, nh * 2 * hd)).astype(np.float32)
    K = g.standard_normal((T, nkv * hd)).astype(np.float32)
    V = g.standard_normal((T, nkv * hd)).astype(np.float32)
    c = r.kv_init(T, nkv, hd, quantized)
    OUT = np.empty((T, nh * hd), np.float32)
    base = 3
    for t in range(T):
        qp = QP[t].reshape(nh, 2, hd)
        q = np.concatenate([rope(rmsnorm(np.ascontiguousarray(qp[h, 0]), qw, 1e-6), rot, base + t, theta)
                            for h in range(nh)])
        gate = np.ascontiguousarray(qp[:, 1, :]).ravel()
        k = np.concatenate([rope(rmsnorm(np.ascontiguousarray(K[t, h * hd:(h + 1) * hd]), kw_, 1e-6),
                                 rot, base + t, theta) for h in range(nkv)])
        o = r.gqa_step(c, q, k, V[t], nh)
        OUT[t] = o * np.array([sigmoid(x) for x in gate], np.float32)
    r.kv_free(c)
    save(name, nh=nh, nkv=nkv, hd=hd, rope_dim=rot, theta=np.float32(theta), base=base,
         q_norm_w=qw, k_norm_w=kw_, QP=QP, K=K, V=V, OUT=OUT, quantized=quantized)


# ---- quantised projection: the reference's Q8_K quantiser and Q8_0 x Q8_K integer dot ------------
def projection():
    """src/ornith_qdot.c:38-70 (qdot_quantize_row_q8_K) and :144-163 (vec_dot_q8_0), driven as matmul_batch_q
    drives them (src/ornith_rforward.c:165-175, :108-115): 6 activation rows of 768 through 33 Q8_0 weight rows,
    with a zero block, ties for the maximum and values on rounding boundaries."""
    g = np.random.default_rng(21)
    n_in, n_out, T = 768, 33, 6
    X = g.standard_normal((T, n_in)).astype(np.float32)
    X[0, :256] = 0.0
    X[1, 5] = 9.0; X[1, 100] = -9.0
    X[2, 300] = -8.0; X[2, 290] = 8.0
    X[3] = np.round(X[3] * 4) / 4
    Wf = (g.standard_normal((n_out, n_in)) * 0.05).astype(np.float32)
    W = np.stack([r.q8_0_encode(row) for row in Wf])
    save("projection_q8_0.npz", X=X, W=W, n_in=n_in, blocks=r.q8k_quantize(X), Y=r.matmul_q8_0(W, n_in, X))


def projection_kquant():
    """The k-quant integer dots (src/ornith_qdot.c:75-105 vec_dot_q4_K, :109-141 vec_dot_q6_K) over rows from the
    reference's own encoder (oq_quantize, src/ornith_quant.c): 5 activation rows of 2048 through 72 weight rows."""
    from oracle.oracle import GGML_Q4_K, GGML_Q6_K
    g = np.random.default_rng(22)
    n_in, n_out, T = 2048, 72, 5
    X = g.standard_normal((T, n_in)).astype(np.float32)
    X[0, 256:512] = 0.0
    X[1, 5] = 9.0; X[1, 100] = -9.0
    Wf = (g.standard_normal((n_out, n_in)) * 0.05).astype(np.float32)
    Wf[7] = 0.0
    W4, W6 = r.quantize_rows(GGML_Q4_K, Wf), r.quantize_rows(GGML_Q6_K, Wf)
    save("projection_kquant.npz", X=X, n_in=n_in, W_q4_k=W4, W_q6_k=W6,
         Y_q4_k=r.matmul_q(GGML_Q4_K, W4, n_in, X), Y_q6_k=r.matmul_q(GGML_Q6_K, W6, n_in, X))


if __name__ == "__main__":
    projection()
    projection_kquant()
    delta_parity()
    gqa(42, 4, 2, 8, 11, "attn_gqa.npz", 0)
    gqa(123, 4, 2, 16, 13, "attn_gqa_int8.npz", 1)
    conv()
    codecs()
    delta_head128()
    linear_layer("linear_layer_tiled.npz", 0, False, True, 11)
    linear_layer("linear_layer_grouped.npz", 1, True, False, 12)
    full_layer("full_layer_f32.npz", 0, 21)
    full_layer("full_layer_int8.npz", 1, 22)
