"""The CPU oracle against (a) the committed golden vectors produced by the
reference's own code, (b) the known-answer values in the reference's tests
(tests/test_tensor.c:39-117, tests/test_quant.c:108-143, tests/test_attn.c) and
(c) the reference objects themselves where they were built (oracle/_ref)."""
import math

import numpy as np
import pytest

from oracle.oracle import (HEADMAP_GROUPED, HEADMAP_TILED, KV_F32, KV_INT8_HEAD, KV_Q8_0,
                           FullLayer, LinearLayer, Ref)


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---- known answers restated from tests/test_tensor.c ---------------------------
def test_tensor_known_answers(oracle):
    out = oracle.rmsnorm(np.array([1, 2, 3, 4], np.float32), None, 0.0)
    rms = math.sqrt(7.5)
    assert abs(out[0] - 1 / rms) < 1e-5 and abs(out[3] - 4 / rms) < 1e-5          # :39-47
    s = oracle.softmax([1, 2, 3])
    z = math.exp(-2) + math.exp(-1) + 1
    assert abs(s.sum() - 1) < 1e-6 and s[2] > s[1] > s[0] and abs(s[0] - math.exp(-2) / z) < 1e-5
    assert abs(oracle.sigmoid(0) - 0.5) < 1e-6 and abs(oracle.silu(0)) < 1e-6      # :61-64
    assert abs(oracle.silu(1) - 0.7310586) < 1e-5
    v = np.array([0.3, -0.7, 1.1, 0.5], np.float32)                                # :72-85
    w = oracle.rope_partial(v, 4, 5, 10000.0)
    assert abs(np.linalg.norm(v) - np.linalg.norm(w)) < 1e-4
    assert (oracle.rope_partial([1, 2, 3, 4], 4, 0, 10000.0) == np.array([1, 2, 3, 4], np.float32)).all()
    assert abs(oracle.softplus(0.0) - 0.6931472) < 1e-5                            # :87-94
    assert abs(oracle.softplus(100.0) - 100.0) < 1e-3
    assert 0 <= oracle.softplus(-100.0) < 1e-3
    y = oracle.l2norm_eps(np.array([3, 4, 0, 0], np.float32), 0.0)                 # :96-107
    assert abs(y[0] - 0.6) < 1e-5 and abs(y[1] - 0.8) < 1e-5
    assert oracle.l2norm_eps(np.array([1e-4, 0], np.float32), 1e-6)[0] < 1.0
    a, _ = oracle.rng_fill(123, 8, -1, 1)
    b, _ = oracle.rng_fill(123, 8, -1, 1)
    assert (a == b).all()


# ---- known answers restated from tests/test_quant.c:108-143 ---------------------
def test_quant_known_answers(oracle):
    assert oracle.q8_0_encode(np.zeros(64, np.float32)).size == 68
    with pytest.raises(ValueError):
        oracle.q8_0_encode(np.zeros(7, np.float32))
    for x in (1.0, -0.5, 0.0):
        assert oracle.f16_to_f32(oracle.f32_to_f16(x)) == x
    rel = max(abs(oracle.f16_to_f32(oracle.f32_to_f16(i * 0.137)) - np.float32(i * 0.137)) / (i * 0.137)
              for i in range(1, 1001))
    assert rel < 1e-3
    src = (np.sin(np.arange(64) * np.float32(0.3)) * 5.0).astype(np.float32)
    deq = oracle.q8_0_decode(oracle.q8_0_encode(src))
    assert np.abs(deq - src).max() <= np.abs(src).max() / 127.0 + 1e-4
    assert oracle.lib.orc_kv_bytes_per_token(2, 16, KV_INT8_HEAD) * 2 <= oracle.lib.orc_kv_bytes_per_token(2, 16, KV_F32)
    assert oracle.lib.orc_kv_bytes_per_token(2, 256, KV_Q8_0) == 1088


# ---- golden vectors produced by the reference -------------------------------------
def test_codec_goldens_bit_exact(oracle, golden):
    g = golden("q8_0_vectors.npz")
    assert (oracle.q8_0_encode(g["x"]) == g["bytes"]).all()
    assert (bits(oracle.q8_0_decode(g["bytes"])) == bits(g["decoded"])).all()
    f = golden("f16_vectors.npz")
    assert [oracle.f32_to_f16(v) for v in f["f"]] == list(f["h"])
    back = np.array([oracle.f16_to_f32(h) for h in range(65536)], np.float32).view(np.uint32)
    assert (back == f["all_h_to_f32_bits"]).all()
    k = golden("kv_int8_vectors.npz")
    for row, codes, scale in zip(k["x"], k["codes"], k["scales"]):
        q, s = oracle.kv_int8_encode(row)
        assert (q == codes).all() and s == scale


def test_delta_goldens(oracle, golden):
    g = golden("attn_delta_parity.npz")                       # tests/test_attn.c:28-83
    T = g["alpha"].size
    S = np.zeros_like(g["S_final"])
    O = np.stack([oracle.delta_step(S, g["Q"][t], g["K"][t], g["V"][t], g["alpha"][t], g["beta"][t])
                  for t in range(T)])
    assert (bits(O) == bits(g["O_step"])).all() and (bits(S) == bits(g["S_final"])).all()
    for chunk in (1, 2, 3, 4, 5, 8, 16, T):                   # the reference's chunk list, tol 2e-4
        Sp = np.zeros_like(S)
        Op = oracle.delta_prefill(Sp, g["Q"], g["K"], g["V"], g["alpha"], g["beta"], chunk)
        assert np.abs(Op - O).max() < 2e-4 and np.abs(Sp - S).max() < 2e-4
    Sp = np.zeros_like(S)                                      # split prefill, carried state (:70-80)
    Oa = oracle.delta_prefill(Sp, g["Q"][:7], g["K"][:7], g["V"][:7], g["alpha"][:7], g["beta"][:7], 3)
    Ob = oracle.delta_prefill(Sp, g["Q"][7:].copy(), g["K"][7:].copy(), g["V"][7:].copy(),
                              g["alpha"][7:].copy(), g["beta"][7:].copy(), 4)
    assert np.abs(np.vstack([Oa, Ob]) - O).max() < 2e-4
    h = golden("delta_head128.npz")
    S = np.zeros_like(h["S_final"])
    O = np.stack([oracle.delta_step(S, h["Q"][t], h["K"][t], h["V"][t], h["alpha"][t], h["beta"][t])
                  for t in range(h["alpha"].size)])
    assert (bits(O) == bits(h["O_step"])).all() and (bits(S) == bits(h["S_final"])).all()
    S = np.zeros_like(S)
    O = oracle.delta_prefill(S, h["Q"], h["K"], h["V"], h["alpha"], h["beta"], 8)
    assert (bits(O) == bits(h["O_chunk8"])).all() and (bits(S) == bits(h["S_chunk8"])).all()


def test_gqa_goldens(oracle, golden):
    g = golden("attn_gqa.npz")                                 # tests/test_attn.c:87-119
    nh, nkv, hd = int(g["nh"]), int(g["nkv"]), int(g["hd"])
    T = g["Q"].shape[0]
    assert (bits(oracle.gqa_reference(g["Q"], g["K"], g["V"], T, nh, nkv, hd)) == bits(g["O_naive"])).all()
    kv = oracle.kv(T, nkv, hd, KV_F32)
    O = np.stack([oracle.gqa_step(kv, g["Q"][t], g["K"][t], g["V"][t], nh) for t in range(T)])
    assert (bits(O) == bits(g["O_step"])).all()
    assert np.abs(O - g["O_naive"]).max() < 1e-5
    kv1 = oracle.kv(1, nkv, hd, KV_F32)                        # T=1 returns V (:108-115)
    o1 = oracle.gqa_step(kv1, g["Q"][0], g["K"][0], g["V"][0], nh)
    assert np.abs(o1[:hd] - g["V"][0][:hd]).max() < 1e-5
    full = oracle.gqa_step(kv1, g["Q"][0], g["K"][0], g["V"][0], nh)   # full cache: silent no-op
    assert kv1.len == 1 and (full == 0).all()

    q = golden("attn_gqa_int8.npz")                            # tests/test_attn.c:123-158
    nh, nkv, hd = int(q["nh"]), int(q["nkv"]), int(q["hd"])
    T = q["Q"].shape[0]
    kv = oracle.kv(T, nkv, hd, KV_INT8_HEAD)
    O = np.stack([oracle.gqa_step(kv, q["Q"][t], q["K"][t], q["V"][t], nh) for t in range(T)])
    assert (bits(O) == bits(q["O_step"])).all()
    assert np.abs(O - q["O_naive"]).max() < 5e-2
    Kq, Vq, Ks, Vs = kv.rows_int8()
    assert (Kq == q["Kq"]).all() and (Vq == q["Vq"]).all() and (Ks == q["Ks"]).all() and (Vs == q["Vs"]).all()


def test_conv_golden(oracle, golden):
    g = golden("attn_conv.npz")                                # tests/test_attn.c:162-192
    K, (T, Cn) = 4, g["X"].shape
    buf = np.zeros((K - 1) * Cn, np.float32)
    OUT = oracle.conv_prefill(buf, K, g["X"], g["w"], g["b"])
    assert (bits(OUT) == bits(g["OUT"])).all() and (bits(buf) == bits(g["buf_final"].ravel())).all()
    buf2 = np.zeros_like(buf)
    steps = np.stack([oracle.conv_step(buf2, K, g["X"][t].copy(), g["w"], g["b"]) for t in range(T)])
    assert np.abs(steps - OUT).max() < 1e-6
    expect = g["b"] + g["w"][:, K - 1] * g["X"][0]             # causality at t = 0
    assert np.abs(OUT[0] - expect).max() < 1e-5


@pytest.mark.parametrize("name", ["linear_layer_tiled.npz", "linear_layer_grouped.npz"])
def test_linear_layer_goldens(oracle, golden, name):
    g = golden(name)
    layer = LinearLayer(int(g["nk"]), int(g["nv"]), int(g["dk"]), int(g["dv"]), g["conv_w"], g["a_coef"],
                        g["dt_bias"], g["norm_w"], conv_b=g["conv_b"] if g["conv_b"].size else None,
                        head_map=int(g["head_map"]), out_scale=None if int(g["scaled"]) else 1.0)
    T = g["QKV"].shape[0]
    S = np.zeros_like(g["S_final"]); buf = np.zeros(g["conv_final"].size, np.float32)
    OUT = np.stack([oracle.linear_attn_step(layer, S, buf, g["QKV"][t], g["A"][t], g["B"][t], g["Z"][t])
                    for t in range(T)])
    assert (bits(OUT) == bits(g["OUT"])).all()
    assert (bits(S) == bits(g["S_final"])).all() and (bits(buf) == bits(g["conv_final"].ravel())).all()
    for chunk in (1, 5, 32):                                   # chunked prefill == steps
        S2 = np.zeros_like(S); buf2 = np.zeros_like(buf)
        O2 = oracle.linear_attn_prefill(layer, S2, buf2, g["QKV"], g["A"], g["B"], g["Z"], chunk)
        assert np.abs(O2 - OUT).max() / np.abs(OUT).max() < 2e-4
        assert np.abs(S2 - S).max() < 2e-4 and (buf2 == buf).all()


@pytest.mark.parametrize("name,mode", [("full_layer_f32.npz", KV_F32), ("full_layer_int8.npz", KV_INT8_HEAD)])
def test_full_layer_goldens(oracle, golden, name, mode):
    g = golden(name)
    layer = FullLayer(int(g["nh"]), int(g["nkv"]), int(g["hd"]), g["q_norm_w"], g["k_norm_w"],
                      rope_dim=int(g["rope_dim"]), theta=float(g["theta"]))
    T = g["QP"].shape[0]
    kv = oracle.kv(T, layer.nkv, layer.hd, mode)
    OUT = np.stack([oracle.full_attn_step(layer, kv, int(g["base"]) + t, g["QP"][t], g["K"][t], g["V"][t])
                    for t in range(T)])
    assert (bits(OUT) == bits(g["OUT"])).all()
    kv2 = oracle.kv(T, layer.nkv, layer.hd, mode)
    assert (oracle.full_attn_prefill(layer, kv2, int(g["base"]), g["QP"], g["K"], g["V"]) == OUT).all()


def test_q8_0_kv_mode_is_the_stated_composition(oracle):
    """Q8_0 KV mode == encode -> decode -> f32 attention, bytes kept."""
    rng = np.random.default_rng(3)
    nh, nkv, hd, T = 4, 2, 64, 9
    Q = rng.standard_normal((T, nh * hd)).astype(np.float32)
    K = rng.standard_normal((T, nkv * hd)).astype(np.float32)
    V = rng.standard_normal((T, nkv * hd)).astype(np.float32)
    a, b = oracle.kv(T, nkv, hd, KV_Q8_0), oracle.kv(T, nkv, hd, KV_F32)
    for t in range(T):
        kd = oracle.q8_0_decode(oracle.q8_0_encode(K[t])); vd = oracle.q8_0_decode(oracle.q8_0_encode(V[t]))
        assert (oracle.gqa_step(a, Q[t], K[t], V[t], nh) == oracle.gqa_step(b, Q[t], kd, vd, nh)).all()
    Kb, Vb = a.rows_q8_0()
    assert (Kb.reshape(T, -1) == np.stack([oracle.q8_0_encode(K[t]) for t in range(T)])).all()


@pytest.mark.skipif(not Ref.available(), reason="reference objects not built on this machine")
def test_oracle_equals_reference_objects(oracle):
    """Seeded comparison against the reference's own compiled code, bit for bit."""
    r = Ref()
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(32 * 2000) * 3).astype(np.float32)
    assert (oracle.q8_0_encode(x) == r.q8_0_encode(x)).all()
    for v in (rng.standard_normal(5000) * 10.0 ** rng.integers(-9, 6, 5000)).astype(np.float32):
        assert oracle.f32_to_f16(v) == r.lib.oq_f32_to_f16(float(v))
    dk = dv = 64; T = 33
    Q = rng.standard_normal((T, dk)).astype(np.float32) / 8
    K = rng.standard_normal((T, dk)).astype(np.float32) / 8
    V = rng.standard_normal((T, dv)).astype(np.float32)
    al = rng.uniform(0.3, 0.999, T).astype(np.float32); be = rng.uniform(0.1, 0.9, T).astype(np.float32)
    for chunk in (1, 7, 32, 64):
        S1 = np.zeros((dv, dk), np.float32); S2 = S1.copy()
        assert (oracle.delta_prefill(S1, Q, K, V, al, be, chunk) == r.delta_prefill(S2, Q, K, V, al, be, chunk)).all()
        assert (S1 == S2).all()
    nh, nkv, hd, T = 8, 2, 32, 17
    Qs = rng.standard_normal((T, nh * hd)).astype(np.float32)
    Ks = rng.standard_normal((T, nkv * hd)).astype(np.float32)
    Vs = rng.standard_normal((T, nkv * hd)).astype(np.float32)
    for mode, quant in ((KV_F32, 0), (KV_INT8_HEAD, 1)):
        kv = oracle.kv(T, nkv, hd, mode); rc = r.kv_init(T, nkv, hd, quant)
        for t in range(T):
            assert (oracle.gqa_step(kv, Qs[t], Ks[t], Vs[t], nh) == r.gqa_step(rc, Qs[t], Ks[t], Vs[t], nh)).all()
        r.kv_free(rc)


@pytest.mark.skipif(not Ref.available(), reason="reference objects not built on this machine")
def test_projection_oracle_equals_reference_objects(oracle):
    """Q8_K quantiser and the Q8_0 x Q8_K integer dot: the restatement against the reference's own objects, bit
    for bit, on rows with zero blocks, ties for the maximum and values on rounding boundaries."""
    ref = Ref()
    orc = oracle
    g = np.random.default_rng(21)
    n_in, n_out, T = 768, 33, 6
    X = g.standard_normal((T, n_in)).astype(np.float32)
    X[0, :256] = 0.0
    X[1, 5] = 9.0; X[1, 100] = -9.0
    X[2, 300] = -8.0; X[2, 290] = 8.0
    X[3] = np.round(X[3] * 4) / 4
    assert (orc.q8k_quantize(X) == ref.q8k_quantize(X)).all()
    W = np.stack([orc.q8_0_encode(r) for r in (g.standard_normal((n_out, n_in)) * 0.05).astype(np.float32)])
    a, b = orc.matmul_q8_0(W, n_in, X), ref.matmul_q8_0(W, n_in, X)
    assert (a.view(np.uint32) == b.view(np.uint32)).all()


def test_projection_golden_bit_exact(oracle, golden):
    """The reference-made projection fixture (tests/golden/make_golden.py::projection): blocks and outputs."""
    g = golden("projection_q8_0.npz")
    assert (oracle.q8k_quantize(g["X"]) == g["blocks"]).all()
    y = oracle.matmul_q8_0(g["W"], int(g["n_in"]), g["X"])
    assert (bits(y) == bits(g["Y"])).all()


@pytest.mark.skipif(not Ref.available(), reason="reference objects not built on this machine")
@pytest.mark.parametrize("wtype", ["q8_0", "q4_k", "q6_k"])
def test_kquant_dots_equal_reference_objects(oracle, wtype):
    """The integer dots of all three weight types (src/ornith_qdot.c:75-163) against the reference's own objects,
    bit for bit: rows from the reference's encoder, and rows of random block bytes (every code, sub-block scale
    and minimum occurs; finite f16 scales)."""
    from oracle import oracle as O
    ref = Ref()
    wt = {"q8_0": O.GGML_Q8_0, "q4_k": O.GGML_Q4_K, "q6_k": O.GGML_Q6_K}[wtype]
    g = np.random.default_rng(31 + wt)
    n_in, n_out, T = 1024, 24, 5
    X = g.standard_normal((T, n_in)).astype(np.float32)
    X[0, :256] = 0.0
    W = ref.quantize_rows(wt, (g.standard_normal((n_out, n_in)) * 0.05).astype(np.float32))
    assert W.shape[1] == O.QROW_BYTES[wt](n_in)
    assert (bits(oracle.matmul_q(wt, W, n_in, X)) == bits(ref.matmul_q(wt, W, n_in, X))).all()
    Wr = g.integers(0, 256, W.shape, dtype=np.uint8)
    blk = Wr.reshape(n_out, n_in // (32 if wt == O.GGML_Q8_0 else 256), -1)
    for col in {O.GGML_Q8_0: (1,), O.GGML_Q4_K: (1, 3), O.GGML_Q6_K: (209,)}[wt]:
        blk[:, :, col] &= 0x3B                                       # f16 exponent below 15: finite, |d| < 1
    a, b = oracle.matmul_q(wt, Wr, n_in, X), ref.matmul_q(wt, Wr, n_in, X)
    assert np.isfinite(a).all() and (bits(a) == bits(b)).all()


def test_kquant_golden_bit_exact(oracle, golden):
    """The reference-made k-quant fixture (tests/golden/make_golden.py::projection_kquant)."""
    from oracle import oracle as O
    g = golden("projection_kquant.npz")
    for name, wt in (("q4_k", O.GGML_Q4_K), ("q6_k", O.GGML_Q6_K)):
        y = oracle.matmul_q(wt, g["W_" + name], int(g["n_in"]), g["X"])
        assert (bits(y) == bits(g["Y_" + name])).all(), name


def _dequant_q4_k(rows, n):
    """Q4_K rows -> f32 by the format's definition: value = d * scale_j * code - dmin * min_j (144-byte super-blocks:
    f16 d, f16 dmin, 12 bytes of 6-bit (scale, min) pairs, 128 bytes of 4-bit codes)."""
    blk = rows.reshape(rows.shape[0], n // 256, 144)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    dmin = blk[:, :, 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    sc = blk[:, :, 4:16].astype(np.int32)
    scale = np.empty(blk.shape[:2] + (8,), np.int32); mn = np.empty_like(scale)
    for j in range(8):
        if j < 4:
            scale[..., j] = sc[..., j] & 63; mn[..., j] = sc[..., j + 4] & 63
        else:
            scale[..., j] = (sc[..., j + 4] & 15) | ((sc[..., j - 4] >> 6) << 4)
            mn[..., j] = (sc[..., j + 4] >> 4) | ((sc[..., j] >> 6) << 4)
    qs = blk[:, :, 16:144].astype(np.int32).reshape(blk.shape[0], blk.shape[1], 4, 32)
    codes = np.stack([qs & 15, qs >> 4], axis=3).reshape(blk.shape[0], blk.shape[1], 8, 32)     # sub-blocks 2p, 2p+1
    w = d[..., None, None] * scale[..., None] * codes - dmin[..., None, None] * mn[..., None]
    return w.reshape(rows.shape[0], n).astype(np.float64)


def _dequant_q6_k(rows, n):
    """Q6_K rows -> f32: value = d * sc[e / 16] * (code - 32) (210-byte super-blocks: 128 low nibbles, 64 bytes of
    2-bit high parts, 16 int8 scales, f16 d)."""
    blk = rows.reshape(rows.shape[0], n // 256, 210)
    ql = blk[:, :, 0:128].astype(np.int32); qh = blk[:, :, 128:192].astype(np.int32)
    sc = blk[:, :, 192:208].copy().view(np.int8).astype(np.int32)
    d = blk[:, :, 208:210].copy().view(np.float16).astype(np.float32)[..., 0]
    w = np.empty(blk.shape[:2] + (256,), np.float64)
    for e in range(256):
        h, c, l = e // 128, (e % 128) // 32, e % 32
        lo = (ql[..., 64 * h + 32 * (c % 2) + l] >> (4 * (c // 2))) & 15
        hi = (qh[..., 32 * h + l] >> (2 * c)) & 3
        w[..., e] = d * sc[..., e // 16] * ((lo | (hi << 4)) - 32)
    return w.reshape(rows.shape[0], n)


@pytest.mark.parametrize("wtype", ["q4_k", "q6_k"])
def test_kquant_dots_against_the_format_definition(oracle, wtype):
    """Independent of the reference's integer dot: dequantise random blocks by the format's definition in numpy,
    dequantise the Q8_K activations (d * code), and compare the plain dot product with the oracle's integer path.
    The two differ only by f32 rounding of the per-super-block terms."""
    from oracle import oracle as O
    wt = {"q4_k": O.GGML_Q4_K, "q6_k": O.GGML_Q6_K}[wtype]
    g = np.random.default_rng(71 + wt)
    n_in, n_out, T = 1024, 16, 4
    W = g.integers(0, 256, (n_out, O.QROW_BYTES[wt](n_in)), dtype=np.uint8)
    blk = W.reshape(n_out, n_in // 256, -1)
    for col in {O.GGML_Q4_K: (1, 3), O.GGML_Q6_K: (209,)}[wt]:
        blk[:, :, col] &= 0x3B
    X = g.standard_normal((T, n_in)).astype(np.float32)
    q = oracle.q8k_quantize(X)                                      # [T][n_in/256][292]
    d = q[:, :, 0:4].copy().view(np.float32)[..., 0]
    codes = q[:, :, 4:260].copy().view(np.int8).astype(np.float64)
    act = (d[..., None].astype(np.float64) * codes).reshape(T, n_in)
    w = (_dequant_q4_k if wt == O.GGML_Q4_K else _dequant_q6_k)(W, n_in)
    want = act @ w.T
    got = oracle.matmul_q(wt, W, n_in, X)
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max(), float(np.abs(got - want).max() / np.abs(want).max())
