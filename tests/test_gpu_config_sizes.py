"""Parity at the workload sizes the task names, against the CPU oracle (never against another GPU path).

* one 35B-shaped gated delta-net layer, f32: prefill 512 tokens, then 128 decode steps (seed 0)
* one 35B-shaped GQA layer, f32 activations: prefill 4096 tokens, then 256 decode steps, once with an
  f32 cache and once with a Q8_0 cache (seed 1); the cache bytes are compared with the oracle's
* 512 consecutive GQA decode steps
* the 32768-token prompt of the long-prefill workload, sampled: a few delta-net heads over the whole
  prompt against 32768 CPU steps; the tensor-core GQA prefill at a handful of query positions
* the per-GPU shard shapes of the 8-GPU head-sharded decode (4 query heads over 1 KV head at an 8192-token
  context; 8 value / 8 key heads)
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from tests._cases import TOL, bf16_round, device_full, device_linear, full_case, full_inputs, linear_case, linear_inputs, rel_err

pytestmark = pytest.mark.gpu
TOL_BF16_IO = TOL + 2.0 ** -9 + 5e-4     # bf16-stored outputs: half an ulp on top of the bar


def _note(case, **kw):
    """Worst errors of a case, printed for the record (`pytest -s` shows them)."""
    print("parity:", case, " ".join(f"{k}={v:.3g}" for k, v in kw.items()))


def _t(x, dt=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dt is None else t.to(dt)


def test_delta_net_layer_prefill_512_then_128_steps(oracle):
    """16 key / 32 value heads x 128, f32 activations, zero initial state, seed 0: the prefill output of every
    token, the output of every decode step, the final recurrent state (2e-3) and the conv history (bit-exact)."""
    import torch
    from ornithology_b200 import device as D
    layer, kw = linear_case(0)
    dl = device_linear(layer, kw)
    T, steps = 512, 128
    QKV, A, Bm, Z = linear_inputs(0, layer, T + steps)
    S = np.zeros((layer.nv, 128, 128), np.float32); buf = np.zeros(3 * layer.cc, np.float32)
    st = D.LinearState(dl, 1)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = oracle.linear_attn_prefill(layer, S, buf, QKV[:T], A[:T], Bm[:T], Z[:T], chunk=64)
    out = D.linear_attn_prefill(dl, st, pos, _t(QKV[:T])[None], _t(A[:T])[None], _t(Bm[:T])[None], _t(Z[:T])[None], T, chunk=64)
    worst = rel_err(out.cpu().numpy()[0], ref)
    assert worst < TOL, worst
    assert rel_err(st.S.cpu().numpy()[0], S) < TOL
    D.advance(pos, T)
    assert (st.conv_image(0, T).cpu().numpy().ravel().view(np.uint32) == buf.view(np.uint32)).all()
    dQ, dA, dB, dZ = _t(QKV), _t(A), _t(Bm), _t(Z)
    for t in range(T, T + steps):
        out = D.linear_attn_step(dl, st, pos, dQ[t:t + 1], dA[t:t + 1], dB[t:t + 1], dZ[t:t + 1])
        ref = oracle.linear_attn_step(layer, S, buf, QKV[t], A[t], Bm[t], Z[t])
        worst = max(worst, rel_err(out.cpu().numpy()[0], ref))
        D.advance(pos)
    assert worst < TOL, worst
    _note("delta-net 512+128", out=worst, state=rel_err(st.S.cpu().numpy()[0], S))
    assert rel_err(st.S.cpu().numpy()[0], S) < TOL
    assert (st.conv_image(0, T + steps).cpu().numpy().ravel().view(np.uint32) == buf.view(np.uint32)).all()


@pytest.mark.parametrize("mode", ["f32", "q8_0"])
def test_gqa_layer_prefill_4096_then_256_steps(oracle, mode):
    """16 query / 2 KV heads x 256, f32 activations, seed 1: causal prefill of 4096 tokens, 256 decode steps.  The
    oracle runs the engine's path (one ornith_gqa_step per token).  Outputs within 2e-3; the cache rows — after
    k RMSNorm, partial RoPE and, for Q8_0, the codec — are compared with the oracle's: V rows and the Q8_0 K rows
    byte for byte, f32 K rows bit for bit outside the rotated dims and to the last place inside them."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(1)
    dl = device_full(layer)
    T, steps = 4096, 256
    dm, om = {"f32": (D.KV_F32, O.KV_F32), "q8_0": (D.KV_Q8_0, O.KV_Q8_0)}[mode]
    QP, K, V = full_inputs(1, layer, T + steps)
    kv = D.KvBatch(dm, layer.nkv, layer.hd, [T + steps])
    okv = oracle.kv(T + steps, layer.nkv, layer.hd, om)
    kv_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = oracle.full_attn_prefill(layer, okv, 0, QP[:T], K[:T], V[:T])
    out = D.full_attn_prefill(dl, kv, kv_len, _t(QP[:T])[None], _t(K[:T])[None], _t(V[:T])[None], T)
    worst = rel_err(out.cpu().numpy()[0], ref)
    assert worst < TOL, worst
    D.advance(kv_len, T)
    dQ, dK, dV = _t(QP), _t(K), _t(V)
    for t in range(T, T + steps):
        out = D.full_attn_step(dl, kv, kv_len, dQ[t:t + 1], dK[t:t + 1], dV[t:t + 1], max_len=T + steps)
        ref = oracle.full_attn_step(layer, okv, t, QP[t], K[t], V[t])
        worst = max(worst, rel_err(out.cpu().numpy()[0], ref))
        D.advance(kv_len)
    assert worst < TOL, worst
    _note("gqa 4096+256 " + mode, out=worst)
    n = T + steps
    Kg, Vg = kv.rows(0, n)
    Ko, Vo = okv.rows_q8_0() if mode == "q8_0" else okv.rows_f32()
    Ko = np.asarray(Ko)[:n].reshape(Kg.shape); Vo = np.asarray(Vo)[:n].reshape(Vg.shape)
    assert (Vg.view(np.uint8) == Vo.view(np.uint8)).all(), "V rows differ"
    if mode == "q8_0":
        dk = int((Kg != Ko).sum())
        assert dk == 0, f"{dk} of {Kg.size} K bytes differ"
    else:
        # f32 rows: everything but the 64 rotated dims is bit-exact; the rotated dims go through the device's sincosf
        # where the CPU uses libm's cosf / sinf, which differ in the last place for some angles
        rot = layer.rope_dim
        assert (Kg[..., rot:].view(np.uint32) == Ko[..., rot:].view(np.uint32)).all(), "non-rotated K dims differ"
        a, b = Kg[..., :rot].astype(np.float64), Ko[..., :rot].astype(np.float64)
        assert np.abs(a - b).max() <= 4e-7 * np.abs(b).max(), "rotated K dims differ by more than a few ulp"
        frac = float((Kg[..., :rot].view(np.uint32) != Ko[..., :rot].view(np.uint32)).mean())
        _note("gqa f32 K rows, rotated dims", worst=float(np.abs(a - b).max() / np.abs(b).max()), fraction_differing=frac,
              bytes_differing=float((Kg.view(np.uint8) != Ko.view(np.uint8)).sum()), bytes=float(Kg.view(np.uint8).size))
        assert frac < 0.2, f"{frac:.3f} of the rotated values differ in the last place"


def test_gqa_512_consecutive_decode_steps(oracle):
    """The stated bar for decode: within 2e-3 at every one of 512 consecutive steps (Q8_0 cache, from empty)."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(3)
    dl = device_full(layer)
    steps = 512
    QP, K, V = full_inputs(33, layer, steps)
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [steps])
    okv = oracle.kv(steps, layer.nkv, layer.hd, O.KV_Q8_0)
    kv_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    dQ, dK, dV = _t(QP), _t(K), _t(V)
    worst = 0.0
    for t in range(steps):
        out = D.full_attn_step(dl, kv, kv_len, dQ[t:t + 1], dK[t:t + 1], dV[t:t + 1], max_len=steps)
        ref = oracle.full_attn_step(layer, okv, t, QP[t], K[t], V[t])
        worst = max(worst, rel_err(out.cpu().numpy()[0], ref))
        D.advance(kv_len)
    assert worst < TOL, worst
    _note("gqa 512 decode steps", out=worst)
    Kg, Vg = kv.rows(0, steps)
    Ko, Vo = okv.rows_q8_0()
    assert (Kg == np.asarray(Ko)[:steps].reshape(Kg.shape)).all() and (Vg == np.asarray(Vo)[:steps].reshape(Vg.shape)).all()


def test_delta_net_32768_token_prompt_sampled_heads(oracle):
    """The long-prefill workload for a sample of heads: 2 key / 4 value heads x 128 over a 32768-token prompt, bf16
    activations, in one call of the tensor-core scan (512 chunks), against the CPU scan of the same tokens: every
    output row and the final state."""
    import torch
    from ornithology_b200 import device as D
    layer, kw = linear_case(2, nk=2, nv=4)
    dl = device_linear(layer, kw)
    T = 32768
    QKV, A, Bm, Z = linear_inputs(22, layer, T, bf16=True)
    S = np.zeros((layer.nv, 128, 128), np.float32); buf = np.zeros(3 * layer.cc, np.float32)
    ref = oracle.linear_attn_prefill(layer, S, buf, QKV, A, Bm, Z, chunk=64)
    st = D.LinearState(dl, 1)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    bf = torch.bfloat16
    out = D.linear_attn_prefill(dl, st, pos, _t(QKV, bf)[None], _t(A, bf)[None], _t(Bm, bf)[None], _t(Z, bf)[None], T, chunk=64)
    out = out.float().cpu().numpy()[0]
    _note("delta-net 32768 tokens bf16", out=rel_err(out, ref), tail=rel_err(out[-2048:], ref[-2048:]),
          state=rel_err(st.S.cpu().numpy()[0], S), bar=TOL_BF16_IO)
    assert rel_err(out, ref) < TOL_BF16_IO
    # the tail of the prompt on its own scale (errors must not build up over 512 chunks)
    assert rel_err(out[-2048:], ref[-2048:]) < TOL_BF16_IO
    assert rel_err(st.S.cpu().numpy()[0], S) < TOL
    assert (st.conv_image(0, T).cpu().numpy().ravel().view(np.uint32) == buf.view(np.uint32)).all()


def _q8_0_rows_to_f32(rows):
    """[..., 8, 34] Q8_0 bytes -> [..., 256] f32, the codec's own arithmetic (code x f16 scale, one multiply)."""
    rows = np.ascontiguousarray(rows)
    blocks = rows.reshape(-1, 34)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    q = blocks[:, 2:].copy().view(np.int8).astype(np.float32)
    return (q * d).reshape(rows.shape[:-2] + (rows.shape[-2] * 32,))


def test_gqa_prefill_32768_tokens_sampled_positions(oracle):
    """The tensor-core prefill over a 32768-token prompt (4 query heads over 1 KV head — one GPU's share of the
    8-GPU plan — bf16 activations, Q8_0 cache), checked against the oracle's decode step at query positions at
    both ends of the first tile, mid-prompt and at the last token.  The oracle attends over the rows the append
    kernel stored (their bytes are pinned by the codec tests) and appends its own row for the query position."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(4, nh=4, nkv=1)
    dl = device_full(layer)
    T = 32768
    QP, K, V = full_inputs(44, layer, T, bf16=True)
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [T])
    kv_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    bf = torch.bfloat16
    out = D.full_attn_prefill(dl, kv, kv_len, _t(QP, bf)[None], _t(K, bf)[None], _t(V, bf)[None], T).float().cpu().numpy()[0]
    Kb, Vb = kv.rows(0, T)                       # [T][1][8][34] bytes
    Kd, Vd = _q8_0_rows_to_f32(Kb.reshape(T, 1, 8, 34)), _q8_0_rows_to_f32(Vb.reshape(T, 1, 8, 34))
    worst = 0.0
    for p in (0, 1, 127, 128, 4095, 16383, 32767):
        okv = oracle.kv(p + 1, layer.nkv, layer.hd, O.KV_Q8_0)
        if p:
            kb = np.ascontiguousarray(Kb[:p]); vb = np.ascontiguousarray(Vb[:p])
            kd = np.ascontiguousarray(Kd[:p]); vd = np.ascontiguousarray(Vd[:p])
            C.memmove(okv.c.Kb, kb.ctypes.data, kb.size); C.memmove(okv.c.Vb, vb.ctypes.data, vb.size)
            C.memmove(okv.c.K, kd.ctypes.data, kd.nbytes); C.memmove(okv.c.V, vd.ctypes.data, vd.nbytes)
        okv.c.len = p
        ref = oracle.full_attn_step(layer, okv, p, QP[p], K[p], V[p])
        Ko, _ = okv.rows_q8_0()
        assert (np.asarray(Ko)[p].reshape(-1) == Kb[p].reshape(-1)).all(), f"row {p}: the appended K row differs from the oracle's"
        worst = max(worst, rel_err(out[p], ref))
        assert rel_err(out[p], ref) < TOL_BF16_IO, p
    _note("gqa prefill 32768 tokens bf16, sampled rows", out=worst, bar=TOL_BF16_IO)


def test_head_sharded_decode_shard_shapes(oracle):
    """One GPU's share of the 8-GPU head-sharded decode at the 397B shape: a full-attention layer with 4 query heads
    over 1 KV head at an 8192-token context (Q8_0 rows, bf16 activations) and a delta-net layer with 8 value / 8 key
    heads, 3 sequences, a few steps, against the oracle."""
    import torch
    from ornithology_b200 import device as D
    bf = torch.bfloat16
    # --- full attention
    layer = full_case(7, nh=4, nkv=1)
    dl = device_full(layer)
    rng = np.random.default_rng(71)
    ctx = [8192, 8192, 8000]
    steps = 3
    caps = [c + steps for c in ctx]
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, caps)
    okvs = []
    rb = layer.nkv * 272
    for b, L in enumerate(ctx):
        Kraw = rng.standard_normal((L, layer.hd)).astype(np.float32)
        Vraw = rng.standard_normal((L, layer.hd)).astype(np.float32)
        Kb = np.stack([oracle.q8_0_encode(r) for r in Kraw]); Vb = np.stack([oracle.q8_0_encode(r) for r in Vraw])
        o = int(kv.seq_off_host[b]) * rb
        kv.K[o:o + Kb.size] = torch.from_numpy(Kb.ravel()).cuda()
        kv.V[o:o + Vb.size] = torch.from_numpy(Vb.ravel()).cuda()
        okv = oracle.kv(caps[b], layer.nkv, layer.hd, O.KV_Q8_0)
        Kd = _q8_0_rows_to_f32(Kb.reshape(L, 8, 34)); Vd = _q8_0_rows_to_f32(Vb.reshape(L, 8, 34))
        C.memmove(okv.c.Kb, Kb.ctypes.data, Kb.size); C.memmove(okv.c.Vb, Vb.ctypes.data, Vb.size)
        C.memmove(okv.c.K, Kd.ctypes.data, Kd.nbytes); C.memmove(okv.c.V, Vd.ctypes.data, Vd.nbytes)
        okv.c.len = L
        okvs.append(okv)
    kv_len = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    data = [full_inputs(700 + b, layer, steps, bf16=True) for b in range(len(ctx))]
    worst_full = worst_lin = 0.0
    for s in range(steps):
        qp, k, v = [np.stack([data[b][i][s] for b in range(len(ctx))]) for i in range(3)]
        out = D.full_attn_step(dl, kv, kv_len, _t(qp, bf), _t(k, bf), _t(v, bf), max_len=max(caps)).float().cpu().numpy()
        for b in range(len(ctx)):
            ref = oracle.full_attn_step(layer, okvs[b], ctx[b] + s, qp[b], k[b], v[b])
            worst_full = max(worst_full, rel_err(out[b], ref))
            assert rel_err(out[b], ref) < TOL_BF16_IO, (s, b)
        D.advance(kv_len)
    # --- delta-net
    lin, kw = linear_case(9, nk=8, nv=8)
    dlin = device_linear(lin, kw)
    B, T = 3, 12
    ins = [linear_inputs(90 + b, lin, T, bf16=True) for b in range(B)]
    S = [np.zeros((lin.nv, 128, 128), np.float32) for _ in range(B)]
    buf = [np.zeros(3 * lin.cc, np.float32) for _ in range(B)]
    st = D.LinearState(dlin, B)
    pos = torch.zeros(B, dtype=torch.int32, device="cuda")
    for t in range(T):
        stack = [np.stack([ins[b][i][t] for b in range(B)]) for i in range(4)]
        out = D.linear_attn_step(dlin, st, pos, *[_t(x, bf) for x in stack]).float().cpu().numpy()
        for b in range(B):
            ref = oracle.linear_attn_step(lin, S[b], buf[b], *[ins[b][i][t] for i in range(4)])
            worst_lin = max(worst_lin, rel_err(out[b], ref))
            assert rel_err(out[b], ref) < TOL_BF16_IO, (t, b)
        D.advance(pos)
    _note("397B shard shapes bf16", gqa_out=worst_full, delta_out=worst_lin,
          delta_state=max(rel_err(st.S[b].cpu().numpy(), S[b]) for b in range(B)), bar=TOL_BF16_IO)
    for b in range(B):
        assert rel_err(st.S[b].cpu().numpy(), S[b]) < TOL
