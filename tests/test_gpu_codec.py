"""KV row codecs on the GPU against the CPU oracle: bit-exact bytes."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_q8_0_encode_decode_bit_exact(oracle, golden):
    import torch
    from ornithology_b200 import device as D
    g = golden("q8_0_vectors.npz")
    rng = np.random.default_rng(99)
    big = (rng.standard_normal(32 * 50000) * 10.0 ** rng.integers(-6, 5, 32 * 50000)).astype(np.float32)
    ties = ((rng.integers(-254, 255, 32 * 2000).astype(np.float32)) * 0.5)      # exact .5 after scaling
    ties[::32] = 127.0
    for x in (g["x"], big, ties.astype(np.float32)):
        xd = torch.from_numpy(x).cuda()
        b = D.q8_0_encode(xd)
        ref = oracle.q8_0_encode(x)
        got = b.cpu().numpy()
        assert got.shape == ref.shape
        bad = np.flatnonzero(got != ref)
        assert bad.size == 0, f"{bad.size} bytes differ, first at {bad[:5]}"
        dec = D.q8_0_decode(b).cpu().numpy()
        want = oracle.q8_0_decode(ref)
        nan = np.isnan(want)                      # 0 * inf blocks: NaN on both sides, payload unspecified
        assert (np.isnan(dec) == nan).all()
        assert (dec.view(np.uint32)[~nan] == want.view(np.uint32)[~nan]).all()
    assert (D.q8_0_encode(torch.from_numpy(g["x"]).cuda()).cpu().numpy() == g["bytes"]).all()


@pytest.mark.parametrize("mode", ["f32", "q8_0", "int8"])
def test_raw_append_rows_bit_exact(oracle, mode):
    """No norm, no RoPE: appended rows must be byte-identical to the CPU codec's."""
    import torch
    from ornithology_b200 import device as D
    from oracle.oracle import KV_F32, KV_INT8_HEAD, KV_Q8_0
    m = {"f32": (D.KV_F32, KV_F32), "q8_0": (D.KV_Q8_0, KV_Q8_0), "int8": (D.KV_INT8_HEAD, KV_INT8_HEAD)}[mode]
    nh, nkv, hd, T = 4, 2, 64, 7
    rng = np.random.default_rng(5)
    layer = D.FullLayer(nh, nkv, hd, None, None, rope_dim=0, gated=False)
    kv = D.KvBatch(m[0], nkv, hd, [T])
    okv = oracle.kv(T, nkv, hd, m[1])
    kv_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    for t in range(T):
        q = rng.standard_normal(nh * hd).astype(np.float32)
        k = (rng.standard_normal(nkv * hd) * (10.0 ** rng.integers(-3, 3))).astype(np.float32)
        v = rng.standard_normal(nkv * hd).astype(np.float32)
        if t == 3:
            k[:hd] = 0.0                                    # an all-zero head row
        out = D.full_attn_step(layer, kv, kv_len, torch.from_numpy(q)[None].cuda(),
                               torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
        ref = oracle.gqa_step(okv, q, k, v, nh)
        err = np.abs(out.cpu().numpy()[0] - ref).max() / np.abs(ref).max()
        assert err < 2e-3, (t, err)
        D.advance(kv_len)
    got = kv.rows(0, T)
    if mode == "f32":
        K, V = okv.rows_f32()
        assert (got[0].view(np.uint32) == K.view(np.uint32)).all() and (got[1].view(np.uint32) == V.view(np.uint32)).all()
    elif mode == "q8_0":
        Kb, Vb = okv.rows_q8_0()
        assert (got[0] == Kb).all() and (got[1] == Vb).all()
    else:
        Kq, Vq, Ks, Vs = okv.rows_int8()
        assert (got[0] == Kq).all() and (got[1] == Vq).all()
        assert (got[2].view(np.uint32) == Ks.view(np.uint32)).all() and (got[3].view(np.uint32) == Vs.view(np.uint32)).all()
