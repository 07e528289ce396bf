"""Full-attention layers on the GPU (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest

from tests._cases import TOL, device_full, full_case, full_inputs, rel_err

pytestmark = pytest.mark.gpu

MODES = ["f32", "q8_0", "int8"]
# With bf16 activations the result itself is stored as bf16: half a bf16 ulp (2^-9) of
# output rounding comes on top of the 2e-3 arithmetic bar.
TOL_BF16_IO = TOL + 2.0 ** -9 + 5e-4


def _modes(name):
    from ornithology_b200 import device as D
    from oracle import oracle as O
    return {"f32": (D.KV_F32, O.KV_F32), "q8_0": (D.KV_Q8_0, O.KV_Q8_0), "int8": (D.KV_INT8_HEAD, O.KV_INT8_HEAD)}[name]


@pytest.mark.parametrize("name,mode", [("full_layer_f32.npz", "f32"), ("full_layer_int8.npz", "int8")])
def test_golden_full_layer_steps(golden, name, mode):
    """Fixtures produced by the reference's own code (tests/golden/make_golden.py)."""
    import torch
    from ornithology_b200 import device as D
    g = golden(name)
    nh, nkv, hd, T, base = int(g["nh"]), int(g["nkv"]), int(g["hd"]), g["QP"].shape[0], int(g["base"])
    layer = D.FullLayer(nh, nkv, hd, g["q_norm_w"], g["k_norm_w"], rope_dim=int(g["rope_dim"]), theta=float(g["theta"]))
    kv = D.KvBatch(_modes(mode)[0], nkv, hd, [T])
    kv_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    rope = torch.full((1,), base, dtype=torch.int32, device="cuda")
    for t in range(T):
        out = D.full_attn_step(layer, kv, kv_len, torch.from_numpy(g["QP"][t:t + 1]).cuda(),
                               torch.from_numpy(g["K"][t:t + 1]).cuda(), torch.from_numpy(g["V"][t:t + 1]).cuda(),
                               rope_pos=rope)
        assert rel_err(out.cpu().numpy()[0], g["OUT"][t]) < TOL, t
        D.advance(kv_len); D.advance(rope)
    # prefill of the same tokens from an empty cache
    kv2 = D.KvBatch(_modes(mode)[0], nkv, hd, [T])
    kv_len.zero_(); rope.fill_(base)
    out = D.full_attn_prefill(layer, kv2, kv_len, torch.from_numpy(g["QP"])[None].cuda(),
                              torch.from_numpy(g["K"])[None].cuda(), torch.from_numpy(g["V"])[None].cuda(), T, rope_pos=rope)
    assert rel_err(out.cpu().numpy()[0], g["OUT"]) < TOL


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("bf16", [False, True])
def test_35b_shape_batched_decode(oracle, mode, bf16):
    """16 query / 2 KV heads x 256, ragged batch: prefill then decode, each sequence
    checked against the oracle at every step; Q8_0 rows checked byte for byte."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(1)
    dl = device_full(layer)
    ctx = [37, 130, 1, 300]                      # prompt lengths, ragged
    steps = 5
    caps = [c + steps for c in ctx]
    caps[2] = ctx[2] + 2                         # this one fills up: later steps must be no-ops
    dm, om = _modes(mode)
    kv = D.KvBatch(dm, layer.nkv, layer.hd, caps)
    dt = torch.bfloat16 if bf16 else torch.float32
    okvs, data = [], []
    for b, c in enumerate(ctx):
        QP, K, V = full_inputs(100 + b, layer, c + steps, bf16)
        data.append((QP, K, V))
        okv = oracle.kv(caps[b], layer.nkv, layer.hd, om)
        ref = oracle.full_attn_prefill(layer, okv, 0, QP[:c], K[:c], V[:c])
        okvs.append(okv)
        # prefill one sequence at a time through a single-sequence view of the same pools
        one = D.KvBatch.__new__(D.KvBatch)
        one.__dict__.update(kv.__dict__)
        import ctypes as C
        from ornithology_b200._lib import CudaKv
        off = kv.seq_off[b:b + 2].clone()
        one.n_seq = 1
        one.c = CudaKv(dm, layer.nkv, layer.hd, 1, kv.c.K, kv.c.V, kv.c.Ks, kv.c.Vs, C.c_void_p(off.data_ptr()))
        z = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = D.full_attn_prefill(dl, one, z, torch.from_numpy(QP[:c])[None].cuda().to(dt),
                                  torch.from_numpy(K[:c])[None].cuda().to(dt),
                                  torch.from_numpy(V[:c])[None].cuda().to(dt), c)
        torch.cuda.synchronize()
        tol = TOL if not bf16 else TOL_BF16_IO
        assert rel_err(out.float().cpu().numpy()[0], ref) < tol, ("prefill", b)
    kv_len = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    for s in range(steps):
        qp = np.stack([data[b][0][ctx[b] + s] for b in range(len(ctx))])
        k = np.stack([data[b][1][ctx[b] + s] for b in range(len(ctx))])
        v = np.stack([data[b][2][ctx[b] + s] for b in range(len(ctx))])
        out = D.full_attn_step(dl, kv, kv_len, torch.from_numpy(qp).cuda().to(dt), torch.from_numpy(k).cuda().to(dt),
                               torch.from_numpy(v).cuda().to(dt), max_len=max(caps)).float().cpu().numpy()
        for b in range(len(ctx)):
            if ctx[b] + s >= caps[b]:
                continue                          # full cache: output untouched, nothing appended
            ref = oracle.full_attn_step(layer, okvs[b], ctx[b] + s, qp[b], k[b], v[b])
            tol = TOL if not bf16 else TOL_BF16_IO
            assert rel_err(out[b], ref) < tol, (s, b)
        D.advance(kv_len)
    if mode == "q8_0" and not bf16:
        # rows were built from GPU-side norm+RoPE values; re-encode those on the CPU and compare bytes
        f32kv = D.KvBatch(D.KV_F32, layer.nkv, layer.hd, caps)
        z = torch.zeros(len(ctx), dtype=torch.int32, device="cuda")
        for s in range(2):
            qp = np.stack([data[b][0][s] for b in range(len(ctx))])
            k = np.stack([data[b][1][s] for b in range(len(ctx))])
            v = np.stack([data[b][2][s] for b in range(len(ctx))])
            D.full_attn_step(dl, f32kv, z, torch.from_numpy(qp).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), max_len=8)
            D.advance(z)
        for b in range(len(ctx)):
            n = min(2, caps[b])
            Kf, Vf = f32kv.rows(b, n)
            Kb, Vb = kv.rows(b, n)
            for t in range(n):
                for h in range(layer.nkv):
                    assert (oracle.q8_0_encode(Kf[t, h]) == Kb[t, h]).all()
                    assert (oracle.q8_0_encode(Vf[t, h]) == Vb[t, h]).all()


def test_prefill_equals_decode_on_gpu():
    """The engine's own contract (prefill == T decode steps) on the CUDA path."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(3, nh=8, nkv=2, hd=128, rope_dim=32)
    dl = device_full(layer)
    T = 70
    QP, K, V = full_inputs(7, layer, T)
    for mode in (D.KV_F32, D.KV_Q8_0):
        kv_a, kv_b = D.KvBatch(mode, 2, 128, [T]), D.KvBatch(mode, 2, 128, [T])
        z = torch.zeros(1, dtype=torch.int32, device="cuda")
        pre = D.full_attn_prefill(dl, kv_a, z, torch.from_numpy(QP)[None].cuda(), torch.from_numpy(K)[None].cuda(),
                                  torch.from_numpy(V)[None].cuda(), T).cpu().numpy()[0]
        outs = []
        for t in range(T):
            outs.append(D.full_attn_step(dl, kv_b, z, torch.from_numpy(QP[t:t + 1]).cuda(), torch.from_numpy(K[t:t + 1]).cuda(),
                                         torch.from_numpy(V[t:t + 1]).cuda()).cpu().numpy()[0])
            D.advance(z)
        assert rel_err(pre, np.stack(outs)) < 1e-4
        assert (kv_a.K.cpu().numpy() == kv_b.K.cpu().numpy()).all() and (kv_a.V.cpu().numpy() == kv_b.V.cpu().numpy()).all()


@pytest.mark.parametrize("L", [1500, 9001])
def test_long_context_split_k(oracle, L):
    """A context long enough for several splits (and a ragged last one)."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(5)
    dl = device_full(layer)
    rng = np.random.default_rng(8)
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [L + 1])
    okv = oracle.kv(L + 1, layer.nkv, layer.hd, 2)
    # fill both caches with the same already-encoded rows (skips an O(L^2) CPU prefill)
    Kraw = rng.standard_normal((L, layer.nkv * layer.hd)).astype(np.float32)
    Vraw = rng.standard_normal((L, layer.nkv * layer.hd)).astype(np.float32)
    Kb = np.stack([oracle.q8_0_encode(r.reshape(layer.nkv, layer.hd)[h]) for r in Kraw for h in range(layer.nkv)])
    Vb = np.stack([oracle.q8_0_encode(r.reshape(layer.nkv, layer.hd)[h]) for r in Vraw for h in range(layer.nkv)])
    kv.K[:Kb.size] = torch.from_numpy(Kb.ravel()).cuda()
    kv.V[:Vb.size] = torch.from_numpy(Vb.ravel()).cuda()
    import ctypes as C
    C.memmove(okv.c.Kb, Kb.ctypes.data, Kb.size); C.memmove(okv.c.Vb, Vb.ctypes.data, Vb.size)
    Kd = np.stack([oracle.q8_0_decode(r) for r in Kb]).astype(np.float32)
    Vd = np.stack([oracle.q8_0_decode(r) for r in Vb]).astype(np.float32)
    C.memmove(okv.c.K, Kd.ctypes.data, Kd.nbytes); C.memmove(okv.c.V, Vd.ctypes.data, Vd.nbytes)
    okv.c.len = L
    QP, K, V = full_inputs(9, layer, 1)
    kv_len = torch.tensor([L], dtype=torch.int32, device="cuda")
    out = D.full_attn_step(dl, kv, kv_len, torch.from_numpy(QP).cuda(), torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    ref = oracle.full_attn_step(layer, okv, L, QP[0], K[0], V[0])
    assert rel_err(out.cpu().numpy()[0], ref) < TOL


def test_long_context_ragged_batch_q8(oracle):
    """Sequences whose contexts reach different numbers of splits, in one pool (non-zero row
    offsets for the tile copies), stepped twice: the in-kernel merge of the split partials
    must see only the live splits of each sequence, and its arrival counters must be re-armed."""
    import ctypes as C
    import torch
    from ornithology_b200 import device as D
    layer = full_case(6)
    dl = device_full(layer)
    rng = np.random.default_rng(21)
    ctx = [9001, 700, 3000, 15]
    caps = [c + 2 for c in ctx]
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, caps)
    okvs = []
    rb = layer.nkv * 272
    for b, L in enumerate(ctx):
        Kraw = rng.standard_normal((L * layer.nkv, layer.hd)).astype(np.float32)
        Vraw = rng.standard_normal((L * layer.nkv, layer.hd)).astype(np.float32)
        Kb = np.stack([oracle.q8_0_encode(r) for r in Kraw])
        Vb = np.stack([oracle.q8_0_encode(r) for r in Vraw])
        o = int(kv.seq_off_host[b]) * rb
        kv.K[o:o + Kb.size] = torch.from_numpy(Kb.ravel()).cuda()
        kv.V[o:o + Vb.size] = torch.from_numpy(Vb.ravel()).cuda()
        okv = oracle.kv(caps[b], layer.nkv, layer.hd, 2)
        C.memmove(okv.c.Kb, Kb.ctypes.data, Kb.size); C.memmove(okv.c.Vb, Vb.ctypes.data, Vb.size)
        Kd = np.stack([oracle.q8_0_decode(r) for r in Kb]).astype(np.float32)
        Vd = np.stack([oracle.q8_0_decode(r) for r in Vb]).astype(np.float32)
        C.memmove(okv.c.K, Kd.ctypes.data, Kd.nbytes); C.memmove(okv.c.V, Vd.ctypes.data, Vd.nbytes)
        okv.c.len = L
        okvs.append(okv)
    kv_len = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    for s in range(2):
        QP, K, V = full_inputs(30 + s, layer, len(ctx))
        out = D.full_attn_step(dl, kv, kv_len, torch.from_numpy(QP).cuda(), torch.from_numpy(K).cuda(),
                               torch.from_numpy(V).cuda(), max_len=max(caps)).cpu().numpy()
        for b, L in enumerate(ctx):
            ref = oracle.full_attn_step(layer, okvs[b], L + s, QP[b], K[b], V[b])
            assert rel_err(out[b], ref) < TOL, (s, b)
        D.advance(kv_len)


def _prefill(D, dl, kv, kv_len, QP, K, V, T, max_len=None, bf16=False):
    import torch
    dt = torch.bfloat16 if bf16 else torch.float32
    to = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda().to(dt)
    return D.full_attn_prefill(dl, kv, kv_len, to(QP), to(K), to(V), T, max_len=max_len).float().cpu().numpy()


def test_tensor_core_prefill_long_prompt(oracle, monkeypatch):
    """1500-token prompt at the 35B head shape (12 tiles of 128 query rows, up to 24 key tiles each):
    the tcgen05 kernel against the oracle, then the same prompt in two calls (the second one
    attends over a non-empty cache), and the mma.sync variant; cache bytes identical throughout."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(21)
    dl = device_full(layer)
    T = 1500
    QP, K, V = full_inputs(210, layer, T)
    okv = oracle.kv(T, layer.nkv, layer.hd, 2)
    ref = oracle.full_attn_prefill(layer, okv, 0, QP, K, V)
    z = torch.zeros(1, dtype=torch.int32, device="cuda")

    monkeypatch.setenv("ORNITH_CUDA_PREFILL_VARIANT", "tc")
    kv_a = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [T])
    out_a = _prefill(D, dl, kv_a, z, QP[None], K[None], V[None], T)[0]
    assert rel_err(out_a, ref) < TOL

    kv_b = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [T])
    T1 = 811                                               # not a multiple of any tile size
    out_b1 = _prefill(D, dl, kv_b, z, QP[None, :T1], K[None, :T1], V[None, :T1], T1)[0]
    n1 = torch.full((1,), T1, dtype=torch.int32, device="cuda")
    out_b2 = _prefill(D, dl, kv_b, n1, QP[None, T1:], K[None, T1:], V[None, T1:], T - T1, max_len=T)[0]
    assert rel_err(np.vstack([out_b1, out_b2]), ref) < TOL
    assert rel_err(np.vstack([out_b1, out_b2]), out_a) < 5e-4

    monkeypatch.setenv("ORNITH_CUDA_PREFILL_VARIANT", "mma")
    kv_c = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [T])
    out_c = _prefill(D, dl, kv_c, z, QP[None], K[None], V[None], T)[0]
    assert rel_err(out_c, ref) < TOL
    for other in (kv_b, kv_c):
        assert (kv_a.K.cpu().numpy() == other.K.cpu().numpy()).all() and (kv_a.V.cpu().numpy() == other.V.cpu().numpy()).all()


def test_tensor_core_prefill_ragged_batch_bf16():
    """Two sequences in one call, one of them continuing a 700-token cache, bf16 activations:
    each must equal the same sequence run alone."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(22)
    dl = device_full(layer)
    T, L0 = 600, 700
    seqs = [full_inputs(220 + b, layer, L0 + T, bf16=True) for b in range(2)]
    z1 = torch.zeros(1, dtype=torch.int32, device="cuda")
    alone = []
    for b, (QP, K, V) in enumerate(seqs):
        kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [L0 + T])
        if b == 1:
            _prefill(D, dl, kv, z1, QP[None, :L0], K[None, :L0], V[None, :L0], L0, bf16=True)
            start = torch.full((1,), L0, dtype=torch.int32, device="cuda")
            alone.append(_prefill(D, dl, kv, start, QP[None, L0:], K[None, L0:], V[None, L0:], T, max_len=L0 + T, bf16=True)[0])
        else:
            alone.append(_prefill(D, dl, kv, z1, QP[None, :T], K[None, :T], V[None, :T], T, bf16=True)[0])
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [T, L0 + T])
    # sequence 1 gets its first L0 tokens through a single-sequence view of the shared pools
    import ctypes as C
    from ornithology_b200._lib import CudaKv
    one = D.KvBatch.__new__(D.KvBatch)
    one.__dict__.update(kv.__dict__)
    off = kv.seq_off[1:3].clone()
    one.n_seq = 1
    one.c = CudaKv(D.KV_Q8_0, layer.nkv, layer.hd, 1, kv.c.K, kv.c.V, kv.c.Ks, kv.c.Vs, C.c_void_p(off.data_ptr()))
    QP1, K1, V1 = seqs[1]
    _prefill(D, dl, one, z1, QP1[None, :L0], K1[None, :L0], V1[None, :L0], L0, bf16=True)
    lens = torch.tensor([0, L0], dtype=torch.int32, device="cuda")
    QPb = np.stack([seqs[0][0][:T], QP1[L0:]]); Kb = np.stack([seqs[0][1][:T], K1[L0:]]); Vb = np.stack([seqs[0][2][:T], V1[L0:]])
    both = _prefill(D, dl, kv, lens, QPb, Kb, Vb, T, max_len=L0 + T, bf16=True)
    for b in range(2):
        assert rel_err(both[b], alone[b]) < 1e-5, b


@pytest.mark.parametrize("L", [1500, 9001])
def test_long_context_split_k_f32_rows(oracle, L):
    """The tf32 tensor-core decode over f32 rows: several splits, a ragged last split and tile."""
    import ctypes as C
    import torch
    from ornithology_b200 import device as D
    layer = full_case(6)
    dl = device_full(layer)
    rng = np.random.default_rng(18)
    kv = D.KvBatch(D.KV_F32, layer.nkv, layer.hd, [L + 1])
    okv = oracle.kv(L + 1, layer.nkv, layer.hd, 0)
    Kraw = rng.standard_normal((L, layer.nkv * layer.hd)).astype(np.float32)
    Vraw = rng.standard_normal((L, layer.nkv * layer.hd)).astype(np.float32)
    kv.K.view(torch.float32)[:Kraw.size] = torch.from_numpy(Kraw.ravel()).cuda()
    kv.V.view(torch.float32)[:Vraw.size] = torch.from_numpy(Vraw.ravel()).cuda()
    C.memmove(okv.c.K, Kraw.ctypes.data, Kraw.nbytes); C.memmove(okv.c.V, Vraw.ctypes.data, Vraw.nbytes)
    okv.c.len = L
    QP, K, V = full_inputs(19, layer, 1)
    kv_len = torch.tensor([L], dtype=torch.int32, device="cuda")
    out = D.full_attn_step(dl, kv, kv_len, torch.from_numpy(QP).cuda(), torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    ref = oracle.full_attn_step(layer, okv, L, QP[0], K[0], V[0])
    assert rel_err(out.cpu().numpy()[0], ref) < TOL


@pytest.mark.parametrize("L", [1500, 9001])
def test_long_context_split_k_int8_rows(oracle, L):
    """The raw-fragment decode over int8-per-head rows (the engine's own quantised cache)."""
    import ctypes as C
    import torch
    from ornithology_b200 import device as D
    layer = full_case(7)
    dl = device_full(layer)
    rng = np.random.default_rng(28)
    n = L * layer.nkv
    kv = D.KvBatch(D.KV_INT8_HEAD, layer.nkv, layer.hd, [L + 1])
    okv = oracle.kv(L + 1, layer.nkv, layer.hd, 1)
    Kq = rng.integers(-127, 128, (n, layer.hd)).astype(np.int8)
    Vq = rng.integers(-127, 128, (n, layer.hd)).astype(np.int8)
    Ks = rng.uniform(0.005, 0.04, n).astype(np.float32)
    Vs = rng.uniform(0.005, 0.04, n).astype(np.float32)
    kv.K[:Kq.size] = torch.from_numpy(Kq.view(np.uint8).ravel()).cuda()
    kv.V[:Vq.size] = torch.from_numpy(Vq.view(np.uint8).ravel()).cuda()
    kv.Ks[:n] = torch.from_numpy(Ks).cuda()
    kv.Vs[:n] = torch.from_numpy(Vs).cuda()
    C.memmove(okv.c.Kq, Kq.ctypes.data, Kq.nbytes); C.memmove(okv.c.Vq, Vq.ctypes.data, Vq.nbytes)
    C.memmove(okv.c.Ks, Ks.ctypes.data, Ks.nbytes); C.memmove(okv.c.Vs, Vs.ctypes.data, Vs.nbytes)
    okv.c.len = L
    QP, K, V = full_inputs(29, layer, 1)
    kv_len = torch.tensor([L], dtype=torch.int32, device="cuda")
    out = D.full_attn_step(dl, kv, kv_len, torch.from_numpy(QP).cuda(), torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    ref = oracle.full_attn_step(layer, okv, L, QP[0], K[0], V[0])
    assert rel_err(out.cpu().numpy()[0], ref) < TOL


@pytest.mark.parametrize("mode", MODES)
def test_groups_of_16_query_heads(oracle, mode):
    """397B head shape on one GPU: 32 query heads over 2 KV heads.  Each group of 16 is walked by two
    CTAs of 8 heads; decode steps over a ragged batch against the oracle."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(9, nh=32, nkv=2)
    dl = device_full(layer)
    dm, om = _modes(mode)
    ctx, steps = [75, 210], 3
    caps = [c + steps for c in ctx]
    kv = D.KvBatch(dm, layer.nkv, layer.hd, caps)
    okvs, data = [], []
    for b, c in enumerate(ctx):
        QP, K, V = full_inputs(300 + b, layer, c + steps)
        data.append((QP, K, V))
        okv = oracle.kv(caps[b], layer.nkv, layer.hd, om)
        oracle.full_attn_prefill(layer, okv, 0, QP[:c], K[:c], V[:c])
        okvs.append(okv)
    # fill the device cache token by token through the decode path itself (exercises every context length)
    kv_len = torch.zeros(len(ctx), dtype=torch.int32, device="cuda")
    for t in range(max(ctx)):
        qp = np.stack([data[b][0][min(t, ctx[b] - 1)] for b in range(len(ctx))])
        k = np.stack([data[b][1][min(t, ctx[b] - 1)] for b in range(len(ctx))])
        v = np.stack([data[b][2][min(t, ctx[b] - 1)] for b in range(len(ctx))])
        live = torch.tensor([t < c for c in ctx], device="cuda")
        # sequences that already hold their whole prompt re-append nothing: run them on a scratch copy of the lengths
        if not bool(live.all()):
            break
        D.full_attn_step(dl, kv, kv_len, torch.from_numpy(qp).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                         max_len=max(caps))
        D.advance(kv_len)
    # the shorter prompt is in; finish the longer one alone through a single-sequence view
    import ctypes as C
    from ornithology_b200._lib import CudaKv
    one = D.KvBatch.__new__(D.KvBatch)
    one.__dict__.update(kv.__dict__)
    off = kv.seq_off[1:3].clone()
    one.n_seq = 1
    one.c = CudaKv(dm, layer.nkv, layer.hd, 1, kv.c.K, kv.c.V, kv.c.Ks, kv.c.Vs, C.c_void_p(off.data_ptr()))
    l1 = kv_len[1:2].clone()
    for t in range(ctx[0], ctx[1]):
        D.full_attn_step(dl, one, l1, torch.from_numpy(data[1][0][t:t + 1]).cuda(), torch.from_numpy(data[1][1][t:t + 1]).cuda(),
                         torch.from_numpy(data[1][2][t:t + 1]).cuda(), max_len=max(caps))
        D.advance(l1)
    kv_len = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    for s in range(steps):
        qp = np.stack([data[b][0][ctx[b] + s] for b in range(len(ctx))])
        k = np.stack([data[b][1][ctx[b] + s] for b in range(len(ctx))])
        v = np.stack([data[b][2][ctx[b] + s] for b in range(len(ctx))])
        out = D.full_attn_step(dl, kv, kv_len, torch.from_numpy(qp).cuda(), torch.from_numpy(k).cuda(),
                               torch.from_numpy(v).cuda(), max_len=max(caps)).cpu().numpy()
        for b in range(len(ctx)):
            ref = oracle.full_attn_step(layer, okvs[b], ctx[b] + s, qp[b], k[b], v[b])
            assert rel_err(out[b], ref) < TOL, (s, b)
        D.advance(kv_len)


def test_tensor_core_prefill_is_reproducible():
    """Eight runs of the same 2048-token prompt through the tcgen05 prefill must agree bit for bit."""
    import torch
    from ornithology_b200 import device as D
    layer = full_case(61)
    dl = device_full(layer)
    T = 2048
    QP, K, V = [torch.from_numpy(x).cuda()[None] for x in full_inputs(62, layer, T)]
    first = None
    for rep in range(8):
        kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [T])
        kv_len = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = D.full_attn_prefill(dl, kv, kv_len, QP, K, V, T).cpu().numpy()
        if first is None:
            first = out
        else:
            assert (out == first).all(), rep
