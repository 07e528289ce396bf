"""Session records of device-resident state (ornith_cuda_kv_export/_import, ornith_cuda_linear_export/_import).

The records are the per-layer parts of the engine's session file (writer: src/ornith_rforward.c:1020-1076,
reader: :1078-1171).  `engine_kv_record` / `engine_linear_record` below restate that writer's layout over the
oracle's CPU state, so the tests can check that (1) a record taken on the device has the engine's bytes,
(2) a record written on the CPU side loads into the device and the sequence carries on within the parity bar,
(3) export -> import into a fresh device state continues bit-identically.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from ornithology_b200._lib import BackendError
from tests._cases import TOL, device_full, device_linear, full_case, full_inputs, linear_case, linear_inputs, rel_err


def engine_kv_record(okv, mode):
    """What rmodel_session_save writes for a full-attention layer (src/ornith_rforward.c:1040-1052), plus the
    q = 2 extension for Q8_0 rows."""
    n = okv.len
    if mode == O.KV_F32:
        K, V = okv.rows_f32()
        body = K.tobytes() + V.tobytes()
    elif mode == O.KV_INT8_HEAD:
        Kq, Vq, Ks, Vs = okv.rows_int8()
        body = Kq.tobytes() + Vq.tobytes() + Ks.tobytes() + Vs.tobytes()
    else:
        Kb, Vb = okv.rows_q8_0()
        body = Kb.tobytes() + Vb.tobytes()
    head = np.array([{O.KV_F32: 0, O.KV_INT8_HEAD: 1, O.KV_Q8_0: 2}[mode], n, okv.nkv, okv.hd], np.int32).tobytes()
    return np.frombuffer(head + body, np.uint8)


def engine_linear_record(S, conv_buf, conv_k, cc):
    """The delta-net layer record (src/ornith_rforward.c:1054-1063): S, conv_k, Cc, history oldest first."""
    return np.frombuffer(np.ascontiguousarray(S, np.float32).tobytes() + np.array([conv_k, cc], np.int32).tobytes() +
                         np.ascontiguousarray(conv_buf, np.float32).tobytes(), np.uint8)


def test_record_sizes_and_no_gpu_behaviour():
    """Host-side: the size queries follow the engine's layout; without a GPU the calls fail with a status."""
    import torch
    from ornithology_b200 import _lib, build
    from ornithology_b200._lib import CudaKv, CudaLinearLayer
    build.build()
    lib = _lib.load()
    for mode, row, extra in ((0, 256 * 4, 0), (1, 256, 8), (2, 8 * 34, 0)):
        kv = CudaKv(mode, 2, 256, 1, None, None, None, None, None)
        assert lib.ornith_cuda_kv_record_bytes(C.byref(kv), 100) == 16 + 100 * 2 * (2 * row + extra)
    lin = CudaLinearLayer()
    lin.nk, lin.nv, lin.dk, lin.dv, lin.conv_k = 16, 32, 128, 128, 4
    assert lib.ornith_cuda_linear_record_bytes(C.byref(lin)) == (32 * 128 * 128 + 3 * 8192) * 4 + 8
    if not torch.cuda.is_available():
        kv = CudaKv(0, 2, 256, 1, None, None, None, None, None)
        buf = np.zeros(64, np.uint8)
        assert lib.ornith_cuda_kv_export(C.byref(kv), 0, 0, buf.ctypes.data_as(C.c_void_p), 64, None) != 0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["f32", "int8", "q8_0"])
def test_kv_records_against_the_engine_layout(oracle, mode):
    import torch
    from ornithology_b200 import device as D
    dmode = {"f32": D.KV_F32, "int8": D.KV_INT8_HEAD, "q8_0": D.KV_Q8_0}[mode]
    omode = {"f32": O.KV_F32, "int8": O.KV_INT8_HEAD, "q8_0": O.KV_Q8_0}[mode]
    layer = full_case(51)
    dl = device_full(layer)
    T, more = 70, 5
    QP, K, V = full_inputs(52, layer, T + more)
    caps = [T + more, T + more]                                      # the sequence under test is the second of a batch
    kv = D.KvBatch(dmode, layer.nkv, layer.hd, caps)
    okv = oracle.kv(T + more, layer.nkv, layer.hd, omode)
    kv_len = torch.zeros(2, dtype=torch.int32, device="cuda")
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    two = lambda x: torch.stack([torch.ones_like(t(x)), t(x)])       # sequence 0 carries filler
    oracle.full_attn_prefill(layer, okv, 0, QP[:T], K[:T], V[:T])
    D.full_attn_prefill(dl, kv, kv_len, two(QP[:T]), two(K[:T]), two(V[:T]), T)
    D.advance(kv_len, T)

    rec = D.kv_export(kv, 1, T)
    ref = engine_kv_record(okv, omode)
    assert rec.size == ref.size and (rec[:16] == ref[:16]).all()
    # V rows are the engine's bytes in every mode.  K rows go through RMSNorm + RoPE first, and the device's
    # sincosf and libm's differ in the last place for some angles: f32 rows are bit-exact outside the rotated
    # dims and within 4e-7 inside; in the quantised modes a code may flip by one unit where a rotated value sits
    # on a rounding boundary (and then only there).
    rows = T * layer.nkv
    if mode == "f32":
        nb = rows * layer.hd * 4
        assert (rec[16 + nb:] == ref[16 + nb:]).all()
        a = rec[16:16 + nb].view(np.float32).reshape(T, layer.nkv, layer.hd)
        b = ref[16:16 + nb].view(np.float32).reshape(T, layer.nkv, layer.hd)
        assert (a[..., layer.rope_dim:].view(np.uint32) == b[..., layer.rope_dim:].view(np.uint32)).all()
        assert np.abs(a - b).max() <= 4e-7 * np.abs(b).max()
    elif mode == "int8":
        nb = rows * layer.hd
        kq, kq_ref = rec[16:16 + nb].view(np.int8).reshape(rows, layer.hd), ref[16:16 + nb].view(np.int8).reshape(rows, layer.hd)
        assert (rec[16 + nb:16 + 2 * nb] == ref[16 + nb:16 + 2 * nb]).all(), "V codes differ"
        ks, ks_ref = rec[16 + 2 * nb:16 + 2 * nb + 4 * rows].view(np.float32), ref[16 + 2 * nb:16 + 2 * nb + 4 * rows].view(np.float32)
        assert (rec[16 + 2 * nb + 4 * rows:] == ref[16 + 2 * nb + 4 * rows:]).all(), "V scales differ"
        # a K scale is amax / 127 of the rotated row: the last place may differ when the largest value is a rotated one
        assert np.abs(ks - ks_ref).max() <= 2.4e-7 * np.abs(ks_ref).max() and (ks != ks_ref).mean() < 0.05
        d = np.abs(kq.astype(np.int32) - kq_ref.astype(np.int32))
        assert (d[:, layer.rope_dim:] == 0).all() and d.max() <= 1 and (d != 0).mean() < 1e-3, (int(d.max()), int((d != 0).sum()))
    else:
        nb = rows * (layer.hd // 32) * 34
        assert (rec[16 + nb:] == ref[16 + nb:]).all(), "V rows differ"
        kb, kb_ref = rec[16:16 + nb].reshape(rows, -1, 34), ref[16:16 + nb].reshape(rows, -1, 34)
        assert (kb[:, :, :2] == kb_ref[:, :, :2]).all(), "K block scales differ"
        d = np.abs(kb[:, :, 2:].view(np.int8).astype(np.int32) - kb_ref[:, :, 2:].view(np.int8).astype(np.int32))
        assert (d[:, layer.rope_dim // 32:] == 0).all() and d.max() <= 1 and (d != 0).mean() < 1e-3, (int(d.max()), int((d != 0).sum()))

    # a record made on the CPU side loads into a fresh device cache, and decoding carries on like the CPU engine
    kv2 = D.KvBatch(dmode, layer.nkv, layer.hd, caps)
    len2 = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert D.kv_import(kv2, 1, ref, kv_len=len2) == T and int(len2[1]) == T and int(len2[0]) == 0
    assert D.kv_import(kv2, 0, D.kv_export(kv, 0, T), kv_len=len2) == T     # the filler sequence, device to device
    for s in range(more):
        p = T + s
        out_ref = oracle.full_attn_step(layer, okv, p, QP[p], K[p], V[p])
        outs = []
        for cache, lens in ((kv, kv_len), (kv2, len2)):
            o = D.full_attn_step(dl, cache, lens, two(QP[p]), two(K[p]), two(V[p]), max_len=T + more)
            outs.append(o.cpu().numpy())
            D.advance(lens)
        assert rel_err(outs[0][1], out_ref) < TOL and rel_err(outs[1][1], out_ref) < TOL, s
        assert (outs[0][0] == outs[1][0]).all(), s                   # device -> device: the same bytes, the same result

    # errors: a record of another mode, a record that does not fit
    other = D.KvBatch(D.KV_F32 if dmode != D.KV_F32 else D.KV_Q8_0, layer.nkv, layer.hd, caps)
    with pytest.raises(BackendError):
        D.kv_import(other, 0, rec)
    small = D.KvBatch(dmode, layer.nkv, layer.hd, [9])
    with pytest.raises(BackendError):
        D.kv_import(small, 0, rec)                                   # capacity 9 < 70 positions


@pytest.mark.gpu
def test_linear_records_against_the_engine_layout(oracle):
    import torch
    from ornithology_b200 import device as D
    layer, kw = linear_case(53, nk=4, nv=8)
    dl = device_linear(layer, kw)
    T, more = 75, 6
    ins = linear_inputs(54, layer, T + more)
    S = np.zeros((layer.nv, 128, 128), np.float32); buf = np.zeros(3 * layer.cc, np.float32)
    oracle.linear_attn_prefill(layer, S, buf, *[x[:T] for x in ins], chunk=64)
    B = 2                                                            # the record is taken from the second sequence of a batch
    st = D.LinearState(dl, B)
    pos = torch.zeros(B, dtype=torch.int32, device="cuda")
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    two = lambda x: torch.stack([torch.zeros_like(t(x)), t(x)])
    D.linear_attn_prefill(dl, st, pos, *[two(x[:T]) for x in ins], T, chunk=64)
    D.advance(pos, T)

    rec = st.export_record(1, T)
    ref = engine_linear_record(S, buf, 4, layer.cc)
    ns = layer.nv * 128 * 128 * 4
    assert rec.size == ref.size
    assert (rec[ns:] == ref[ns:]).all(), "conv_k, Cc or the history image differ from the engine's record"
    assert rel_err(rec[:ns].view(np.float32), ref[:ns].view(np.float32)) < TOL

    # the CPU-made record into a fresh device state; the device-made one into another; both carry on
    st_cpu, st_dev = D.LinearState(dl, B), D.LinearState(dl, B)
    st_cpu.import_record(1, T, ref)
    st_dev.import_record(1, T, rec)
    pos2, pos3 = pos.clone(), pos.clone()
    for s in range(more):
        p = T + s
        row = [two(x[p]) for x in ins]
        out_ref = oracle.linear_attn_step(layer, S, buf, *[x[p] for x in ins])
        o1 = D.linear_attn_step(dl, st, pos, *row).cpu().numpy()[1]
        o2 = D.linear_attn_step(dl, st_cpu, pos2, *row).cpu().numpy()[1]
        o3 = D.linear_attn_step(dl, st_dev, pos3, *row).cpu().numpy()[1]
        for c in (pos, pos2, pos3):
            D.advance(c)
        assert rel_err(o1, out_ref) < TOL and rel_err(o2, out_ref) < TOL, s
        assert (o1 == o3).all(), s                                   # export -> import is lossless
    assert (st.S[1].cpu().numpy() == st_dev.S[1].cpu().numpy()).all()
    assert (st.conv_image(1, T + more).cpu().numpy() == st_dev.conv_image(1, T + more).cpu().numpy()).all()
