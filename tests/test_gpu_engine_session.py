"""The host-fed layer calls over device-resident state (ornith_cuda_engine_*) against the oracle: one
full-attention and one delta-net layer of a tiny model (head sizes that take the generic kernels) and of a
35B-like shape (tensor-core kernels), prefill then decode steps, then a session round trip through the records."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from tests._cases import TOL, full_case, full_inputs, linear_case, linear_inputs, rel_err

pytestmark = pytest.mark.gpu


def _fp(x):
    return x.ctypes.data_as(C.c_void_p)


@pytest.mark.parametrize("shape", ["tiny", "35b-like"])
def test_engine_layers_prefill_decode_and_session(oracle, shape):
    from ornithology_b200 import _lib
    lib = _lib.load()
    if shape == "tiny":
        full = full_case(71, nh=4, nkv=2, hd=8, rope_dim=4, theta=1e4)
        lin, kw = linear_case(72, nk=2, nv=4, dk=6, dv=6)
    else:
        full = full_case(73, nh=8, nkv=2, hd=256)
        lin, kw = linear_case(74, nk=2, nv=4)
    T, steps, cap = 70, 4, 80
    eng = [lib.ornith_cuda_engine_new(2, cap, 0, full.nh, full.nkv, full.hd, full.rope_dim, full.theta, full.eps,
                                      lin.nk, lin.nv, lin.dk, lin.dv, 4) for _ in range(2)]
    assert all(eng), lib.ornith_cuda_last_error()

    def ready(e):
        assert lib.ornith_cuda_engine_full_layer(e, 0, _fp(full.q_norm_w), _fp(full.k_norm_w)) == 0
        assert lib.ornith_cuda_engine_linear_layer(e, 1, _fp(kw["conv_w"]), _fp(kw["a_coef"]), _fp(kw["dt_bias"]), _fp(kw["norm_w"])) == 0

    ready(eng[0])
    QP, K, V = full_inputs(75, full, T + steps)
    li = linear_inputs(76, lin, T + steps)
    okv = oracle.kv(cap, full.nkv, full.hd, O.KV_F32)
    S = np.zeros((lin.nv, lin.dv, lin.dk), np.float32); buf = np.zeros(3 * lin.cc, np.float32)

    def run_full(e, pos, n):
        out = np.empty((n, full.nh * full.hd), np.float32)
        q, k, v = [np.ascontiguousarray(x[pos:pos + n]) for x in (QP, K, V)]
        assert lib.ornith_cuda_engine_full_attn(e, 0, pos, n, _fp(q), _fp(k), _fp(v), _fp(out)) == 0, lib.ornith_cuda_last_error()
        return out

    def run_lin(e, pos, n):
        out = np.empty((n, lin.vd), np.float32)
        xs = [np.ascontiguousarray(x[pos:pos + n]) for x in li]
        assert lib.ornith_cuda_engine_linear_attn(e, 1, pos, n, *[_fp(x) for x in xs], _fp(out)) == 0, lib.ornith_cuda_last_error()
        return out

    assert rel_err(run_full(eng[0], 0, T), oracle.full_attn_prefill(full, okv, 0, QP[:T], K[:T], V[:T])) < TOL
    assert rel_err(run_lin(eng[0], 0, T), oracle.linear_attn_prefill(lin, S, buf, *[x[:T] for x in li], chunk=64)) < TOL
    # session round trip into the second object, which then carries on bit-identically
    ready(eng[1])
    for L in (0, 1):
        n = lib.ornith_cuda_engine_record_bytes(eng[0], L, T)
        rec = np.zeros(n, np.uint8)
        assert lib.ornith_cuda_engine_export(eng[0], L, T, _fp(rec), n) == 0
        assert lib.ornith_cuda_engine_import(eng[1], L, T, _fp(rec), n) == 0, lib.ornith_cuda_last_error()
    for s in range(steps):
        p = T + s
        a, b = run_full(eng[0], p, 1), run_full(eng[1], p, 1)
        assert (a == b).all() and rel_err(a[0], oracle.full_attn_step(full, okv, p, QP[p], K[p], V[p])) < TOL, s
        a, b = run_lin(eng[0], p, 1), run_lin(eng[1], p, 1)
        assert (a == b).all() and rel_err(a[0], oracle.linear_attn_step(lin, S, buf, *[x[p] for x in li])) < TOL, s
    # errors: a layer used as the other kind, a position past the capacity
    assert lib.ornith_cuda_engine_linear_attn(eng[0], 0, 0, 1, None, None, None, None, None) != 0
    out = np.empty((1, full.nh * full.hd), np.float32)
    assert lib.ornith_cuda_engine_full_attn(eng[0], 0, cap, 1, _fp(QP[:1]), _fp(K[:1]), _fp(V[:1]), _fp(out)) != 0
    for e in eng:
        lib.ornith_cuda_engine_free(e)
