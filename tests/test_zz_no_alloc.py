"""The allocation-free decode entry point, ornith_cuda_full_attn_step_static.

It exists for hosts that may not allocate device memory on the token path (a fixed
device-memory budget handed out at start-up, no cudaMalloc between two tokens): its
scratch is an array built into the library instead of a caller buffer.  The test
drives it through the C ABI and requires the same output as the regular entry point
(which gets caller scratch), on two consecutive steps, so the second call runs over
the first call's leftovers in the shared array.  The file name sorts last on purpose:
a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from tests._cases import TOL, device_full, full_case, full_inputs, rel_err

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def test_static_scratch_entry_matches_regular_entry_twice():
    import torch
    from ornithology_b200 import _lib, device as D
    lib = _lib.load()
    layer = full_case(31)                                  # 16 query / 2 KV heads x 256
    dl = device_full(layer)
    ctx, steps = [200, 37, 1000], 2
    caps = [c + steps for c in ctx]
    B = len(ctx)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def filled_cache():
        kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, caps)
        g = torch.Generator(device="cuda").manual_seed(5)
        done = torch.zeros(B, dtype=torch.int32, device="cuda")
        T = max(ctx)
        k = torch.randn(B, T, layer.nkv * layer.hd, generator=g, device="cuda")
        v = torch.randn(B, T, layer.nkv * layer.hd, generator=g, device="cuda")
        D.kv_append(dl, kv, done, k, v, T=T)               # rows past a sequence's context are never read
        return kv

    kv_a, kv_b = filled_cache(), filled_cache()
    len_a = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    len_b = len_a.clone()
    for s in range(steps):
        QP, K, V = [torch.from_numpy(np.stack(x)).cuda() for x in
                    zip(*[[a[0] for a in full_inputs(900 + 10 * s + b, layer, 1)] for b in range(B)])]
        ref = D.full_attn_step(dl, kv_a, len_a, QP, K, V, max_len=max(caps))          # caller scratch
        out = torch.full_like(ref, float("nan"))
        st = lib.ornith_cuda_full_attn_step_static(C.byref(dl.c), C.byref(kv_b.c), _p(len_b), None, _p(QP), _p(K),
                                                   _p(V), _p(out), D.ACT_F32, max(caps), stream)
        assert st == 0, lib.ornith_cuda_last_error()
        torch.cuda.synchronize()
        assert rel_err(out.cpu().numpy(), ref.cpu().numpy()) < TOL, s
        assert (kv_a.K.cpu().numpy() == kv_b.K.cpu().numpy()).all()                   # same rows appended
        D.advance(len_a); D.advance(len_b)


def test_static_scratch_entry_rejects_oversized_requests():
    import torch
    from ornithology_b200 import _lib, device as D
    lib = _lib.load()
    layer = full_case(32)
    dl = device_full(layer)
    B, L = 640, 32768                                      # the query rows alone (10 MiB) exceed the built-in 8 MiB
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [8] * B)
    lens = torch.zeros(B, dtype=torch.int32, device="cuda")
    z = torch.zeros(B, layer.nh * 2 * layer.hd, device="cuda")
    kvin = torch.zeros(B, layer.nkv * layer.hd, device="cuda")
    out = torch.zeros(B, layer.nh * layer.hd, device="cuda")
    st = lib.ornith_cuda_full_attn_step_static(C.byref(dl.c), C.byref(kv.c), _p(lens), None, _p(z), _p(kvin), _p(kvin),
                                               _p(out), D.ACT_F32, L, None)
    assert st != 0
    assert b"built-in" in lib.ornith_cuda_last_error()


def test_static_scratch_entry_fits_long_contexts_at_the_coarse_split():
    """20 sequences x 16 heads with a 32768-token bound: the partials of 512-token splits (21 MB) do not fit the
    built-in array, those of the 2048-token splits the tensor-core kernel accepts (5.6 MB) do, so the call must be
    served, and must agree with the regular entry point given ample scratch."""
    import torch
    from ornithology_b200 import _lib, device as D
    lib = _lib.load()
    layer = full_case(33)
    dl = device_full(layer)
    B, bound = 20, 32768
    ctx = [3000 + 97 * b for b in range(B)]
    caps = [c + 1 for c in ctx]
    g = torch.Generator(device="cuda").manual_seed(6)
    T = max(ctx)
    k = torch.randn(B, T, layer.nkv * layer.hd, generator=g, device="cuda")
    v = torch.randn(B, T, layer.nkv * layer.hd, generator=g, device="cuda")
    kvs = []
    for _ in range(2):
        kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, caps)
        D.kv_append(dl, kv, torch.zeros(B, dtype=torch.int32, device="cuda"), k, v, T=T)
        kvs.append(kv)
    lens = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    QP, K, V = [torch.from_numpy(np.stack(x)).cuda() for x in
                zip(*[[a[0] for a in full_inputs(950 + b, layer, 1)] for b in range(B)])]
    ref = D.full_attn_step(dl, kvs[0], lens, QP, K, V, max_len=bound)
    out = torch.full_like(ref, float("nan"))
    st = lib.ornith_cuda_full_attn_step_static(C.byref(dl.c), C.byref(kvs[1].c), _p(lens), None, _p(QP), _p(K), _p(V),
                                               _p(out), D.ACT_F32, bound, None)
    assert st == 0, lib.ornith_cuda_last_error()
    torch.cuda.synchronize()
    assert rel_err(out.cpu().numpy(), ref.cpu().numpy()) < TOL
