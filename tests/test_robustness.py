"""Failure paths, exercised without faulting anything: the allocation hook (host-side injection), the status word
of a bounded wait that gives up, the per-stream buffer release, and one process driving two devices."""
import ctypes as C

import numpy as np
import pytest

HOOK = C.CFUNCTYPE(C.c_int, C.c_size_t, C.c_void_p)
ORNITH_ERR_OOM, ORNITH_ERR_BACKEND = 4, 6


@pytest.fixture(scope="module")
def lib():
    from ornithology_b200 import _lib, build
    build.build()
    return _lib.load()


def test_allocation_hook_fails_the_nth_allocation(lib):
    """No GPU needed: the hook is consulted before the device is touched, so a host can test its out-of-memory
    handling anywhere (reference behaviour: the OOM checks of the init functions, src/ornith_attn.c:32-46)."""
    import torch
    calls = []

    def refuse_third(nbytes, _user):
        calls.append(int(nbytes))
        return 1 if len(calls) == 3 else 0

    hook = HOOK(refuse_third)
    lib.ornith_cuda_set_alloc_hook(C.cast(hook, C.c_void_p), None)
    try:
        p = C.c_void_p()
        codes = [lib.ornith_cuda_malloc(C.byref(p), 1000 + i) for i in range(4)]
        ok = 0 if torch.cuda.is_available() else ORNITH_ERR_BACKEND      # without a GPU the allocation itself cannot succeed
        assert codes == [ok, ok, ORNITH_ERR_OOM, ok]
        assert calls == [1000, 1001, 1002, 1003]
    finally:
        lib.ornith_cuda_set_alloc_hook(None, None)
    lib.ornith_cuda_malloc(C.byref(p), 64)
    assert len(calls) == 4                                               # hook cleared


@pytest.mark.gpu
def test_allocation_failure_reaches_the_drop_in(lib):
    """Tier 1 with a hook that refuses everything: the KV mirror cannot be built, the step records an error and
    leaves the host images untouched, as it does without a GPU; once the hook is gone the same call works."""
    from ornithology_b200 import attn
    refuse = HOOK(lambda nbytes, user: 1)
    c = attn.kv_init(8, 1, 16)
    q = np.ones(16, np.float32)
    out = np.full(16, 7.0, np.float32)
    lib.ornith_cuda_set_alloc_hook(C.cast(refuse, C.c_void_p), None)
    try:
        attn.gqa_step(c, q, q, q, 1, out=out)
        assert (out == 7.0).all() and c.len == 0
        assert b"refused by the allocation hook" in lib.ornith_cuda_last_error()
    finally:
        lib.ornith_cuda_set_alloc_hook(None, None)
    attn.gqa_step(c, q, q, q, 1, out=out)
    assert c.len == 1 and np.allclose(out, 1.0, atol=1e-6)               # one cached row: the output is v
    attn.kv_free(c)


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_the_context_survives(lib, oracle):
    """The waits inside the tensor-core kernels are bounded.  The self-test kernel waits a few polls on a barrier
    nobody arrives on: it must come back, set the device's status word, and the next synchronisation must turn
    that into ORNITH_ERR_BACKEND; afterwards the same context computes correctly."""
    import torch
    from ornithology_b200 import device as D
    from tests._cases import TOL, device_full, full_case, full_inputs, rel_err
    assert lib.ornith_cuda_poll_status() == 0
    assert lib.ornith_cuda_selftest_wait_timeout(8) == ORNITH_ERR_BACKEND
    assert b"gave up a bounded wait" in lib.ornith_cuda_last_error() and b"self-test" in lib.ornith_cuda_last_error()
    assert lib.ornith_cuda_poll_status() == 0                            # reading the word clears it
    assert lib.ornith_cuda_sync(None) == 0
    layer = full_case(2)
    dl = device_full(layer)
    QP, K, V = full_inputs(5, layer, 3)
    kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [3])
    okv = oracle.kv(3, layer.nkv, layer.hd, 2)
    kv_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    for t in range(3):
        out = D.full_attn_step(dl, kv, kv_len, torch.from_numpy(QP[t:t + 1]).cuda(), torch.from_numpy(K[t:t + 1]).cuda(),
                               torch.from_numpy(V[t:t + 1]).cuda())
        assert rel_err(out.cpu().numpy()[0], oracle.full_attn_step(layer, okv, t, QP[t], K[t], V[t])) < TOL
        D.advance(kv_len)


@pytest.mark.gpu
def test_stream_release_frees_the_decode_work_buffer(lib, oracle):
    """The large-batch delta-net decode keeps one work buffer per (device, stream); a host that destroys streams
    releases it first.  The step still works (and re-allocates) afterwards."""
    import torch
    from ornithology_b200 import device as D
    from tests._cases import TOL, device_linear, linear_case, rel_err
    layer, kw = linear_case(3, nk=4, nv=8)
    dl = device_linear(layer, kw)
    B = 48                                                               # 384 (sequence, head) units: the two-kernel path
    g = np.random.default_rng(9)
    ins = [g.standard_normal((B, n)).astype(np.float32) for n in (layer.cc, layer.nv, layer.nv, layer.vd)]
    side = torch.cuda.Stream()
    ref0 = None
    for rep in range(2):
        st = D.LinearState(dl, B)
        pos = torch.zeros(B, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            out = D.linear_attn_step(dl, st, pos, *[torch.from_numpy(x).cuda() for x in ins]).cpu().numpy()
        assert lib.ornith_cuda_stream_release(C.c_void_p(side.cuda_stream), 0) == 0
        S = np.zeros((layer.nv, 128, 128), np.float32); buf = np.zeros(3 * layer.cc, np.float32)
        ref0 = oracle.linear_attn_step(layer, S, buf, *[x[0] for x in ins]) if ref0 is None else ref0
        assert rel_err(out[0], ref0) < TOL, rep
    assert lib.ornith_cuda_stream_release(None, 1) == 0                  # every stream of the device


@pytest.mark.gpu
def test_one_process_two_devices(lib, oracle):
    """The shared-memory opt-in of a kernel and the SM count belong to a device: a process that computes on GPU 0 and
    then on GPU 1 must get the same answers on both (plain launches only, nothing crosses between the GPUs)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from ornithology_b200 import device as D
    from tests._cases import TOL, device_full, device_linear, full_case, full_inputs, linear_case, linear_inputs, rel_err
    layer = full_case(12)
    lin, kw = linear_case(13, nk=4, nv=8)
    T = 130
    QP, K, V = full_inputs(14, layer, T + 1)
    okv = oracle.kv(T + 1, layer.nkv, layer.hd, 2)
    ref_pre = oracle.full_attn_prefill(layer, okv, 0, QP[:T], K[:T], V[:T])
    ref_step = oracle.full_attn_step(layer, okv, T, QP[T], K[T], V[T])
    li = linear_inputs(15, lin, T)
    S = np.zeros((lin.nv, 128, 128), np.float32); buf = np.zeros(3 * lin.cc, np.float32)
    ref_lin = oracle.linear_attn_prefill(lin, S, buf, *li, chunk=64)
    try:
        for dev in (0, 1):
            assert lib.ornith_cuda_set_device(dev) == 0
            torch.cuda.set_device(dev)
            d = f"cuda:{dev}"
            dl = device_full(layer, device=d)
            kv = D.KvBatch(D.KV_Q8_0, layer.nkv, layer.hd, [T + 1], device=d)
            kv_len = torch.zeros(1, dtype=torch.int32, device=d)
            to = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(d)
            out = D.full_attn_prefill(dl, kv, kv_len, to(QP[:T])[None], to(K[:T])[None], to(V[:T])[None], T)
            assert rel_err(out.cpu().numpy()[0], ref_pre) < TOL, dev
            D.advance(kv_len, T)
            out = D.full_attn_step(dl, kv, kv_len, to(QP[T:T + 1]), to(K[T:T + 1]), to(V[T:T + 1]))
            assert rel_err(out.cpu().numpy()[0], ref_step) < TOL, dev
            dlin = device_linear(lin, kw, device=d)
            st = D.LinearState(dlin, 1)
            pos = torch.zeros(1, dtype=torch.int32, device=d)
            out = D.linear_attn_prefill(dlin, st, pos, *[to(x)[None] for x in li], T, chunk=64)
            assert rel_err(out.cpu().numpy()[0], ref_lin) < TOL, dev
            assert rel_err(st.S.cpu().numpy()[0], S) < TOL, dev
            # the integer projections opt into their shared memory per device as well
            from oracle import oracle as O
            g = np.random.default_rng(16)
            Wq = g.integers(0, 256, (96, O.QROW_BYTES[O.GGML_Q4_K](512)), dtype=np.uint8)
            blk = Wq.reshape(96, 2, 144); blk[:, :, 1] &= 0x3B; blk[:, :, 3] &= 0x3B
            Xq = g.standard_normal((5, 512)).astype(np.float32)
            got = D.matmul_q(D.QWeight(O.GGML_Q4_K, Wq, 512, device=d), to(Xq)).cpu().numpy()
            assert (got.view(np.uint32) == oracle.matmul_q(O.GGML_Q4_K, Wq, 512, Xq).view(np.uint32)).all(), dev
    finally:
        lib.ornith_cuda_set_device(0)
        torch.cuda.set_device(0)


@pytest.mark.gpu
def test_gather_layout_matches_a_transpose(lib):
    """[world][rows][width] rank blocks -> [rows][world * width] full-width rows, bf16 and f32."""
    import torch
    for dt, eb in ((torch.bfloat16, 2), (torch.float32, 4)):
        world, rows, width = 4, 37, 136
        g = torch.randn(world, rows, width, device="cuda").to(dt)
        full = torch.empty(rows, world * width, dtype=dt, device="cuda")
        assert lib.ornith_cuda_gather_layout(C.c_void_p(g.data_ptr()), C.c_void_p(full.data_ptr()), world, rows, width, eb, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(full, g.movedim(0, 1).reshape(rows, world * width))
