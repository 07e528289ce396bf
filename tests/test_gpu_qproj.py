"""The quantised projections (Q8_0 weights x Q8_K activations) against the engine's integer path.

The oracle restates qdot_quantize_row_q8_K and vec_dot_q8_0 (src/ornith_qdot.c:38-70, :144-163) and is pinned
bit for bit to the reference's own objects (tests/test_oracle_pins.py).  The activation codes and scales must be
the engine's bytes; the products carry one f16 rounding per weight and must stay within 2e-3 of the output's
maximum (measured: about 1e-4)."""
import numpy as np
import pytest

from tests._cases import TOL, bf16_round, rel_err

pytestmark = pytest.mark.gpu


def _acts(seed, T, n_in):
    g = np.random.default_rng(seed)
    X = g.standard_normal((T, n_in)).astype(np.float32)
    X[0, :256] = 0.0                                   # an all-zero block
    if T > 1:
        X[1, 5] = 7.5; X[1, 200] = -7.5                # a tie for the maximum: the first one fixes the sign of the scale
        if n_in > 256:
            X[1, 256 + 9] = -6.25; X[1, 256 + 3] = 6.25    # and the other way round
    if T > 2:
        X[2] *= 1e-3                                   # small values
        X[2, 100] = 0.5 * 127 / 127                    # codes on rounding boundaries
    return X


def test_q8k_blocks_are_the_engines_bytes(oracle):
    import torch
    from ornithology_b200 import device as D
    for T, n_in in ((5, 512), (3, 2048), (9, 256)):
        X = _acts(11 + T, T, n_in)
        ref = oracle.q8k_quantize(X)
        got = D.q8k_quantize(torch.from_numpy(X).cuda(), n_in)
        assert (got == ref).all(), (T, n_in, int((got != ref).sum()))
        Xb = bf16_round(X)
        got = D.q8k_quantize(torch.from_numpy(Xb).cuda().to(torch.bfloat16), n_in)
        assert (got == oracle.q8k_quantize(Xb)).all(), ("bf16", T, n_in)


@pytest.mark.parametrize("T,n_in,n_out", [(1, 2048, 8192), (64, 2048, 8192), (70, 2048, 520), (5, 512, 40), (8, 4096, 2048)])
def test_projection_against_the_integer_path(oracle, T, n_in, n_out):
    import torch
    from ornithology_b200 import device as D
    g = np.random.default_rng(100 + T)
    Wf = (g.standard_normal((n_out, n_in)) * 0.04).astype(np.float32)
    Wf[3] = 0.0                                         # a row of zero blocks
    W = np.stack([oracle.q8_0_encode(r) for r in Wf])
    X = _acts(T, T, n_in)
    ref = oracle.matmul_q8_0(W, n_in, X)
    w = D.Q8_0Weight(W, n_in)
    got = D.matmul_q8_0(w, torch.from_numpy(X).cuda()).cpu().numpy()
    err = rel_err(got, ref)
    print("parity: projection", (T, n_in, n_out), f"err={err:.3g}")
    assert err < TOL, err
    assert (got[:, 3] == 0).all()
    # bf16 activations in, bf16 out
    Xb = bf16_round(X)
    got = D.matmul_q8_0(w, torch.from_numpy(Xb).cuda().to(torch.bfloat16)).float().cpu().numpy()
    assert rel_err(got, oracle.matmul_q8_0(W, n_in, Xb)) < TOL + 2.0 ** -9


# ---- the integer path for all three weight types, bit for bit ---------------------------------------------------

def _random_rows(seed, wtype, n_out, n_in):
    """Rows of random block bytes with finite f16 scales: every code, sub-block scale and minimum value occurs,
    which the encoder's output (small scales, centred codes) does not give."""
    from oracle import oracle as O
    g = np.random.default_rng(seed)
    rb = O.QROW_BYTES[wtype](n_in)
    W = g.integers(0, 256, (n_out, rb), dtype=np.uint8)
    if wtype == O.GGML_Q8_0:
        W.reshape(n_out, -1, 34)[:, :, 1] &= 0x3B                 # |d| < 1: exponent below 15
    elif wtype == O.GGML_Q4_K:
        blk = W.reshape(n_out, -1, 144); blk[:, :, 1] &= 0x3B; blk[:, :, 3] &= 0x3B
    else:
        W.reshape(n_out, -1, 210)[:, :, 209] &= 0x3B
    return W


def _encoded_rows(seed, wtype, n_out, n_in):
    """Rows from the reference's own encoder when its library is at hand, else None."""
    from oracle import oracle as O
    try:
        ref = O.Ref()
    except Exception:
        return None
    g = np.random.default_rng(seed)
    Wf = (g.standard_normal((n_out, n_in)) * 0.04).astype(np.float32)
    Wf[3] = 0.0
    return ref.quantize_rows(wtype, Wf)


@pytest.mark.parametrize("wtype", ["q4_k", "q6_k", "q8_0"])
@pytest.mark.parametrize("T,n_in,n_out", [(1, 2048, 8192), (64, 2048, 1024), (70, 2048, 520), (5, 512, 40), (8, 4096, 512),
                                           (33, 256, 64), (12, 2048, 4096), (24, 2048, 3300), (40, 4096, 6500), (20, 2304, 8192),
                                           (300, 2048, 200), (50, 2048, 4000)])
def test_integer_projection_is_bit_exact(oracle, monkeypatch, wtype, T, n_in, n_out):
    """Q4_K / Q6_K / Q8_0 rows x Q8_K activations: every output equals the engine's integer path bit for bit
    (tensor-core kernel; the plain kernel for Q6_K rows that do not start on 16-byte boundaries: n_in = 512, 256),
    over ragged row and token counts, more than one pass of 64 tokens, f32 and bf16 activations."""
    import torch
    from oracle import oracle as O
    from ornithology_b200 import device as D
    wt = {"q4_k": O.GGML_Q4_K, "q6_k": O.GGML_Q6_K, "q8_0": O.GGML_Q8_0}[wtype]
    X = _acts(T, T, n_in)
    for kind, W in (("random", _random_rows(7 * T + wt, wt, n_out, n_in)), ("encoded", _encoded_rows(T + wt, wt, n_out, n_in))):
        if W is None:
            continue
        ref = oracle.matmul_q(wt, W, n_in, X)
        w = D.QWeight(wt, W, n_in)
        got = D.matmul_q(w, torch.from_numpy(X).cuda()).cpu().numpy()
        bad = got.view(np.uint32) != ref.view(np.uint32)
        assert not bad.any(), (kind, int(bad.sum()), np.argwhere(bad)[:4].tolist())
        Xb = bf16_round(X)
        gotb = D.matmul_q(w, torch.from_numpy(Xb).cuda().to(torch.bfloat16)).float().cpu().numpy()
        assert (gotb == bf16_round(oracle.matmul_q(wt, W, n_in, Xb))).all(), kind
        if kind == "random" and T <= 8:
            monkeypatch.setenv("ORNITH_CUDA_PROJ_PLAIN", "1")
            plain = D.matmul_q(w, torch.from_numpy(X).cuda()).cpu().numpy()
            monkeypatch.delenv("ORNITH_CUDA_PROJ_PLAIN")
            assert (plain.view(np.uint32) == ref.view(np.uint32)).all(), "plain kernel"


def test_projections_sharing_one_image(oracle):
    """One quantisation of the input, three products against it (what the engine does for attn_qkv / attn_gate /
    ssm_alpha of a layer): each equals the integer path bit for bit."""
    import torch
    from oracle import oracle as O
    from ornithology_b200 import device as D
    T, n_in = 7, 2048
    X = _acts(3, T, n_in)
    img = D.q8k_image(torch.from_numpy(X).cuda(), n_in)
    for wt, n_out in ((O.GGML_Q8_0, 8192), (O.GGML_Q6_K, 4096), (O.GGML_Q4_K, 96)):
        W = _random_rows(wt + n_out, wt, n_out, n_in)
        got = D.matmul_q(D.QWeight(wt, W, n_in), None, image=img, T=T).cpu().numpy()
        assert (got.view(np.uint32) == oracle.matmul_q(wt, W, n_in, X).view(np.uint32)).all(), (wt, n_out)


def test_grouped_projections(oracle):
    """The projections of one input as one launch per weight type (attn_qkv, attn_gate, ssm_alpha, ssm_beta of a
    delta-net layer; a mixed list falls into one launch per run of equal types): bit-exact like the single calls."""
    import torch
    from oracle import oracle as O
    from ornithology_b200 import device as D
    n_in = 2048
    for T in (3, 64, 100):
        X = _acts(40 + T, T, n_in)
        img = D.q8k_image(torch.from_numpy(X).cuda(), n_in)
        spec = [(O.GGML_Q8_0, 8192), (O.GGML_Q8_0, 4096), (O.GGML_Q8_0, 32), (O.GGML_Q8_0, 32), (O.GGML_Q6_K, 520), (O.GGML_Q6_K, 72),
                (O.GGML_Q4_K, 40)]
        Ws = [_random_rows(11 * i + T, wt, n_out, n_in) for i, (wt, n_out) in enumerate(spec)]
        ws = [D.QWeight(wt, W, n_in) for (wt, _), W in zip(spec, Ws)]
        outs = D.matmul_q_group(ws, img, T)
        for (wt, n_out), W, y in zip(spec, Ws, outs):
            ref = oracle.matmul_q(wt, W, n_in, X)
            assert (y.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all(), (T, wt, n_out)


def test_integer_projection_golden(golden):
    """Weights from the reference's encoder and outputs from the reference's integer dot (tests/golden/make_golden.py)."""
    import torch
    from ornithology_b200 import device as D
    g = golden("projection_kquant.npz")
    X = torch.from_numpy(g["X"]).cuda()
    for name, wt in (("q4_k", D.GGML_Q4_K), ("q6_k", D.GGML_Q6_K)):
        got = D.matmul_q(D.QWeight(wt, g["W_" + name], int(g["n_in"])), X).cpu().numpy()
        assert (got.view(np.uint32) == g["Y_" + name].view(np.uint32)).all(), name


def test_integer_projection_errors():
    """A weight type without an integer path (Q5_K; the engine falls back to dequantisation there) and a width
    that is not a multiple of 256 are refused with a status, not computed."""
    import torch
    from ornithology_b200 import device as D
    from ornithology_b200._lib import BackendError
    w = D.QWeight(D.GGML_Q4_K, np.zeros(144 * 4, np.uint8), 256)
    w.wtype = 13
    with pytest.raises(BackendError):
        D.matmul_q(w, torch.zeros(2, 256, device="cuda"))
    w = D.QWeight(D.GGML_Q4_K, np.zeros(144 * 4, np.uint8), 256)
    w.n_in = 300
    with pytest.raises(BackendError):
        D.matmul_q(w, torch.zeros(2, 300, device="cuda"))
