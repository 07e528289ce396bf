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
