"""Shared builders for the GPU parity tests: the same seeded layer handed to the
CPU oracle and to the CUDA library."""
import numpy as np

from oracle import oracle as O

TOL = 2e-3          # max |gpu - ref| / max |ref| per tensor (the stated parity bar)


def rel_err(got, ref):
    got = np.asarray(got, np.float64); ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "non-finite values in the CUDA result"
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def bf16_round(x):
    """float32 values rounded to bfloat16 (RNE) and widened back."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


def linear_case(seed, nk=16, nv=32, dk=128, dv=128, head_map=O.HEADMAP_TILED, bias=False, scaled=True):
    g = np.random.default_rng(seed)
    cc = 2 * nk * dk + nv * dv
    kw = dict(conv_w=g.uniform(-0.2, 0.2, (cc, 4)).astype(np.float32),
              a_coef=g.uniform(-0.8, -0.2, nv).astype(np.float32),
              dt_bias=g.uniform(-0.05, 0.05, nv).astype(np.float32),
              norm_w=g.uniform(0.9, 1.1, dv).astype(np.float32),
              conv_b=g.uniform(-0.1, 0.1, cc).astype(np.float32) if bias else None,
              head_map=head_map, out_scale=None if scaled else 1.0)
    return O.LinearLayer(nk, nv, dk, dv, **kw), kw


def linear_inputs(seed, layer, T, bf16=False):
    g = np.random.default_rng(seed)
    arrs = [g.standard_normal((T, layer.cc)), g.standard_normal((T, layer.nv)),
            g.standard_normal((T, layer.nv)), g.standard_normal((T, layer.vd))]
    arrs = [a.astype(np.float32) for a in arrs]
    if bf16:
        arrs = [bf16_round(a) for a in arrs]
    return arrs


def device_linear(layer, kw, device="cuda:0"):
    from ornithology_b200 import device as D
    return D.LinearLayer(layer.nk, layer.nv, layer.dk, layer.dv, kw["conv_w"], kw["a_coef"], kw["dt_bias"],
                         kw["norm_w"], conv_b=kw["conv_b"], head_map=kw["head_map"],
                         out_scale=layer.out_scale, device=device)


def full_case(seed, nh=16, nkv=2, hd=256, rope_dim=64, theta=1e7):
    g = np.random.default_rng(seed)
    qw = g.uniform(0.9, 1.1, hd).astype(np.float32)
    kw = g.uniform(0.9, 1.1, hd).astype(np.float32)
    return O.FullLayer(nh, nkv, hd, qw, kw, rope_dim=rope_dim, theta=theta)


def full_inputs(seed, layer, T, bf16=False):
    g = np.random.default_rng(seed)
    arrs = [g.standard_normal((T, layer.nh * 2 * layer.hd)), g.standard_normal((T, layer.nkv * layer.hd)),
            g.standard_normal((T, layer.nkv * layer.hd))]
    arrs = [a.astype(np.float32) for a in arrs]
    if bf16:
        arrs = [bf16_round(a) for a in arrs]
    return arrs


def device_full(layer, device="cuda:0"):
    from ornithology_b200 import device as D
    return D.FullLayer(layer.nh, layer.nkv, layer.hd, layer.q_norm_w, layer.k_norm_w, rope_dim=layer.rope_dim,
                       theta=layer.theta, eps=layer.eps, gated=True, device=device)
