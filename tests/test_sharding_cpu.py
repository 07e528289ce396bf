"""Multi-GPU partitioning, checked on the CPU: a head shard is a smaller layer.

The oracle runs a full layer and the per-rank sub-layers that `stack.head_shard` /
`stack.shard_linear_weights` produce; concatenating the ranks' head outputs must give the full
layer's output bit for bit (heads never interact: reference src/ornith_rforward.c:488-498,
src/ornith_attn.c:115-147).  The world_size-2 test does the same with two gloo ranks and an
all-gather, which is the one collective of the head-sharded plan.
"""
import os
import sys

import numpy as np
import pytest

from oracle import oracle as O
from ornithology_b200 import stack as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("arch", ["35b", "397b"])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_head_shards_cover_every_head_once(arch, world):
    a = S.ARCHS[arch]
    shards = [S.head_shard(a, r, world) for r in range(world)]
    assert sorted(h for s in shards for h in s.v_heads) == list(range(a["nv"]))
    assert sorted(h for s in shards for h in s.q_heads) == list(range(a["nh"]))
    group = a["nh"] // a["nkv"]
    for s in shards:
        # the key heads a rank holds are exactly those its value heads pair with (tiled map)
        assert sorted({hv % a["nk"] for hv in s.v_heads}) == list(s.k_heads)
        # local tiled map == global tiled map
        for i, hv in enumerate(s.v_heads):
            assert list(s.k_heads)[i % len(s.k_heads)] == hv % a["nk"]
        assert sorted({h // group for h in s.q_heads}) == list(s.kv_heads)
        assert len(s.q_heads) % len(s.kv_heads) == 0


def _small_arch():
    return dict(S.ARCHS["35b"], nk=4, nv=8, dk=32, dv=32, nh=8, nkv=2, hd=64, rope_dim=16, layers=4)


def _linear_full_and_shards(world, seed=0, T=5):
    a = _small_arch()
    w = S.linear_weights(a, seed, 0)
    full = O.LinearLayer(a["nk"], a["nv"], a["dk"], a["dv"], w["conv_w"], w["a_coef"], w["dt_bias"], w["norm_w"])
    g = np.random.default_rng(seed + 1)
    ins = [g.standard_normal((T, n)).astype(np.float32) for n in (full.cc, a["nv"], a["nv"], full.vd)]
    return a, w, full, ins


def _run_linear(orc, layer, ins):
    S_ = np.zeros((layer.nv, layer.dv, layer.dk), np.float32)
    buf = np.zeros(3 * layer.cc, np.float32)
    return np.stack([orc.linear_attn_step(layer, S_, buf, *[np.ascontiguousarray(x[t]) for x in ins])
                     for t in range(ins[0].shape[0])])


def _shard_inputs(a, sh, chan, ins):
    heads = np.array(list(sh.v_heads))
    vcols = np.concatenate([np.arange(h * a["dv"], (h + 1) * a["dv"]) for h in sh.v_heads])
    return [ins[0][:, chan], ins[1][:, heads], ins[2][:, heads], ins[3][:, vcols]], vcols


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_delta_net_layers_reproduce_the_full_layer(oracle, world):
    a, w, full, ins = _linear_full_and_shards(world)
    ref = _run_linear(oracle, full, ins)
    out = np.zeros_like(ref)
    for r in range(world):
        sh = S.head_shard(a, r, world)
        ws, chan = S.shard_linear_weights(a, w, sh)
        sub = O.LinearLayer(len(sh.k_heads), len(sh.v_heads), a["dk"], a["dv"], ws["conv_w"], ws["a_coef"],
                            ws["dt_bias"], ws["norm_w"])
        sins, vcols = _shard_inputs(a, sh, chan, ins)
        out[:, vcols] = _run_linear(oracle, sub, sins)
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_full_layers_reproduce_the_full_layer(oracle, world):
    a = _small_arch()
    fw = S.full_weights(a, 0, 3)
    full = O.FullLayer(a["nh"], a["nkv"], a["hd"], fw["q_norm_w"], fw["k_norm_w"], rope_dim=a["rope_dim"])
    g = np.random.default_rng(2)
    T = 6
    QP = g.standard_normal((T, a["nh"] * 2 * a["hd"])).astype(np.float32)
    K = g.standard_normal((T, a["nkv"] * a["hd"])).astype(np.float32)
    V = g.standard_normal((T, a["nkv"] * a["hd"])).astype(np.float32)
    kv = oracle.kv(T, a["nkv"], a["hd"], O.KV_Q8_0)
    ref = np.stack([oracle.full_attn_step(full, kv, t, QP[t], K[t], V[t]) for t in range(T)])
    out = np.zeros_like(ref)
    for r in range(world):
        sh = S.head_shard(a, r, world)
        sub = O.FullLayer(len(sh.q_heads), len(sh.kv_heads), a["hd"], fw["q_norm_w"], fw["k_norm_w"], rope_dim=a["rope_dim"])
        qcols = np.concatenate([np.arange(h * 2 * a["hd"], (h + 1) * 2 * a["hd"]) for h in sh.q_heads])
        kcols = np.concatenate([np.arange(h * a["hd"], (h + 1) * a["hd"]) for h in sh.kv_heads])
        ocols = np.concatenate([np.arange(h * a["hd"], (h + 1) * a["hd"]) for h in sh.q_heads])
        skv = oracle.kv(T, len(sh.kv_heads), a["hd"], O.KV_Q8_0)
        out[:, ocols] = np.stack([oracle.full_attn_step(sub, skv, t, np.ascontiguousarray(QP[t, qcols]),
                                                        np.ascontiguousarray(K[t, kcols]), np.ascontiguousarray(V[t, kcols]))
                                  for t in range(T)])
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()


def test_sequence_sharding_is_a_partition():
    ctx = np.arange(1, 65) * 100
    for world in (1, 2, 4, 8):
        parts = [S.sequence_shard(ctx, r, world) for r in range(world)]
        assert sorted(i for p in parts for i in p) == list(range(64))
        loads = [int(ctx[p].sum()) for p in parts]
        assert max(loads) - min(loads) <= ctx.max()        # balanced by total context


def _gloo_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle.oracle import Oracle
    orc = Oracle()
    a, w, full, ins = _linear_full_and_shards(world)
    sh = S.head_shard(a, rank, world)
    ws, chan = S.shard_linear_weights(a, w, sh)
    sub = O.LinearLayer(len(sh.k_heads), len(sh.v_heads), a["dk"], a["dv"], ws["conv_w"], ws["a_coef"], ws["dt_bias"], ws["norm_w"])
    sins, _ = _shard_inputs(a, sh, chan, ins)
    mine = torch.from_numpy(_run_linear(orc, sub, sins))               # [T, vd / world]
    gathered = S.gather_heads(mine, world)                              # the plan's one collective
    if rank == 0:
        ref = _run_linear(orc, full, ins)
        q.put(bool((gathered.numpy().view(np.uint32) == ref.view(np.uint32)).all()))
    dist.destroy_process_group()


def test_two_gloo_ranks_all_gather_head_outputs():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 400)
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert q.get(timeout=10) is True


def test_c_head_shard_matches_the_python_plan():
    """The C entry point a host engine would call (ornith_cuda_head_shard) and the Python harness agree on who owns
    which heads, for both model shapes and every rank count that divides the heads; bad splits are refused."""
    import ctypes as C
    from ornithology_b200 import _lib, build
    from ornithology_b200.stack import ARCHS, head_shard
    build.build()
    lib = _lib.load()
    for name, a in ARCHS.items():
        for world in (1, 2, 4, 8, 16):
            if a["nv"] % world or a["nh"] % world:
                continue
            for rank in range(world):
                sh = _lib.CudaShard()
                assert lib.ornith_cuda_head_shard(a["nk"], a["nv"], a["nh"], a["nkv"], rank, world, C.byref(sh)) == 0
                py = head_shard(a, rank, world)
                assert (sh.v_head0, sh.n_v_heads) == (py.v_heads.start, len(py.v_heads)), (name, world, rank)
                assert (sh.k_head0, sh.n_k_heads) == (py.k_heads.start, len(py.k_heads))
                assert (sh.q_head0, sh.n_q_heads) == (py.q_heads.start, len(py.q_heads))
                assert (sh.kv_head0, sh.n_kv_heads) == (py.kv_heads.start, len(py.kv_heads))
    sh = _lib.CudaShard()
    assert lib.ornith_cuda_head_shard(16, 32, 16, 2, 0, 3, C.byref(sh)) != 0          # 3 ranks do not divide the heads
    assert lib.ornith_cuda_head_shard(16, 32, 16, 2, 5, 4, C.byref(sh)) != 0          # rank out of range
