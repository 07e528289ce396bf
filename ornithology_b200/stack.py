"""The attention stack of an Ornith model as the engine wires it: 3 gated delta-net
layers for every full-attention layer (reference: src/ornith_model.h:79-82,
src/ornith_rforward.c:686-706), each layer reduced to what lies between its
projections.  One object holds every layer's weights, KV cache, recurrent state
and conv history for a batch of sequences on ONE GPU, optionally as one shard of
a multi-GPU plan:

* sequence sharding — a rank owns whole sequences; layers are complete; nothing is
  exchanged inside the stack;
* head sharding — a rank owns nv/G value heads of every delta-net layer (with the
  key heads they pair with) and nh/G query heads of every full layer with the one
  KV head they read; the per-head outputs are re-assembled by an all-gather
  before the output projection.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import device as D

ARCHS = {   # reference: src/ornith_model.c:5-77
    "35b": dict(hidden=2048, layers=40, interval=4, nh=16, nkv=2, hd=256, rope_dim=64, theta=1e7,
                nk=16, nv=32, dk=128, dv=128, conv_k=4, eps=1e-6),
    "397b": dict(hidden=4096, layers=60, interval=4, nh=32, nkv=2, hd=256, rope_dim=64, theta=1e7,
                 nk=16, nv=64, dk=128, dv=128, conv_k=4, eps=1e-6),
}


def is_full_layer(arch: dict, i: int) -> bool:
    return arch["interval"] > 0 and i % arch["interval"] == arch["interval"] - 1


@dataclass
class HeadShard:
    """What one rank of a head-sharded plan owns (world = G ranks)."""
    rank: int
    world: int
    v_heads: range          # value heads of the delta-net layers
    k_heads: range          # key heads those value heads pair with (tiled map)
    q_heads: range          # query heads of the full layers
    kv_heads: range         # KV heads they read (replicated when world > n_kv_heads)


def head_shard(arch: dict, rank: int, world: int) -> HeadShard:
    nk, nv, nh, nkv = arch["nk"], arch["nv"], arch["nh"], arch["nkv"]
    if nv % world or nh % world:
        raise ValueError(f"{world} ranks do not divide {nv} value heads / {nh} query heads")
    pv, ph = nv // world, nh // world
    v0 = rank * pv
    if pv >= nk:
        if pv % nk:
            raise ValueError("value heads per rank must be a multiple of the key heads")
        k_heads = range(0, nk)
    else:
        if nk % pv:
            raise ValueError("key heads must be a multiple of the value heads per rank")
        k0 = v0 % nk
        k_heads = range(k0, k0 + pv)
    group = nh // nkv
    kv_lo, kv_hi = (rank * ph) // group, (rank * ph + ph - 1) // group
    return HeadShard(rank, world, range(v0, v0 + pv), k_heads, range(rank * ph, rank * ph + ph),
                     range(kv_lo, kv_hi + 1))


def sequence_shard(contexts, rank: int, world: int):
    """Indices of the sequences rank `rank` owns under sequence sharding: equal counts per
    rank, balanced by total context (longest first onto the least loaded rank with room)."""
    contexts = np.asarray(contexts)
    n = len(contexts)
    cap = -(-n // world)
    load = [0] * world
    owned = [[] for _ in range(world)]
    for i in sorted(range(n), key=lambda i: (-int(contexts[i]), i)):
        r = min((r for r in range(world) if len(owned[r]) < cap), key=lambda r: (load[r], r))
        owned[r].append(i)
        load[r] += int(contexts[i])
    return sorted(owned[rank])


def gather_heads(local: torch.Tensor, world: int) -> torch.Tensor:
    """All-gather of per-rank head outputs [..., width/world] -> [..., width] (rank r owns the
    r-th block of heads), the one collective of the head-sharded plan; it runs before the
    output projection (reference call sites: src/ornith_rforward.c:452, :316)."""
    import torch.distributed as dist
    if world == 1:
        return local
    local = local.contiguous()
    flat = local.reshape(-1, local.shape[-1])
    buf = torch.empty((world * flat.shape[0], flat.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, flat)                      # rank blocks stacked along dim 0
    out = buf.view(world, flat.shape[0], flat.shape[1]).movedim(0, 1).reshape(flat.shape[0], -1)
    return out.reshape(*local.shape[:-1], world * local.shape[-1])


def linear_weights(arch: dict, seed: int, layer: int):
    """Seeded synthetic weights of one delta-net layer (value ranges as in the
    reference's fixture model, tests/test_session.c:76, :121-126)."""
    g = np.random.default_rng([seed, layer, 1])
    cc = 2 * arch["nk"] * arch["dk"] + arch["nv"] * arch["dv"]
    return dict(conv_w=g.uniform(-0.2, 0.2, (cc, arch["conv_k"])).astype(np.float32),
                a_coef=g.uniform(-0.8, -0.2, arch["nv"]).astype(np.float32),
                dt_bias=g.uniform(-0.05, 0.05, arch["nv"]).astype(np.float32),
                norm_w=g.uniform(0.9, 1.1, arch["dv"]).astype(np.float32))


def full_weights(arch: dict, seed: int, layer: int):
    g = np.random.default_rng([seed, layer, 2])
    return dict(q_norm_w=g.uniform(0.9, 1.1, arch["hd"]).astype(np.float32),
                k_norm_w=g.uniform(0.9, 1.1, arch["hd"]).astype(np.float32))


def shard_linear_weights(arch: dict, w: dict, sh: HeadShard):
    """Slice one delta-net layer's weights down to a rank's heads; channel order
    stays [q | k | v] (reference: src/ornith_rforward.c:470)."""
    dk, dv, qd = arch["dk"], arch["dv"], arch["nk"] * arch["dk"]
    kq = np.concatenate([np.arange(h * dk, (h + 1) * dk) for h in sh.k_heads])
    vv = np.concatenate([np.arange(h * dv, (h + 1) * dv) for h in sh.v_heads])
    chan = np.concatenate([kq, qd + kq, 2 * qd + vv])
    heads = np.array(list(sh.v_heads))
    return dict(conv_w=w["conv_w"][chan], a_coef=w["a_coef"][heads], dt_bias=w["dt_bias"][heads],
                norm_w=w["norm_w"]), chan


class AttnStack:
    """All attention layers of one model for `n_seq` sequences on one device."""

    def __init__(self, arch_name: str, capacities, kv_mode=D.KV_Q8_0, seed=0, device="cuda:0",
                 shard: HeadShard | None = None, n_layers: int | None = None):
        self.arch = arch = ARCHS[arch_name] if isinstance(arch_name, str) else arch_name
        self.n_seq = len(capacities)
        self.kv_mode = kv_mode
        self.device = torch.device(device)
        self.shard = shard
        self.layers = []                # (kind, layer, state)
        nk, nv, nh, nkv = arch["nk"], arch["nv"], arch["nh"], arch["nkv"]
        if shard is not None:
            nk, nv, nh, nkv = len(shard.k_heads), len(shard.v_heads), len(shard.q_heads), len(shard.kv_heads)
        self.nk, self.nv, self.nh, self.nkv = nk, nv, nh, nkv
        for i in range(arch["layers"] if n_layers is None else n_layers):
            if is_full_layer(arch, i):
                w = full_weights(arch, seed, i)
                layer = D.FullLayer(nh, nkv, arch["hd"], w["q_norm_w"], w["k_norm_w"], rope_dim=arch["rope_dim"],
                                    theta=arch["theta"], eps=arch["eps"], gated=True, device=device)
                state = D.KvBatch(kv_mode, nkv, arch["hd"], capacities, device=device)
                self.layers.append(("full", layer, state))
            else:
                w = linear_weights(arch, seed, i)
                if shard is not None:
                    w, _ = shard_linear_weights(arch, w, shard)
                layer = D.LinearLayer(nk, nv, arch["dk"], arch["dv"], w["conv_w"], w["a_coef"], w["dt_bias"],
                                      w["norm_w"], conv_k=arch["conv_k"], head_map=D.HEADMAP_TILED,
                                      eps=arch["eps"], device=device)
                self.layers.append(("linear", layer, D.LinearState(layer, self.n_seq, device=device)))
        self.pos = torch.zeros(self.n_seq, dtype=torch.int32, device=device)   # tokens seen per sequence
        self.max_capacity = max(int(c) for c in capacities)

    # ---- shapes of one layer's inputs / output, per sequence -------------------------
    def input_widths(self, kind):
        a = self.arch
        if kind == "full":
            return (self.nh * 2 * a["hd"], self.nkv * a["hd"], self.nkv * a["hd"])
        cc = 2 * self.nk * a["dk"] + self.nv * a["dv"]
        return (cc, self.nv, self.nv, self.nv * a["dv"])

    def output_width(self, kind):
        return self.nh * self.arch["hd"] if kind == "full" else self.nv * self.arch["dv"]

    def random_inputs(self, seed, dtype=torch.bfloat16, device=None, pin=False):
        """One token of N(0,1) activations per sequence for every layer."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        out = []
        for kind, _, _ in self.layers:
            ts = [torch.randn(self.n_seq, w, generator=g, dtype=torch.float32).to(dtype) for w in self.input_widths(kind)]
            if pin:
                ts = [t.pin_memory() for t in ts]
            elif device is not None:
                ts = [t.to(device) for t in ts]
            out.append(ts)
        return out

    # ---- one decode token per sequence through every layer ---------------------------
    def decode_step(self, inputs, outputs=None, max_len=None):
        """inputs[i] = device tensors of layer i (qkv,a,b,z | qproj,k,v); returns the
        per-layer head outputs.  `max_len` bounds the longest context after the append."""
        if max_len is None:
            max_len = self.max_capacity
        outs = []
        for i, (kind, layer, state) in enumerate(self.layers):
            out = None if outputs is None else outputs[i]
            if kind == "full":
                outs.append(D.full_attn_step(layer, state, self.pos, *inputs[i], out=out, max_len=max_len))
            else:
                outs.append(D.linear_attn_step(layer, state, self.pos, *inputs[i], out=out))
        D.advance(self.pos)
        return outs

    def decode_step_gathered(self, inputs, world, max_len=None):
        """Head-sharded decode step: every layer's local head outputs are all-gathered (NCCL
        over NVLink) into the full-width row the output projection consumes."""
        outs = self.decode_step(inputs, max_len=max_len)
        return [gather_heads(o, world) for o in outs]

    def shard_inputs(self, full_inputs):
        """Slice full-width per-layer inputs (as an unsharded stack takes them) down to this
        rank's heads."""
        if self.shard is None:
            return full_inputs
        a, sh = self.arch, self.shard
        dev = self.device
        qcols = torch.tensor(np.concatenate([np.arange(h * 2 * a["hd"], (h + 1) * 2 * a["hd"]) for h in sh.q_heads]), device=dev)
        kcols = torch.tensor(np.concatenate([np.arange(h * a["hd"], (h + 1) * a["hd"]) for h in sh.kv_heads]), device=dev)
        _, chan = shard_linear_weights(a, linear_weights(a, 0, 0), sh)
        chan = torch.tensor(chan, device=dev)
        heads = torch.tensor(list(sh.v_heads), device=dev)
        vcols = torch.tensor(np.concatenate([np.arange(h * a["dv"], (h + 1) * a["dv"]) for h in sh.v_heads]), device=dev)
        out = []
        for (kind, _, _), ins in zip(self.layers, full_inputs):
            if kind == "full":
                out.append([ins[0][..., qcols].contiguous(), ins[1][..., kcols].contiguous(), ins[2][..., kcols].contiguous()])
            else:
                out.append([ins[0][..., chan].contiguous(), ins[1][..., heads].contiguous(), ins[2][..., heads].contiguous(),
                            ins[3][..., vcols].contiguous()])
        return out

    def launches_per_step(self):
        """Kernel launches of one decode step, mirroring the library's dispatch: a full-attention layer is
        append + split-K decode (+ a merge kernel unless the decode kernel merges itself: Q8_0 rows, head_dim 256,
        groups of at most 16 query heads); a delta-net layer is one kernel, or front-end + state kernel above 296
        (sequence, value head) units; one launch advances the positions."""
        n_full = sum(1 for k, _, _ in self.layers if k == "full")
        n_lin = len(self.layers) - n_full
        fused_merge = self.kv_mode == D.KV_Q8_0 and self.arch["hd"] == 256 and self.nh // max(self.nkv, 1) <= 16
        two_kernels = self.arch["dk"] == 128 and self.arch["dv"] == 128 and self.n_seq * self.nv > 296
        return (2 if fused_merge else 3) * n_full + (2 if two_kernels else 1) * n_lin + 1

    # ---- synthetic prefill of the state (bench set-up) -------------------------------
    def fill(self, contexts, seed=0, linear_tokens=64, block=2048):
        """Bring every sequence to its context length: KV rows from seeded N(0,1) k/v
        activations pushed through the append kernel (k RMSNorm + RoPE + encode);
        recurrent state and conv history from `linear_tokens` tokens of N(0,1)
        activations pushed through the chunked prefill."""
        contexts = [int(c) for c in contexts]
        assert len(contexts) == self.n_seq
        a = self.arch
        g = torch.Generator(device=self.device).manual_seed(seed)
        kvd = self.nkv * a["hd"]
        for kind, layer, state in self.layers:
            if kind == "full":
                done = torch.zeros(self.n_seq, dtype=torch.int32, device=self.device)
                remaining = list(contexts)
                while max(remaining) > 0:
                    T = min(block, max(remaining))
                    # sequences shorter than T simply hit their target: cap the append per sequence
                    k = torch.randn(self.n_seq, T, kvd, generator=g, device=self.device, dtype=torch.float32).to(torch.bfloat16)
                    v = torch.randn(self.n_seq, T, kvd, generator=g, device=self.device, dtype=torch.float32).to(torch.bfloat16)
                    # run the append for the longest; shorter ones are trimmed by re-setting their length
                    D.kv_append(layer, state, done, k, v, T=T)
                    step = torch.tensor([min(T, r) for r in remaining], dtype=torch.int32, device=self.device)
                    done += step
                    remaining = [max(0, r - T) for r in remaining]
            else:
                T = linear_tokens
                ins = [torch.randn(self.n_seq, T, w, generator=g, device=self.device, dtype=torch.float32).to(torch.bfloat16)
                       for w in self.input_widths("linear")]
                z = torch.zeros(self.n_seq, dtype=torch.int32, device=self.device)
                D.linear_attn_prefill(layer, state, z, *ins, T, chunk=32)
        self.pos = torch.tensor(contexts, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)

    # ---- algorithmic bytes one decode step must move (the roofline numerator) ---------
    def decode_bytes(self, contexts, act_bytes=2):
        a = self.arch
        total_lin = total_full = 0
        cc = 2 * self.nk * a["dk"] + self.nv * a["dv"]
        vd = self.nv * a["dv"]
        for kind, layer, state in self.layers:
            if kind == "linear":
                per_seq = (2 * self.nv * a["dv"] * a["dk"] * 4            # state read + write
                           + (a["conv_k"] - 1) * cc * 4 + cc * 4          # conv history read + one slot written
                           + cc * act_bytes + 2 * self.nv * act_bytes + 2 * vd * act_bytes)
                total_lin += per_seq * self.n_seq
            else:
                rb = state.row_bytes
                extra = 4 if state.mode == D.KV_INT8_HEAD else 0
                for L in contexts:
                    total_full += (2 * self.nkv * (rb + extra) * (L + 1)   # K and V rows read once per kv head
                                   + 2 * self.nkv * (rb + extra)           # appended rows
                                   + self.nh * a["hd"] * 3 * act_bytes     # q + gate in, out
                                   + 2 * self.nkv * a["hd"] * act_bytes)   # k, v in
        return total_lin, total_full
