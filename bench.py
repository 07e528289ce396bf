#!/usr/bin/env python
"""Attention-stack decode benchmark.

Headline workload: batched decode through a 40-layer 35B-shaped attention stack (30 gated
delta-net + 10 GQA layers, 3:1).  One step = one token for each of 64 concurrent sequences per
GPU, Q8_0 KV cache, fp32 recurrent state, bf16 activations, contexts uniform in [1k, 32k].
Multi-GPU runs shard by sequence: N x 64 sequences are drawn once and dealt to the ranks so that
the summed contexts balance (weak scaling, nothing is exchanged inside the stack).

Further legs on the same JSON line (each an object of its own):
  prefill     long prefill at the 397B shape: one delta-net and one GQA layer over a 32768-token prompt,
              head-sharded over the ranks, head outputs all-gathered slab by slab while the next slab computes
  strong      the 64 sequences of the headline workload split over the N GPUs (N > 1)
  decode_397b 8-GPU-style head-sharded decode at the 397B shape: 256 sequences at an 8192-token context,
              per-layer times with and without the all-gather (N > 1)
  single_layer  one delta-net layer (prefill 512 + 128 decode steps) and one GQA layer (prefill 4096 + 256
              decode steps, f32 and Q8_0 caches), f32 activations, batch 1, with the CPU reference beside them (N = 1)
  projections   the nine integer-path projections (Q8_0 / Q6_K weights x Q8_K activations) of one delta-net and one GQA
              layer for the 64 tokens of a step, and one prompt-sized product (N = 1)

The timed headline loop replays the step (81 launches) as one CUDA graph (--no-graph: a loop of launches).

    python bench.py --gpus 1 --steps 20 --warmup 5
    torchrun ... bench.py --gpus N ...
    python bench.py --impl reference     # the CPU path on the host cores

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes (read + write) per launch over algorithmic bytes, from the ncu captures summarised in
# profiles/gqa_decode_q8_raw_24seq_8k-16k.txt (308.5 MB moved for 303.8 MB) and
# profiles/linear_decode_ring_64seq.txt, profiles/linear_decode_128_64seq.txt (the state a launch writes is partly still dirty in L2 when
# it ends, so DRAM writes are undercounted there; 1.0 = the algorithmic bytes are what moves).
DRAM_OVER_ALGORITHMIC = {"full_attn_step": 1.015, "linear_attn_step": 1.0}

METRIC = "attn_stack_decode_tokens_per_s"
UNIT = "tok/s"


def draw_contexts(n, lo, hi, seed):
    return np.random.default_rng(seed).integers(lo, hi + 1, n).astype(np.int64)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a cuBLAS GEMM on this pool: (burst, sustained, source)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


def _timed(fn, dev, world, reps):
    """Device time of fn() in ms: the median of `reps` separately timed calls after one warm-up call (a one-off stall
    of a collective or an allocation does not end up in the figure), max over ranks."""
    import torch
    import torch.distributed as dist
    fn()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    ev[0].record()
    for i in range(reps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([float(np.median([ev[i].elapsed_time(ev[i + 1]) for i in range(reps)]))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


class SlabGather:
    """All-gather of head outputs that overlaps the layer: the prompt is processed in slabs of tokens, and the
    gather of slab k (NCCL, on its own stream) runs while slab k+1 is computed.  Only the last slab's gather is
    exposed.  Nothing but plain NCCL touches another GPU's memory."""

    def __init__(self, dev, world):
        import torch
        self.dev, self.world = dev, world
        self.comm = torch.cuda.Stream(dev) if world > 1 else None
        self.bufs = {}

    def run(self, layer_fn, T, slab, width, dtype):
        """layer_fn(t0, n) -> [1, n, width] output of tokens t0..t0+n; returns the gathered blocks, one [world][1][n][width] per slab."""
        import torch
        import torch.distributed as dist
        if self.world == 1:
            for t0 in range(0, T, slab):
                layer_fn(t0, min(slab, T - t0))
            return None
        key = (T, slab, width, dtype)
        if key not in self.bufs:                        # one gathered block [world][1][n][width] per slab (slab-major, no re-layout copy)
            self.bufs[key] = [torch.empty((self.world, 1, min(slab, T - t0), width), dtype=dtype, device=self.dev)
                              for t0 in range(0, T, slab)]
        out = self.bufs[key]
        main = torch.cuda.current_stream(self.dev)
        for k, t0 in enumerate(range(0, T, slab)):
            n = min(slab, T - t0)
            o = layer_fn(t0, n).contiguous()
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self.comm):
                self.comm.wait_event(ev)
                dist.all_gather_into_tensor(out[k], o)
                o.record_stream(self.comm)
        main.wait_stream(self.comm)
        return out


def run_prefill(dev, rank, world, T=32768, reps=3, shape="397b", slab=8192, shard_of=1):
    """Long prefill: one 397B-shaped delta-net layer and one GQA layer over a T-token prompt, batch 1, bf16
    activations, head-sharded over the ranks (64/G value heads; 32/G query heads with the KV heads they read),
    head outputs all-gathered.  Returns per-layer times (max over ranks) and the figures derived from them;
    the stack has 45 delta-net and 15 GQA layers.  shape="35b" (32 value heads, 16 query heads) and a smaller T
    give the small cases the profiles are taken on; shard_of=W on one rank runs the shard one rank of W would own
    (no gather), which is how a shard's kernels are profiled on one GPU."""
    import torch
    from ornithology_b200 import device as D
    from ornithology_b200 import stack as S

    g = torch.Generator(device="cpu").manual_seed(2)
    NV, NH = (64, 32) if shape == "397b" else (32, 16)
    sw = world if world > 1 else max(1, shard_of)       # how many ways the heads are split
    NV_run, NH_run = (NV, NH) if world > 1 else (NV // sw, NH // sw)
    nv, nk = NV // sw, min(16, NV // sw)
    nh, nkv = NH // sw, max(1, 2 // sw)
    a = S.ARCHS[shape]
    w = S.linear_weights(dict(a, nk=nk, nv=nv), 0, 0)
    lin = D.LinearLayer(nk, nv, 128, 128, w["conv_w"], w["a_coef"], w["dt_bias"], w["norm_w"], device=dev)
    lst = D.LinearState(lin, 1)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    lin_in = [torch.randn(1, T, n, generator=g).to(torch.bfloat16).to(dev) for n in (lin.cc, nv, nv, lin.vd)]
    fw = S.full_weights(a, 0, 3)
    full = D.FullLayer(nh, nkv, 256, fw["q_norm_w"], fw["k_norm_w"], device=dev)
    kv = D.KvBatch(D.KV_Q8_0, nkv, 256, [T], device=dev)
    full_in = [torch.randn(1, T, n, generator=g).to(torch.bfloat16).to(dev) for n in (nh * 512, nkv * 256, nkv * 256)]
    gather = SlabGather(dev, world)

    def lin_whole():
        pos.zero_()
        return D.linear_attn_prefill(lin, lst, pos, *lin_in, T, chunk=64)

    def full_whole():
        pos.zero_()
        return D.full_attn_prefill(full, kv, pos, *full_in, T)

    def lin_slab(t0, n):
        pos.fill_(t0)                                   # conv ring phase = index of the first token of the slab
        return D.linear_attn_prefill(lin, lst, pos, *[x[:, t0:t0 + n] for x in lin_in], n, chunk=64)

    def full_slab(t0, n):
        pos.fill_(t0)                                   # rows already in the cache
        return D.full_attn_prefill(full, kv, pos, *[x[:, t0:t0 + n] for x in full_in], n, max_len=T)

    # one rank: the layer in one call; several ranks: slabs of tokens, gather of slab k under the compute of slab k+1
    if world == 1:
        ms_lin = ms_lin_k = _timed(lin_whole, dev, world, reps)
        ms_full = ms_full_k = _timed(full_whole, dev, world, reps)
    else:
        ms_lin = _timed(lambda: gather.run(lin_slab, T, slab, lin.vd, torch.bfloat16), dev, world, reps)
        ms_full = _timed(lambda: gather.run(full_slab, T, slab, nh * 256, torch.bfloat16), dev, world, reps)
        ms_lin_k = _timed(lin_whole, dev, world, reps)
        ms_full_k = _timed(full_whole, dev, world, reps)
    # algorithmic work of the whole layer (all ranks): causal QK^T + PV; chunked scan of 64-token chunks
    fl_full = 4.0 * 256 * NH_run * T * (T + 1) / 2
    fl_lin = float(NV_run) * (T / 64) * (6 * 64 * 128 * 128 + 2 * 64 * 64 * 256)
    burst, sustained, src = measured_tensor_peak()
    stack_ms = 45 * ms_lin + 15 * ms_full
    from ornithology_b200 import _lib
    torch.cuda.synchronize(dev)
    wait_status = int(_lib.load().ornith_cuda_poll_status())       # non-zero: a bounded wait inside a kernel gave up
    tf_full = fl_full / (ms_full_k * 1e-3) / 1e12
    tf_lin = fl_lin / (ms_lin_k * 1e-3) / 1e12
    sustained_leg = None
    if world == 1 and rank == 0:
        # the GQA layer back to back for about a second, clocks sampled: the figure to set against the sustained
        # (power-capped) tensor peak, which is how a long prompt's 15 such layers actually run
        n = max(3, min(200, int(1000.0 / max(ms_full_k, 0.05))))
        sampler = ClockSampler(dev.index if dev.index is not None else 0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            full_whole()
        e1.record()
        torch.cuda.synchronize(dev)
        clk = sampler.stop()
        ms_sus = e0.elapsed_time(e1) / n
        tf_sus = fl_full / (ms_sus * 1e-3) / 1e12
        sustained_leg = {"calls": n, "ms": ms_sus, "tflops": tf_sus, "peak": sustained, "frac": tf_sus / sustained,
                         "peak_source": f"of {src} (bf16 sustained)", "clocks": clk}
    return {"workload": "%d-token prompt, %s-shaped layers, batch 1, bf16, head-sharded x%d%s"
                        % (T, shape.upper(), sw, "" if world > 1 or sw == 1 else " (one shard timed on one GPU, no gather)"),
            "tokens": T, "delta_net_ms_per_layer": ms_lin, "gqa_ms_per_layer": ms_full, "wait_status_rank0": wait_status,
            "delta_net_ms_no_gather": ms_lin_k, "gqa_ms_no_gather": ms_full_k,
            "gather": "none" if world == 1 else f"NCCL all-gather per {slab}-token slab on a second stream, under the next slab's compute",
            "stack_layers": "45 delta-net + 15 GQA", "stack_ms": stack_ms, "stack_tok_per_s": T / (stack_ms * 1e-3),
            "gqa_tflops": tf_full, "delta_net_tflops": tf_lin,
            "roofline": {"bound": "tensor", "kernel": "k_gqa_prefill_tc", "achieved": tf_full, "peak": burst * world,
                         "unit": "TFLOP/s", "frac": tf_full / (burst * world), "peak_source": f"of {src} (bf16 burst)",
                         "flop_per_layer": fl_full, "ms": ms_full_k},
            "roofline_delta_net": {"bound": "tensor", "kernel": "k_delta_scan_tc5 (+ conv and chunk preparation)",
                                   "achieved": tf_lin, "peak": burst * world, "unit": "TFLOP/s",
                                   "frac": tf_lin / (burst * world), "flop_per_layer": fl_lin, "ms": ms_lin_k,
                                   "note": "tf32 products run at half the bf16 rate; a sequential scan: chunks x chain latency bound it, not the pipe"},
            "gqa_sustained": sustained_leg,
            "tensor_peak_tflops": burst * world, "tensor_peak_sustained_tflops": sustained * world,
            "gqa_frac_of_tensor_peak": tf_full / (burst * world), "peak_source": f"of {src}"}


def run_decode_397b(dev, rank, world, n_seq=256, ctx=8192, steps=10, warmup=3):
    """Head-sharded batched decode at the 397B shape: n_seq sequences at a ctx-token context, Q8_0 KV, fp32 state,
    bf16 activations; a rank owns 64/G value heads of the delta-net layers (with the key heads they pair with) and
    32/G query heads of the full layers with the KV head they read (replicated beyond 2 ranks); every layer's head
    outputs are all-gathered.  One delta-net layer and one GQA layer are timed (all sequences, `steps` consecutive
    steps each); the stack has 45 + 15 of them."""
    import torch
    import torch.distributed as dist
    from ornithology_b200 import device as D
    from ornithology_b200 import stack as S
    a = S.ARCHS["397b"]
    sh = S.head_shard(a, rank, world)
    nv, nk, nh, nkv = len(sh.v_heads), len(sh.k_heads), len(sh.q_heads), len(sh.kv_heads)
    w, _ = S.shard_linear_weights(a, S.linear_weights(a, 4, 0), sh)
    lin = D.LinearLayer(nk, nv, 128, 128, w["conv_w"], w["a_coef"], w["dt_bias"], w["norm_w"], device=dev)
    fw = S.full_weights(a, 4, 3)
    full = D.FullLayer(nh, nkv, 256, fw["q_norm_w"], fw["k_norm_w"], device=dev)
    total = warmup + steps + 2
    kv = D.KvBatch(D.KV_Q8_0, nkv, 256, [ctx + 2 * total] * n_seq, device=dev)     # room for one pass of steps and the warm-up
    st = D.LinearState(lin, n_seq, device=dev)
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    bf = torch.bfloat16
    # state: a short seeded prompt through the prefill; cache: seeded N(0,1) rows through the append kernel
    z0 = torch.zeros(n_seq, dtype=torch.int32, device=dev)
    pre = [torch.randn(n_seq, 64, n, generator=g, device=dev).to(bf) for n in (lin.cc, nv, nv, lin.vd)]
    D.linear_attn_prefill(lin, st, z0, *pre, 64, chunk=64)
    del pre
    done = torch.zeros(n_seq, dtype=torch.int32, device=dev)
    for t0 in range(0, ctx, 1024):
        n = min(1024, ctx - t0)
        k = torch.randn(n_seq, n, nkv * 256, generator=g, device=dev).to(bf)
        v = torch.randn(n_seq, n, nkv * 256, generator=g, device=dev).to(bf)
        D.kv_append(full, kv, done, k, v, T=n)
        done += n
    pos = torch.full((n_seq,), ctx, dtype=torch.int32, device=dev)
    lin_in = [torch.randn(n_seq, n, generator=g, device=dev).to(bf) for n in (lin.cc, nv, nv, lin.vd)]
    full_in = [torch.randn(n_seq, n, generator=g, device=dev).to(bf) for n in (nh * 512, nkv * 256, nkv * 256)]
    lin_out = torch.empty(n_seq, lin.vd, dtype=bf, device=dev)
    full_out = torch.empty(n_seq, nh * 256, dtype=bf, device=dev)
    g_lin = torch.empty(world, n_seq, lin.vd, dtype=bf, device=dev)
    g_full = torch.empty(world, n_seq, nh * 256, dtype=bf, device=dev)
    max_len = ctx + 2 * total

    def lin_step(gather):
        D.linear_attn_step(lin, st, pos, *lin_in, out=lin_out)
        if gather and world > 1:
            dist.all_gather_into_tensor(g_lin, lin_out)

    def full_step(gather):
        D.full_attn_step(full, kv, pos, *full_in, out=full_out, max_len=max_len)
        D.advance(pos)
        if gather and world > 1:
            dist.all_gather_into_tensor(g_full, full_out)

    def loop(fn, gather):
        def run():
            pos.fill_(ctx)                              # every pass runs the same `steps` positions (appended rows are overwritten)
            for _ in range(steps):
                fn(gather)
        return _timed(run, dev, world, 1) / steps

    for _ in range(warmup):
        lin_step(True); full_step(True)
    pos.fill_(ctx)
    ms_lin, ms_full = loop(lin_step, True), loop(full_step, True)
    ms_lin_k, ms_full_k = loop(lin_step, False), loop(full_step, False)
    cc = lin.cc
    b_lin = n_seq * (2 * nv * 128 * 128 * 4 + 4 * cc * 4 + cc * 2 + 2 * nv * 2 + 2 * lin.vd * 2)
    b_full = n_seq * (2 * nkv * 272 * (ctx + total) + 2 * nkv * 272 + nh * 256 * 3 * 2 + 2 * nkv * 256 * 2)
    peak, src = measured_peaks()
    stack_ms = 45 * ms_lin + 15 * ms_full
    return {"workload": "397B-shaped head-sharded decode x%d: %d sequences at a %d-token context, Q8_0 KV, fp32 state, bf16" % (world, n_seq, ctx),
            "per_rank_heads": {"value": nv, "key": nk, "query": nh, "kv": nkv},
            "steps_timed": steps, "delta_net_ms_per_layer": ms_lin, "gqa_ms_per_layer": ms_full,
            "delta_net_ms_no_gather": ms_lin_k, "gqa_ms_no_gather": ms_full_k,
            "gather_bytes_per_layer": {"delta_net": n_seq * lin.vd * 2 * world, "gqa": n_seq * nh * 256 * 2 * world},
            "stack_layers": "45 delta-net + 15 GQA", "stack_ms_per_step": stack_ms, "stack_tok_per_s": n_seq / (stack_ms * 1e-3),
            "delta_net": {"bytes_per_rank": b_lin, "gbs": b_lin / (ms_lin_k * 1e-3) / 1e9, "frac": b_lin / (ms_lin_k * 1e-3) / 1e9 / peak},
            "gqa": {"bytes_per_rank": b_full, "gbs": b_full / (ms_full_k * 1e-3) / 1e9, "frac": b_full / (ms_full_k * 1e-3) / 1e9 / peak},
            "peak_gbs": peak, "peak_source": f"of {src}",
            "note": "KV heads are replicated beyond 2 ranks, so the GQA bytes per rank stop shrinking at 2 ranks"}


def run_single_layer(dev, cpu=True):
    """The two single-layer workloads, batch 1, f32 activations: a 35B-shaped delta-net layer (prefill 512 tokens,
    then 128 decode steps, seed 0) and a 35B-shaped GQA layer (prefill 4096 tokens, then 256 decode steps, with an f32
    and with a Q8_0 cache, seed 1).  Batch-1 decode is launch-bound on a GPU: one or two kernels of a few
    microseconds per step.  The CPU reference is timed beside them on bounded samples (see `cpu`)."""
    import torch
    from ornithology_b200 import device as D
    from ornithology_b200 import stack as S
    a = S.ARCHS["35b"]
    res = {}
    f32 = torch.float32
    # ---- delta-net layer
    w = S.linear_weights(a, 0, 0)
    lin = D.LinearLayer(a["nk"], a["nv"], 128, 128, w["conv_w"], w["a_coef"], w["dt_bias"], w["norm_w"], device=dev)
    g = torch.Generator(device="cpu").manual_seed(0)
    T, steps = 512, 128
    ins = [torch.randn(1, T + steps, n, generator=g).to(dev) for n in (lin.cc, a["nv"], a["nv"], lin.vd)]
    st = D.LinearState(lin, 1)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)

    def lin_prefill():
        pos.zero_()
        return D.linear_attn_prefill(lin, st, pos, *[x[:, :T] for x in ins], T, chunk=64)

    def lin_decode():
        pos.fill_(T)
        for t in range(T, T + steps):
            D.linear_attn_step(lin, st, pos, *[x[:, t] for x in ins])
            D.advance(pos)

    res["delta_net"] = {"prefill_tokens": T, "decode_steps": steps, "prefill_ms": _timed(lin_prefill, dev, 1, 3),
                        "decode_ms_per_step": _timed(lin_decode, dev, 1, 2) / steps}
    res["delta_net"]["prefill_tok_per_s"] = T / (res["delta_net"]["prefill_ms"] * 1e-3)
    res["delta_net"]["decode_tok_per_s"] = 1e3 / res["delta_net"]["decode_ms_per_step"]
    # ---- GQA layer, both caches
    fw = S.full_weights(a, 1, 3)
    full = D.FullLayer(a["nh"], a["nkv"], 256, fw["q_norm_w"], fw["k_norm_w"], device=dev)
    g = torch.Generator(device="cpu").manual_seed(1)
    T, steps = 4096, 256
    fin = [torch.randn(1, T + steps, n, generator=g).to(dev) for n in (a["nh"] * 512, a["nkv"] * 256, a["nkv"] * 256)]
    for name, mode in (("gqa_f32_kv", D.KV_F32), ("gqa_q8_0_kv", D.KV_Q8_0)):
        kv = D.KvBatch(mode, a["nkv"], 256, [T + steps], device=dev)
        kv_len = torch.zeros(1, dtype=torch.int32, device=dev)

        def full_prefill():
            kv_len.zero_()
            return D.full_attn_prefill(full, kv, kv_len, *[x[:, :T] for x in fin], T)

        def full_decode():
            kv_len.fill_(T)
            for t in range(T, T + steps):
                D.full_attn_step(full, kv, kv_len, *[x[:, t] for x in fin], max_len=T + steps)
                D.advance(kv_len)

        r = {"prefill_tokens": T, "decode_steps": steps, "prefill_ms": _timed(full_prefill, dev, 1, 3),
             "decode_ms_per_step": _timed(full_decode, dev, 1, 2) / steps}
        r["prefill_tok_per_s"] = T / (r["prefill_ms"] * 1e-3)
        r["decode_tok_per_s"] = 1e3 / r["decode_ms_per_step"]
        r["prefill_tflops"] = 4.0 * 256 * a["nh"] * T * (T + 1) / 2 / (r["prefill_ms"] * 1e-3) / 1e12
        res[name] = r
    res["note"] = "batch 1: decode is launch-bound (one or two kernels of a few microseconds per step), not a bandwidth case"
    if cpu:
        res["cpu"] = cpu_single_layer()
    return res


def run_projections(dev, n_tok=64, cpu=True):
    """The quantised projections that bracket the attention kernels of one 35B-shaped delta-net layer and one
    full-attention layer (hidden 2048), through the engine's integer path (Q8_K activations; Q8_0 weights around the
    delta-net core, Q6_K around the full-attention core), 64 tokens (one decode step of the headline batch), bf16
    activations.  Projections that read the same input share one quantisation, as in the engine, and go as one grouped
    launch.  Each layer's
    sequence is timed over 16 distinct weight sets used in turn (larger than L2 together), as one CUDA graph; the
    roofline figure is the weight bytes (what a decode-sized batch has to stream) over the time.  Each projection is
    also timed alone against a ready image.  `prompt` is attn_qkv over 4096 tokens (tensor-core bound).  The CPU
    figure is the engine's integer path on one host thread over a sample of the output rows."""
    import torch
    from ornithology_b200 import device as D
    from oracle import oracle as O
    orc = O.Oracle()
    Q8, Q6 = D.GGML_Q8_0, D.GGML_Q6_K
    # (name, weight type, n_in, n_out, input): inputs "h" = the layer's normalised hidden state, "o" = the core's output
    layers = {"delta_net": [("attn_qkv", Q8, 2048, 8192, "h"), ("attn_gate", Q8, 2048, 4096, "h"), ("ssm_alpha", Q8, 2048, 32, "h"),
                            ("ssm_beta", Q8, 2048, 32, "h"), ("ssm_out", Q8, 4096, 2048, "o")],
              "full_attn": [("attn_q", Q6, 2048, 8192, "h"), ("attn_k", Q6, 2048, 512, "h"), ("attn_v", Q6, 2048, 512, "h"),
                            ("attn_output", Q6, 4096, 2048, "o")]}
    g = np.random.default_rng(8)
    peak, src = measured_peaks()
    copies = 16

    def rows(wt, n_out, n_in):                         # random block bytes with finite scales: the timing does not depend on the values
        rb = O.QROW_BYTES[wt](n_in)
        W = g.integers(0, 256, (n_out, rb), dtype=np.uint8)
        if wt == Q8:
            W.reshape(n_out, -1, 34)[:, :, 1] &= 0x3B
        else:
            W.reshape(n_out, -1, 210)[:, :, 209] &= 0x3B
        return W

    def graph_ms(fn):
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()                 # the launches of a pass replayed as one graph: the timing is
        with torch.cuda.graph(graph, stream=side):     # then the kernels', not the Python call overhead
            fn()
        return _timed(graph.replay, dev, 1, 3) / copies

    res, per, tot_bytes, tot_ms, launches = {}, {}, 0.0, 0.0, 0
    W_cpu = None
    for lname, projs in layers.items():
        xs = {"h": torch.from_numpy(g.standard_normal((n_tok, 2048)).astype(np.float32)).to(dev).to(torch.bfloat16),
              "o": torch.from_numpy(g.standard_normal((n_tok, 4096)).astype(np.float32)).to(dev).to(torch.bfloat16)}
        imgs = {k: D.q8k_image(v, v.shape[1]) for k, v in xs.items()}
        sets, outs, nbytes = [], {}, 0.0
        for c in range(copies):
            ws = {}
            for name, wt, n_in, n_out, _ in projs:
                W = rows(wt, n_out, n_in)
                if name == "attn_qkv" and c == 0:
                    W_cpu = W
                ws[name] = D.QWeight(wt, W, n_in, device=dev)
            sets.append(ws)
        for name, wt, n_in, n_out, _ in projs:
            outs[name] = torch.empty(n_tok, n_out, dtype=torch.bfloat16, device=dev)
            nbytes += float(n_out) * O.QROW_BYTES[wt](n_in)

        def layer_pass():
            for ws in sets:                            # per distinct input: one quantisation, one grouped launch of its projections
                for src_in in ("h", "o"):
                    names = [p[0] for p in projs if p[4] == src_in]
                    D.q8k_image(xs[src_in], xs[src_in].shape[1], image=imgs[src_in])
                    D.matmul_q_group([ws[nm] for nm in names], imgs[src_in], n_tok, outs=[outs[nm] for nm in names])
        ms = graph_ms(layer_pass)
        res[lname] = {"us": ms * 1e3, "weight_bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak,
                      "launches": 4}
        tot_bytes += nbytes; tot_ms += ms; launches += 4
        for name, wt, n_in, n_out, src_in in projs:
            def one():
                for ws in sets:
                    D.matmul_q(ws[name], None, out=outs[name], image=imgs[src_in], T=n_tok)
            m1 = graph_ms(one)
            b1 = float(n_out) * O.QROW_BYTES[wt](n_in)
            per[name] = {"type": {Q8: "q8_0", Q6: "q6_k"}[wt], "n_in": n_in, "n_out": n_out, "us": m1 * 1e3, "gbs": b1 / (m1 * 1e-3) / 1e9,
                         "frac": b1 / (m1 * 1e-3) / 1e9 / peak}
        del sets
    # a prompt-sized batch of the largest projection
    Tp = 4096
    wp = [D.QWeight(Q8, rows(Q8, 8192, 2048), 2048, device=dev) for _ in range(copies)]
    xp = torch.from_numpy(g.standard_normal((Tp, 2048)).astype(np.float32)).to(dev).to(torch.bfloat16)
    ip = D.q8k_image(xp, 2048)
    op = torch.empty(Tp, 8192, dtype=torch.bfloat16, device=dev)

    def prompt_pass():
        for w in wp:
            D.q8k_image(xp, 2048, image=ip)
            D.matmul_q(w, None, out=op, image=ip, T=Tp)
    mp = graph_ms(prompt_pass)
    prompt = {"shape": "attn_qkv 2048 -> 8192, q8_0", "tokens": Tp, "us": mp * 1e3, "tops": 2.0 * Tp * 2048 * 8192 / (mp * 1e-3) / 1e12,
              "note": "int8 mma.sync with int32 sums (exact); integer multiply-adds per sub-block scale share the issue slots"}
    out = {"workload": f"integer-path projections of one delta-net layer (Q8_0) and one full-attention layer (Q6_K), {n_tok} tokens, bf16",
           "per_layer": res, "per_projection": per, "prompt": prompt, "total_us": tot_ms * 1e3, "total_weight_bytes": tot_bytes,
           "launches": launches,
           "roofline": {"bound": "hbm", "kernel": "k_matmul_kq", "achieved": tot_bytes / (tot_ms * 1e-3) / 1e9, "peak": peak,
                        "unit": "GB/s", "frac": tot_bytes / (tot_ms * 1e-3) / 1e9 / peak, "peak_source": f"of {src}"},
           "note": "a decode-sized batch: each projection is a few microseconds of weight traffic, so launch latency is a "
                   "large part of the small ones; results are the engine's bit for bit"}
    if cpu:
        sample = 256
        x = xs["h"].float().cpu().numpy()
        t0 = time.perf_counter()
        orc.matmul_q(Q8, W_cpu[:sample], 2048, x)
        dt = time.perf_counter() - t0
        out["cpu"] = {"kind": "port", "cores": 1, "shape": "attn_qkv", "ms": dt * 1e3 * 8192 / sample,
                      "sample": f"{sample} of the 8192 output rows, {n_tok} tokens, scaled by rows"}
    return out


def cpu_single_layer():
    """The CPU reference on the two single-layer workloads (one thread: the attention core is single-threaded in the
    engine).  The delta-net layer runs in full; of the GQA layer the decode steps run in full (64 of them, at the
    4096-token context) and the O(T^2) prefill is timed on its first 1024 tokens and scaled by the number of
    (query, key) pairs."""
    from oracle import oracle as O
    from ornithology_b200.stack import ARCHS, full_weights, linear_weights
    a = ARCHS["35b"]
    orc = O.Oracle()
    ref = O.Ref() if O.Ref.available() else None
    g = np.random.default_rng(0)
    w = linear_weights(a, 0, 0)
    lin = O.LinearLayer(a["nk"], a["nv"], a["dk"], a["dv"], w["conv_w"], w["a_coef"], w["dt_bias"], w["norm_w"])
    T, steps = 512, 128
    ins = [g.standard_normal((T + steps, n)).astype(np.float32) for n in (lin.cc, a["nv"], a["nv"], lin.vd)]
    S = np.zeros((a["nv"], 128, 128), np.float32); buf = np.zeros(3 * lin.cc + 1, np.float32)
    t0 = time.perf_counter()
    orc.linear_attn_prefill(lin, S, buf[:3 * lin.cc], *[x[:T] for x in ins], chunk=64)
    t1 = time.perf_counter()
    for t in range(T, T + steps):
        if ref is not None:
            O.ref_linear_step(ref, lin, S, buf, *[x[t] for x in ins])
        else:
            orc.linear_attn_step(lin, S, buf[:3 * lin.cc], *[x[t] for x in ins])
    t2 = time.perf_counter()
    out = {"kind": "reference" if ref is not None else "port", "cores": 1,
           "delta_net": {"prefill_ms": (t1 - t0) * 1e3, "prefill_tok_per_s": T / (t1 - t0),
                         "decode_ms_per_step": (t2 - t1) * 1e3 / steps, "decode_tok_per_s": steps / (t2 - t1),
                         "sample": "in full (prefill through the restated chunked scan, decode steps through the engine's own objects)"}}
    fw = full_weights(a, 1, 3)
    full = O.FullLayer(a["nh"], a["nkv"], a["hd"], fw["q_norm_w"], fw["k_norm_w"], rope_dim=a["rope_dim"], theta=a["theta"])
    T, Ts, dsteps = 4096, 1024, 64
    fin = [g.standard_normal((T + dsteps, n)).astype(np.float32) for n in (a["nh"] * 512, a["nkv"] * 256, a["nkv"] * 256)]
    okv = orc.kv(T + dsteps, a["nkv"], a["hd"], O.KV_F32)
    t0 = time.perf_counter()
    orc.full_attn_prefill(full, okv, 0, *[x[:Ts] for x in fin])
    t1 = time.perf_counter()
    import ctypes as C
    rows = g.standard_normal((T, a["nkv"] * a["hd"])).astype(np.float32)      # stand-in rows up to the 4096-token context
    C.memmove(okv.c.K, rows.ctypes.data, rows.nbytes); C.memmove(okv.c.V, rows.ctypes.data, rows.nbytes)
    okv.c.len = T
    t2 = time.perf_counter()
    for t in range(T, T + dsteps):
        orc.full_attn_step(full, okv, t, *[x[t] for x in fin])
    t3 = time.perf_counter()
    scale = (T * (T + 1) / 2) / (Ts * (Ts + 1) / 2)
    out["gqa_f32_kv"] = {"prefill_ms": (t1 - t0) * 1e3 * scale, "prefill_tok_per_s": T / ((t1 - t0) * scale),
                         "decode_ms_per_step": (t3 - t2) * 1e3 / dsteps, "decode_tok_per_s": dsteps / (t3 - t2),
                         "sample": f"prefill: first {Ts} tokens timed ({(t1 - t0):.1f} s), scaled x{scale:.1f} by (query, key) pairs; "
                                   f"decode: {dsteps} steps at the {T}-token context"}
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while active."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()                  # the exact process started above
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# CPU path (the checker libraries, timed): a bounded sample of the same workload
# ---------------------------------------------------------------------------------------
def cpu_sample(contexts, n_seq_sample, seed, threads, passes=3):
    """Time `passes` interleave groups of one decode token for `n_seq_sample` sequences
    (3 delta-net layers + 1 GQA layer) on the host, and scale to the 40-layer stack.
    Uses the reference's own compiled objects when they were built, else the port."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as O
    from ornithology_b200.stack import ARCHS, full_weights, linear_weights
    a = ARCHS["35b"]
    orc = O.Oracle()
    ref = O.Ref() if O.Ref.available() else None
    kind = "reference" if ref is not None else "port"
    lin_layers = []
    for i in range(3):
        w = linear_weights(a, seed, i)
        lin_layers.append(O.LinearLayer(a["nk"], a["nv"], a["dk"], a["dv"], w["conv_w"], w["a_coef"], w["dt_bias"], w["norm_w"]))
    fw = full_weights(a, seed, 3)
    full = O.FullLayer(a["nh"], a["nkv"], a["hd"], fw["q_norm_w"], fw["k_norm_w"], rope_dim=a["rope_dim"], theta=a["theta"])
    ctx = [int(c) for c in contexts[:n_seq_sample]]
    g = np.random.default_rng(seed + 1)
    seqs = []
    import ctypes as C
    pool = g.standard_normal((max(ctx) + 64, a["nkv"] * a["hd"]), dtype=np.float32)   # stand-in for decoded rows
    for n, L in enumerate(ctx):                  # state set-up is not timed
        Kd = pool[n % 32:n % 32 + L]
        Vd = pool[32 + n % 32:32 + n % 32 + L]
        if ref is not None:                      # the reference's own f32 cache (src/ornith_attn.h:57-69)
            kv = ref.kv_init(L + 1, a["nkv"], a["hd"], 0)
            C.memmove(kv.K, Kd.ctypes.data, Kd.nbytes); C.memmove(kv.V, Vd.ctypes.data, Vd.nbytes)
            kv.len = L
        else:
            kv = orc.kv(L + 1, a["nkv"], a["hd"], O.KV_Q8_0)
            C.memmove(kv.c.K, Kd.ctypes.data, Kd.nbytes); C.memmove(kv.c.V, Vd.ctypes.data, Vd.nbytes)
            kv.c.len = L
        S = [(g.standard_normal((a["nv"], a["dv"], a["dk"])) * 0.05).astype(np.float32) for _ in range(3)]
        buf = [g.standard_normal(3 * lin_layers[0].cc + 1).astype(np.float32) for _ in range(3)]
        ins_l = [[g.standard_normal(w).astype(np.float32) for w in (lin_layers[0].cc, a["nv"], a["nv"], lin_layers[0].vd)] for _ in range(3)]
        ins_f = [g.standard_normal(w).astype(np.float32) for w in (a["nh"] * 2 * a["hd"], a["nkv"] * a["hd"], a["nkv"] * a["hd"])]
        seqs.append((kv, L, S, buf, ins_l, ins_f))

    def one(s):
        kv, L, S, buf, ins_l, ins_f = s
        if ref is not None:                      # the reference's own functions, Q8_0 rows via its codec
            for i in range(3):
                O.ref_linear_step(ref, lin_layers[i], S[i], buf[i], *ins_l[i])
            kv.len = L                           # every pass appends at the same position
            O.ref_full_step(ref, full, kv, L, *ins_f, q8_0=True)
        else:
            for i in range(3):
                orc.linear_attn_step(lin_layers[i], S[i], buf[i], *ins_l[i])
            kv.c.len = L
            orc.full_attn_step(full, kv, L, *ins_f)

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _ in range(passes):
            list(ex.map(one, seqs))
    dt = time.perf_counter() - t0
    groups = a["layers"] // a["interval"]
    tok_s = len(seqs) * passes / (dt * groups)   # sequence-tokens per second through all 40 layers
    sample = (f"{passes} of the {groups} 3+1 layer groups of one decode step, {len(seqs)} sequences "
              f"(contexts sum {sum(ctx)}), scaled x{groups}/{passes}; {threads} threads, one sequence per thread; "
              f"{dt:.2f} s wall = {dt * threads:.0f} s of CPU work")
    return tok_s, kind, sample, dt


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = min(os.cpu_count() or 1, 32)
    contexts = draw_contexts(args.seqs, args.min_ctx, args.max_ctx, args.seed)
    n_sample = args.seqs
    vals, sample, kind = [], "", "port"
    for it in range(args.warmup + args.steps):
        v, kind, sample, _ = cpu_sample(contexts, n_sample, args.seed, threads)
        if it >= args.warmup:
            vals.append(v)
        if it >= 1 and args.steps > 2:            # bounded: the CPU path is slow by construction
            break
    value = float(np.mean(vals)) if vals else v
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "steps_timed": len(vals),
            "step": "each timed step is a bounded sample of one decode step (see cpu_baseline.sample), scaled to the full stack",
            "ms_per_step": 1e3 * args.seqs / value,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, contexts, 1),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(args, contexts, world):
    return {"workload": "batched decode, 40-layer 35B-shaped attention stack (30 delta-net + 10 GQA)",
            "sequences_per_gpu": args.seqs, "context": f"uniform[{args.min_ctx},{args.max_ctx}] seed {args.seed}",
            "sum_context_rank0": int(np.sum(contexts[:args.seqs])), "kv_cache": "Q8_0", "state": "fp32",
            "activations": "bf16", "parallelism": f"sequence-sharded x{world}, sequences dealt by summed context",
            "l2": "inputs larger than L2 (every step streams all KV rows and all recurrent state)"}


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from ornithology_b200 import device as D
    from ornithology_b200.stack import AttnStack

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ornithology_b200.stack import sequence_shard
    all_ctx = draw_contexts(args.seqs * world, args.min_ctx, args.max_ctx, args.seed)
    # one draw for the whole job, dealt so that every rank gets the same count and the summed contexts balance
    contexts = all_ctx[sequence_shard(all_ctx, rank, world)]
    total_steps = 2 * (args.warmup + args.steps) + 14
    caps = [int(c) + total_steps + 8 for c in contexts]
    stack = AttnStack("35b", caps, kv_mode=D.KV_Q8_0, seed=args.seed, device=dev)
    stack.fill(contexts, seed=args.seed + 17)
    max_len = int(max(caps))

    ins = stack.random_inputs(args.seed + 5, dtype=torch.bfloat16, device=dev)
    outs = [torch.empty(stack.n_seq, stack.output_width(k), dtype=torch.bfloat16, device=dev) for k, _, _ in stack.layers]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- value: inputs resident in HBM --------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()                   # runs from the warm-up to the end of the host-fed timed region
    # The step is a fixed sequence of 81 launches on device-resident arguments (positions live on the device), so it
    # is captured once into a CUDA graph and replayed: launch gaps between the kernels go.  Warm-up runs on the
    # capture stream first (the library keeps its delta-net work buffer per stream and must not allocate under
    # capture).  --no-graph times the plain launch loop instead.
    n_layers = len(stack.layers)
    graph = None
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(args.warmup):
            stack.decode_step(ins, outs, max_len=max_len)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                stack.decode_step(ins, outs, max_len=max_len)
            graph.replay()                # one untimed replay
        except Exception as e:            # noqa: BLE001 - any capture problem: time the launch loop, say so
            sys.stderr.write(f"bench: CUDA graph capture failed ({e}); timing the launch loop\n")
            graph = None
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for s in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            stack.decode_step(ins, outs, max_len=max_len)
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    # per-family times: a separate pass with an event between the layers (events between the launches cost the
    # overlap of a kernel's prologue with its predecessor's tail, so they stay out of the timed region above)
    fam_steps = max(3, min(args.steps, 5))
    stack.decode_step(ins, outs, max_len=max_len)      # untimed: this stream's first step sets up its own work buffer
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n_layers + 1)] for _ in range(fam_steps)]
    for s in range(fam_steps):
        for i, (kind, layer, state) in enumerate(stack.layers):
            ev[s][i].record()
            if kind == "full":
                D.full_attn_step(layer, state, stack.pos, *ins[i], out=outs[i], max_len=max_len)
            else:
                D.linear_attn_step(layer, state, stack.pos, *ins[i], out=outs[i])
        ev[s][n_layers].record()
        D.advance(stack.pos)
    torch.cuda.synchronize(dev)
    ms_lin = np.mean([ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(fam_steps)
                      for i, (k, _, _) in enumerate(stack.layers) if k == "linear"])
    ms_full = np.mean([ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(fam_steps)
                       for i, (k, _, _) in enumerate(stack.layers) if k == "full"])

    # ---- e2e: host buffers, copies inside the timed region -------------------------------
    h_ins = stack.random_inputs(args.seed + 5, dtype=torch.bfloat16, pin=True)
    h_outs = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
    h2d = sum(t.numel() * t.element_size() for layer in h_ins for t in layer)
    d2h = sum(t.numel() * t.element_size() for t in h_outs)

    # Every step copies every layer's inputs up and every layer's output down.  The copies run on
    # their own streams and are ordered against the kernels with per-layer events, so a layer's
    # upload overlaps the layers before it and its download the layers after it.
    s_main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(n_layers)]
    ev_done = [torch.cuda.Event() for _ in range(n_layers)]
    ev_out = [torch.cuda.Event() for _ in range(n_layers)]
    for e in ev_done + ev_out:
        e.record(s_main)

    def e2e_step():
        for i, (kind, layer, state) in enumerate(stack.layers):
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[i])           # the previous step has finished reading ins[i]
                for dst, src in zip(ins[i], h_ins[i]):
                    dst.copy_(src, non_blocking=True)
                ev_in[i].record(s_in)
            s_main.wait_event(ev_in[i])
            s_main.wait_event(ev_out[i])              # the previous step's outs[i] has been downloaded
            if kind == "full":
                D.full_attn_step(layer, state, stack.pos, *ins[i], out=outs[i], max_len=max_len)
            else:
                D.linear_attn_step(layer, state, stack.pos, *ins[i], out=outs[i])
            ev_done[i].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[i])
                h_outs[i].copy_(outs[i], non_blocking=True)
                ev_out[i].record(s_out)
        D.advance(stack.pos)

    def e2e_drain():
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    for _ in range(args.warmup):
        e2e_step()
    e2e_drain()
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        e2e_step()
    e2e_drain()                               # the last downloads are inside the timed region
    e_end.record()
    barrier()
    ms_e2e = e_start.elapsed_time(e_end)
    clocks = sampler.stop() if rank == 0 else None

    ctx_now = [int(c) + args.warmup + args.steps // 2 for c in contexts]      # contexts mid-way through the timed steps
    b_lin, b_full = stack.decode_bytes(ctx_now)
    # every rank's own figures: step time, per-family times, algorithmic bytes, summed context
    mine = torch.tensor([ms_total / args.steps, float(ms_lin), float(ms_full), float(b_lin), float(b_full),
                         float(np.sum(contexts))], dtype=torch.float64, device=dev)
    per_rank = [torch.zeros_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, mine)
    else:
        per_rank = [mine]
    per_rank = [[float(x) for x in t.cpu()] for t in per_rank]
    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = float(times[0]), float(times[1])
    launches = stack.launches_per_step()
    n_lin = sum(1 for k, _, _ in stack.layers if k == "linear")
    n_full = n_layers - n_lin

    # ---- strong scaling: the 64 sequences of the workload split over the ranks ------------
    strong = None
    if world > 1 and not args.no_extras:
        ctx64 = draw_contexts(args.seqs, args.min_ctx, args.max_ctx, args.seed)
        mine64 = ctx64[sequence_shard(ctx64, rank, world)]
        del stack, ins, outs, h_ins, h_outs
        torch.cuda.empty_cache()
        small = AttnStack("35b", [int(c) + 3 * args.steps + 16 for c in mine64], kv_mode=D.KV_Q8_0, seed=args.seed, device=dev)
        small.fill(mine64, seed=args.seed + 17)
        s_ins = small.random_inputs(args.seed + 5, dtype=torch.bfloat16, device=dev)
        s_max = int(max(mine64)) + 3 * args.steps + 16

        def s_loop():
            for _ in range(args.steps):
                small.decode_step(s_ins, max_len=s_max)
        ms = _timed(s_loop, dev, world, 1) / args.steps
        strong = {"workload": "the %d sequences of the headline workload split over %d GPUs (%d per GPU), balanced by summed context"
                              % (args.seqs, world, len(mine64)),
                  "ms_per_step": ms, "tok_per_s": args.seqs / (ms * 1e-3), "scaling": "strong",
                  "note": "few sequences per GPU: the delta-net layers run one CTA per (sequence, head) and the step is latency-bound"}
        del small, s_ins
        torch.cuda.empty_cache()

    prefill = None
    if not args.no_prefill:
        prefill = run_prefill(dev, rank, world)
    decode_397b = None
    if world > 1 and not args.no_extras:
        decode_397b = run_decode_397b(dev, rank, world)
    single = projections = None
    if world == 1 and not args.no_extras:
        single = run_single_layer(dev, cpu=not args.no_cpu)
        projections = run_projections(dev, cpu=not args.no_cpu)

    if rank == 0:
        tokens = args.seqs * world * args.steps
        value = tokens / (ms_total * 1e-3)
        e2e = tokens / (ms_e2e * 1e-3)
        peak, src = measured_peaks()
        slow = max(range(world), key=lambda r: per_rank[r][0])                    # the rank the step waits for
        _, r_lin, r_full, rb_lin, rb_full, _ = per_rank[slow]
        fam = {"linear_attn_step": {"ms_per_launch": r_lin, "bytes_per_launch": rb_lin / n_lin,
                                    "gbs": rb_lin / n_lin / (r_lin * 1e-3) / 1e9, "launches_per_step": n_lin},
               "full_attn_step": {"ms_per_launch": r_full, "bytes_per_launch": rb_full / n_full,
                                  "gbs": rb_full / n_full / (r_full * 1e-3) / 1e9, "launches_per_step": n_full}}
        dom = max(fam, key=lambda k: fam[k]["ms_per_launch"] * fam[k]["launches_per_step"])
        roof = {"bound": "hbm", "kernel": dom, "achieved": fam[dom]["gbs"], "peak": peak, "unit": "GB/s",
                "frac": fam[dom]["gbs"] / peak, "peak_source": f"of {src}",
                "traffic": fam[dom]["bytes_per_launch"] * DRAM_OVER_ALGORITHMIC[dom], "families": fam,
                "rank": slow, "timing": "per-family times from a separate pass with an event between the layers",
                "whole_step_gbs": (rb_lin + rb_full) / (per_rank[slow][0] * 1e-3) / 1e9}
        ranks = [{"rank": r, "sum_context": int(per_rank[r][5]), "ms_per_step": per_rank[r][0],
                  "step_gbs": (per_rank[r][3] + per_rank[r][4]) / (per_rank[r][0] * 1e-3) / 1e9} for r in range(world)]
        cpu = None
        if world == 1 and not args.no_cpu:
            threads = min(os.cpu_count() or 1, 32)
            v, kind, sample, _ = cpu_sample(all_ctx, args.seqs, args.seed, threads)
            cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": dict(workload_config(args, contexts, world),
                               launch="the step's launches replayed as one CUDA graph" if graph is not None
                               else "a loop of launches (no CUDA graph)"),
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / args.steps},
                "gpu_launches": launches * args.steps,
                "roofline": roof, "cpu_baseline": cpu, "clocks": clocks, "ranks": ranks, "prefill": prefill,
                "strong": strong, "decode_397b": decode_397b, "single_layer": single, "projections": projections}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=64, help="sequences per GPU")
    ap.add_argument("--min-ctx", type=int, default=1024)
    ap.add_argument("--max-ctx", type=int, default=32768)
    ap.add_argument("--seed", type=int, default=3)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="time the decode step as a loop of launches instead of a CUDA graph replay")
    ap.add_argument("--no-prefill", action="store_true", help="skip the long-prefill leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the strong-scaling, 397B-decode and single-layer legs")
    ap.add_argument("--prefill-only", action="store_true", help="run only the prefill leg (1 GPU) and print its figures")
    ap.add_argument("--prefill-reps", type=int, default=1, help="timed repetitions of each layer in --prefill-only (median reported)")
    ap.add_argument("--projections-only", action="store_true", help="run only the projections leg (1 GPU) and print its figures")
    ap.add_argument("--prefill-tokens", type=int, default=32768)
    ap.add_argument("--prefill-shape", default="397b", choices=["397b", "35b"])
    ap.add_argument("--prefill-shard-of", type=int, default=1, choices=[1, 2, 4, 8],
                    help="with --prefill-only: time the head shard one rank of this many would own")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.projections_only:
        import torch
        torch.cuda.set_device(local_rank)
        print(json.dumps(run_projections(torch.device("cuda", local_rank), cpu=not args.no_cpu)), flush=True)
        return
    if args.prefill_only:
        import torch
        torch.cuda.set_device(local_rank)
        print(json.dumps(run_prefill(torch.device("cuda", local_rank), 0, 1, T=args.prefill_tokens, reps=args.prefill_reps,
                                     shape=args.prefill_shape, shard_of=args.prefill_shard_of)), flush=True)
        return
    if world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
