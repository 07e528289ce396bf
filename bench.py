#!/usr/bin/env python
"""Attention-stack decode benchmark (BASELINE.json configs[2]).

One step = one token for each of 64 concurrent sequences through the 40-layer
35B-shaped attention stack (30 gated delta-net + 10 GQA layers, 3:1), Q8_0 KV
cache, fp32 recurrent state, bf16 activations, contexts uniform in [1k, 32k].
Multi-GPU runs shard by sequence: every rank owns 64 sequences of its own
(weak scaling, nothing is exchanged inside the stack).

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


def run_prefill(dev, rank, world, T=32768, reps=3, shape="397b"):
    """BASELINE.json configs[3]: one 397B-shaped delta-net layer and one GQA layer over a 32768-token
    prompt, batch 1, bf16 activations, head-sharded over the ranks (64/G value heads; 32/G query heads
    with the KV heads they read), head outputs all-gathered.  Returns per-layer times (max over ranks)
    and the figures derived from them; the stack has 45 delta-net and 15 GQA layers.  shape="35b"
    (32 value heads, 16 query heads) and a smaller T give the small cases the profiles are taken on."""
    import torch
    import torch.distributed as dist
    from ornithology_b200 import device as D
    from ornithology_b200 import stack as S

    g = torch.Generator(device="cpu").manual_seed(2)
    NV, NH = (64, 32) if shape == "397b" else (32, 16)
    nv, nk = NV // world, min(16, NV // world)
    nh, nkv = NH // world, max(1, 2 // world)
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

    def timed(fn):
        fn()
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def gather(o):
        if world == 1:
            return o
        full_o = torch.empty((world,) + tuple(o.shape), dtype=o.dtype, device=dev)
        dist.all_gather_into_tensor(full_o, o)
        return full_o

    ms_lin = timed(lambda: gather(D.linear_attn_prefill(lin, lst, pos, *lin_in, T, chunk=64)))
    ms_full = timed(lambda: gather(D.full_attn_prefill(full, kv, pos, *full_in, T)))
    # without the all-gather (the same call when there is one rank)
    ms_lin_k = ms_lin if world == 1 else timed(lambda: D.linear_attn_prefill(lin, lst, pos, *lin_in, T, chunk=64))
    ms_full_k = ms_full if world == 1 else timed(lambda: D.full_attn_prefill(full, kv, pos, *full_in, T))
    # algorithmic work of the whole layer (all ranks): causal QK^T + PV; chunked scan at C = 32
    fl_full = 4.0 * 256 * NH * T * (T + 1) / 2
    fl_lin = float(NV) * (T / 32) * (6 * 32 * 128 * 128 + 2 * 32 * 32 * 256)
    burst, sustained, src = measured_tensor_peak()
    stack_ms = 45 * ms_lin + 15 * ms_full
    return {"workload": "configs[3]: %d-token prompt, %s-shaped layers, batch 1, bf16, head-sharded x%d" % (T, shape.upper(), world),
            "tokens": T, "delta_net_ms_per_layer": ms_lin, "gqa_ms_per_layer": ms_full,
            "delta_net_ms_no_gather": ms_lin_k, "gqa_ms_no_gather": ms_full_k,
            "stack_layers": "45 delta-net + 15 GQA", "stack_ms": stack_ms, "stack_tok_per_s": T / (stack_ms * 1e-3),
            "gqa_tflops": fl_full / (ms_full_k * 1e-3) / 1e12 , "delta_net_tflops": fl_lin / (ms_lin_k * 1e-3) / 1e12,
            "tensor_peak_tflops": burst * world, "tensor_peak_sustained_tflops": sustained * world,
            "gqa_frac_of_tensor_peak": fl_full / (ms_full_k * 1e-3) / 1e12 / (burst * world), "peak_source": f"of {src}"}


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
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * args.seqs / value,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, contexts, 1),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(args, contexts, world):
    return {"workload": "configs[2]: batched decode, 40-layer 35B-shaped attention stack (30 delta-net + 10 GQA)",
            "sequences_per_gpu": args.seqs, "context": f"uniform[{args.min_ctx},{args.max_ctx}] seed {args.seed}",
            "sum_context_rank0": int(np.sum(contexts[:args.seqs])), "kv_cache": "Q8_0", "state": "fp32",
            "activations": "bf16", "parallelism": f"sequence-sharded x{world}",
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
    all_ctx = draw_contexts(args.seqs * world, args.min_ctx, args.max_ctx, args.seed)
    contexts = all_ctx[rank * args.seqs:(rank + 1) * args.seqs]
    total_steps = 2 * (args.warmup + args.steps) + 4
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
    for _ in range(args.warmup):
        stack.decode_step(ins, outs, max_len=max_len)
    n_layers = len(stack.layers)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n_layers + 1)] for _ in range(args.steps)]
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for s in range(args.steps):
        # same work as decode_step, with an event between layers (per-kernel-family timing)
        for i, (kind, layer, state) in enumerate(stack.layers):
            ev[s][i].record()
            if kind == "full":
                D.full_attn_step(layer, state, stack.pos, *ins[i], out=outs[i], max_len=max_len)
            else:
                D.linear_attn_step(layer, state, stack.pos, *ins[i], out=outs[i])
        ev[s][n_layers].record()
        D.advance(stack.pos)
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    ms_lin = np.mean([ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)
                      for i, (k, _, _) in enumerate(stack.layers) if k == "linear"])
    ms_full = np.mean([ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)
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

    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = float(times[0]), float(times[1])

    prefill = None
    if not args.no_prefill:
        prefill = run_prefill(dev, rank, world)

    if rank == 0:
        tokens = args.seqs * world * args.steps
        value = tokens / (ms_total * 1e-3)
        e2e = tokens / (ms_e2e * 1e-3)
        ctx_now = [int(c) + args.warmup + args.steps // 2 for c in contexts]      # contexts mid-way through the timed steps
        b_lin, b_full = stack.decode_bytes(ctx_now)
        n_lin = sum(1 for k, _, _ in stack.layers if k == "linear")
        n_full = n_layers - n_lin
        peak, src = measured_peaks()
        fam = {"linear_attn_step": {"ms_per_launch": float(ms_lin), "bytes_per_launch": b_lin / n_lin,
                                    "gbs": b_lin / n_lin / (ms_lin * 1e-3) / 1e9, "launches_per_step": n_lin},
               "full_attn_step": {"ms_per_launch": float(ms_full), "bytes_per_launch": b_full / n_full,
                                  "gbs": b_full / n_full / (ms_full * 1e-3) / 1e9, "launches_per_step": n_full}}
        dom = max(fam, key=lambda k: fam[k]["ms_per_launch"] * fam[k]["launches_per_step"])
        roof = {"bound": "hbm", "kernel": dom, "achieved": fam[dom]["gbs"], "peak": peak, "unit": "GB/s",
                "frac": fam[dom]["gbs"] / peak, "peak_source": f"of {src}",
                "traffic": fam[dom]["bytes_per_launch"] * DRAM_OVER_ALGORITHMIC[dom], "families": fam,
                "whole_step_gbs": (b_lin + b_full) / (ms_total / args.steps * 1e-3) / 1e9}
        cpu = None
        if world == 1 and not args.no_cpu:
            threads = min(os.cpu_count() or 1, 32)
            v, kind, sample, _ = cpu_sample(all_ctx, args.seqs, args.seed, threads)
            cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": workload_config(args, contexts, world),
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / args.steps},
                "gpu_launches": stack.launches_per_step() * args.steps,
                "roofline": roof, "cpu_baseline": cpu, "clocks": clocks, "prefill": prefill}
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
    ap.add_argument("--no-prefill", action="store_true", help="skip the configs[3] prefill leg")
    ap.add_argument("--prefill-only", action="store_true", help="run only the prefill leg (1 GPU) and print its figures")
    ap.add_argument("--prefill-tokens", type=int, default=32768)
    ap.add_argument("--prefill-shape", default="397b", choices=["397b", "35b"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.prefill_only:
        import torch
        torch.cuda.set_device(local_rank)
        print(json.dumps(run_prefill(torch.device("cuda", local_rank), 0, 1, T=args.prefill_tokens, reps=1,
                                     shape=args.prefill_shape)), flush=True)
        return
    if world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
