#!/usr/bin/env python
"""Benchmark of the fused Pythia decode path: per-token latency (TPOT) of greedy decode.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one generated token: embedding -> 32 fused decoder layers -> final
LayerNorm -> LM head -> argmax.  Default workload: Pythia-6.9B shapes, seeded
random-init fp16 weights, batch 1, 4096 cached positions, CUDA-graph replay.
With N > 1 (launched one rank per GPU by torch.distributed.run) the weights are
sharded by attention heads / MLP columns and each layer does one fp16 all-reduce.

One JSON line is printed by rank 0.  `value` is device time per token with all
inputs resident in HBM; `e2e` is the same loop driven through the public API with
the token id crossing the host every step (pinned host buffers, copies inside the
timed region).  `--impl reference` times the fp32 CPU oracle (the PyTorch forward
the reference checks itself against) on the host cores, on a bounded sample of
the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Pythia-6.9B B=1 decode TPOT (us) at 4K context"  # the default workload; other --model / --ctx are labelled below
FALLBACK_HBM_GBS = 6650.0

SHAPES = {  # hidden, heads, head_dim, rotary, ffn, vocab
    "6b9": (4096, 32, 128, 32, 16384, 50432),
    "2b8": (2560, 32, 80, 20, 10240, 50304),
}

# DRAM traffic of ONE whole-token launch (6.9B, 4096 cached rows): dram__bytes_read.sum +
# dram__bytes_write.sum of ncu captures of 2- and 4-layer models of the same shapes, scaled to 32
# layers (traffic is linear in the layer count): 415.4 MB for the tail + 32 x 470.6 MB per layer.
NCU_TRAFFIC_BYTES_PER_TOKEN_6B9_4K = 15.475e9


def algorithmic_bytes_per_token(model: str, n_layers: int, ctx: float, tp: int = 1) -> float:
    """Every weight and KV byte once, fp16; small vectors included; per GPU when tp > 1."""
    H, NH, D, R, F, V = SHAPES[model]
    per_layer = (2 * (3 * H * H + H * H + 2 * H * F) / tp          # QKV, dense, up, down weights
                 + 2 * (3 * H + F) / tp + 2 * (H + H + 4 * H)      # biases (sharded / replicated), LN params
                 + 2 * 2 * ctx * H / tp                            # K and V history
                 + 2 * 2 * H / tp + 2 * 2 * H)                     # K/V append, hidden in + out
    return n_layers * per_layer + 2 * V * H / tp + 2 * H + 2 * 2 * H


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.samples, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def summary(self, t0: float, t1: float) -> dict:
        if self.proc is not None:
            self.proc.terminate()
        rows = [r for t, r in self.samples if t0 <= t <= t1] or [r for _, r in self.samples[-3:]]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(rows[0][1]) if rows[0][1].replace(".", "").isdigit() else None,
                "power_w_max": max((float(r[2]) for r in rows if r[2].replace(".", "").isdigit()), default=None),
                "samples": len(rows), "reasons": reasons}


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json copy bandwidth)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (earlier measurement on this pool)"


# ------------------------------------------------------------------------------------ CPU oracle arm
def oracle_tpot_us(model: str, n_layers: int, ctx: int, sample_layers: int, reps: int, warmup: int):
    """fp32 PyTorch forward on the host cores: `sample_layers` layers + the LM head, scaled to n_layers."""
    from oracle import pythia_oracle as O
    s = O.SHAPES[model]
    torch.set_num_threads(os.cpu_count() or 1)
    layers = [{k: v.float() for k, v in O.make_layer_weights(s, l, seed=1).items()} for l in range(sample_layers)]
    head = {k: v.float() for k, v in O.make_head_weights(s, seed=1).items()}
    caches = [tuple(c.float() for c in O.make_kv_cache(s, ctx, ctx + 1, 50 + l)) for l in range(sample_layers)]
    cos, sin = O.rope_table(ctx + 1, s.rotary)
    x0 = head["embed_in"][17].reshape(1, -1)
    times = []
    for it in range(warmup + reps):
        t0 = time.perf_counter()
        x = x0
        for l in range(sample_layers):
            x, _, _ = O.layer_decode_fp32(s, x, layers[l], caches[l][0], caches[l][1], cos[ctx], sin[ctx], ctx)
        t1 = time.perf_counter()
        logits = O.final_logits_fp32(x, head)
        int(logits.argmax())
        t2 = time.perf_counter()
        if it >= warmup:
            times.append(((t1 - t0) / sample_layers * n_layers + (t2 - t1)) * 1e6)
    return times, torch.get_num_threads()


def run_reference(args, rank):
    if rank != 0:
        return
    t_start = time.perf_counter()
    times, cores = oracle_tpot_us(args.model, args.layers, args.ctx, args.sample_layers, args.steps, args.warmup)
    us = statistics.mean(times)
    sample = (f"{args.sample_layers} of {args.layers} layers + LM head per step, fp32 torch on CPU, "
              f"layer time scaled x{args.layers / args.sample_layers:g}")
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": "us/token", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": {"value": us, "unit": "us/token", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": us, "unit": "us/token", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t_start,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, tp):
    return {"workload": f"pythia-{args.model} greedy decode, batch 1, {args.layers} layers, {args.ctx} cached positions, "
                        f"one token per step, CUDA graph replay",
            "context": args.ctx, "layers": args.layers,
            "parallelism": (f"tp{tp} ({args.tp_mode} all-reduce)" if tp > 1 else "single"),
            "l2": "inputs larger than L2 (weights + KV read once per token: GBs vs 126 MB)"}


def read_ceiling_gbs(dev, hidden, reps=10):
    """Read bandwidth the decode kernel's own streaming machinery reaches when nothing waits on other
    CTAs: one launch streams a [393216, hidden] fp16 matrix (3.2 GB at hidden 4096, far larger than L2)
    through the same persistent grid, TMA ring and row-GEMV consumers as the LM-head phase
    (cf_debug_stream_rows).  Returns (with the dot products, consumers only touching the stages)."""
    import ctypes as C
    from clusterfusionplus_b200 import _lib
    rows = 393216
    m = torch.empty(rows, hidden, dtype=torch.float16, device=dev).normal_(0, 0.02)
    x = torch.randn(hidden, device=dev).half()
    desc = torch.zeros(1024, dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    out = []
    for touch in (0, 1):
        def call():
            _lib.check(_lib.lib.cf_debug_stream_rows(m.data_ptr(), rows, hidden, x.data_ptr(), touch, desc.data_ptr(), st))
        for _ in range(3):
            call()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = None
        for _ in range(reps):
            torch.cuda.synchronize()
            e0.record()
            call()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        out.append(rows * hidden * 2 / (best * 1e-3) / 1e9)
    del m
    return out[0], out[1]


# ------------------------------------------------------------------------------------ GPU arm
def rand_half(shape, gen, dev, mean=0.0, std=0.02):
    return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std + mean).half()


PARITY_STEPS = 16       # greedy tokens compared between the tensor-parallel and the single-GPU decoder
NEAR_TIE_GAP = 5e-3     # a token mismatch only counts as a near tie below this top-2 logit gap (logit std ~ 1.3)


def build_model(args, dev):
    """ONE seeded random-init model, unsharded, straight on the GPU.  Every rank draws the same
    tensors from the same seed (same generator, same GPU type), so the ranks' shards are slices
    of one model and the tensor-parallel result can be compared with a single-GPU decode of it."""
    H, NH, D, R, F, V = SHAPES[args.model]
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    kvw = NH * D
    layers, caches = [], []
    max_seq = args.ctx + max(args.steps + args.warmup, PARITY_STEPS) + 2 * 8 + 8
    for _ in range(args.layers):
        layers.append({
            "qkv_weight": rand_half((3 * kvw, H), g, dev), "qkv_bias": rand_half((3 * kvw,), g, dev),
            "o_weight": rand_half((H, kvw), g, dev), "o_bias": rand_half((H,), g, dev),
            "ln_weight": rand_half((H,), g, dev, 1.0), "ln_bias": rand_half((H,), g, dev),
            "post_ln_weight": rand_half((H,), g, dev, 1.0), "post_ln_bias": rand_half((H,), g, dev),
            "mlp_up_weight": rand_half((F, H), g, dev), "mlp_up_bias": rand_half((F,), g, dev),
            "mlp_down_weight": rand_half((H, F), g, dev), "mlp_down_bias": rand_half((H,), g, dev),
        })
        k = torch.zeros(max_seq, kvw, dtype=torch.float16, device=dev)
        vv = torch.zeros(max_seq, kvw, dtype=torch.float16, device=dev)
        k[:args.ctx] = rand_half((args.ctx, kvw), g, dev, std=1.0)
        vv[:args.ctx] = rand_half((args.ctx, kvw), g, dev, std=1.0)
        caches.append((k, vv))
    head = {"embed_in": rand_half((V, H), g, dev), "final_ln_weight": rand_half((H,), g, dev, 1.0),
            "final_ln_bias": rand_half((H,), g, dev), "embed_out": rand_half((V, H), g, dev)}
    return layers, head, caches, max_seq


def shard_model(cf, dims, layers, head, caches, rank, tp):
    """This rank's contiguous shards of the one model (heads / MLP columns / vocabulary rows)."""
    loc_layers = [cf.shard_layer_weights(w, dims, rank, tp) for w in layers]
    loc_head = cf.shard_head_weights(head, dims, rank, tp)
    loc_caches = [(cf.shard_cache(k, dims, rank, tp), cf.shard_cache(v, dims, rank, tp)) for k, v in caches]
    return loc_layers, loc_head, loc_caches


def tp_parity(cf, dist, args, dec, dims, layers, head, caches, max_seq, rank, tp, dev):
    """Outside every timed region: PARITY_STEPS greedy tokens from the tensor-parallel decoder; all
    ranks must agree on them; rank 0 then decodes the same steps on ONE GPU over the unsharded
    tensors and compares tokens (a mismatch at a step whose top-2 logit gap is below NEAR_TIE_GAP
    is reported as a near tie: the two decoders add the partial sums in different orders) and the
    first step's final hidden state.  The path's tolerance (max-abs 2e-2, relative L2 1e-3) is stated
    for ONE layer against the fp32 oracle; here two fp16 pipelines are compared after `layers` layers,
    each of which rounds the hidden state to fp16, so both bounds are scaled by sqrt(layers)."""
    scale = max(1.0, float(args.layers)) ** 0.5
    dec.reset(args.ctx, 17)
    toks, hid0 = [], None
    for i in range(PARITY_STEPS):
        dec.step()
        toks.append(int(dec.token.item()))
        if i == 0:
            hid0 = dec.hidden.clone()
    status = cf.device_status()
    gathered = [None] * tp
    dist.all_gather_object(gathered, (toks, int(status)))
    out = {"steps": PARITY_STEPS, "ranks_agree": all(g[0] == gathered[0][0] for g in gathered),
           "device_status": max(g[1] for g in gathered)}
    if rank == 0:
        ref_caches = [(k.clone(), v.clone()) for k, v in caches]
        ref = cf.PythiaDecoder(dims, layers, head, ref_caches, max_seq, use_graph=False)
        ref.reset(args.ctx, 17)
        ref_toks, gaps, herr = [], [], None
        for i in range(PARITY_STEPS):
            ref.step()
            ref_toks.append(int(ref.token.item()))
            top2 = torch.topk(ref.logits, 2).values
            gaps.append(float(top2[0] - top2[1]))
            if i == 0:
                d = (hid0.float() - ref.hidden.float()).reshape(-1)
                herr = (float(d.abs().max()), float(d.norm() / ref.hidden.float().norm()))
        out["device_status"] = max(out["device_status"], int(cf.device_status()))
        ref.close()
        first = next((i for i, (a, b) in enumerate(zip(toks, ref_toks)) if a != b), None)
        near_tie = first is not None and gaps[first] < NEAR_TIE_GAP
        out.update({"equals_single_gpu": first is None or near_tie, "first_mismatch": first,
                    "mismatch_is_near_tie": near_tie if first is not None else None,
                    "min_top2_gap": min(gaps), "hidden_max_abs": herr[0], "hidden_rel_l2": herr[1],
                    "hidden_tolerance": {"max_abs": 2e-2 * scale, "rel_l2": 1e-3 * scale},
                    "hidden_within_tolerance": herr[0] <= 2e-2 * scale and herr[1] <= 1e-3 * scale})
    dist.barrier()
    return out


def phase_timeline(cf, dec, args, n_layers, barrier):
    """Device timeline of one token (`--timeline`): one eager launch with the kernel's phase stamps switched on
    (cf_debug_set_trace: globaltimer written by thread 0 of every CTA at each phase boundary).  Returns, in us since
    the layer's first CTA started and averaged over layers 1..n-1, min / mean / max over the CTAs of: LayerNorm done,
    P1 rows done, P2 entered, P2 done, P3 entered, P3 operands staged, P3 GEMV done, P3 done (exchange over);
    the mean distance between layer starts and the length of the token's tail (final LayerNorm, LM head, arg-max)."""
    import numpy as np
    from clusterfusionplus_b200 import _lib
    NE = 16
    G = cf.launch_info(cf.CF_PYTHIA_6B9 if args.model == "6b9" else cf.CF_PYTHIA_2B8)["grid"]
    dec.use_graph = False
    dec.reset(args.ctx, 17)
    for _ in range(3):
        dec.step()
    barrier()
    tr = torch.zeros(G * (n_layers + 1) * NE, dtype=torch.int64, device=dec.token.device)
    _lib.check(_lib.lib.cf_debug_set_trace(tr.data_ptr(), tr.numel()))
    dec.step()
    torch.cuda.synchronize()
    _lib.check(_lib.lib.cf_debug_set_trace(None, 0))
    barrier()
    dec.use_graph = True
    t = tr.cpu().numpy().reshape(G, n_layers + 1, NE).astype(np.float64)
    names = ["layernorm_done", "p1_done", "p2_entered", "p2_done", "p3_entered", "p3_staged", "p3_gemv_done", "p3_done"]
    acc = np.zeros((len(names), 3))
    for l in range(1, n_layers):
        base = t[:, l, 0].min()
        for e in range(len(names)):
            v = (t[:, l, e + 1] - base) / 1e3
            acc[e] += (v.min(), v.mean(), v.max())
    acc /= max(1, n_layers - 1)
    starts = np.array([(t[:, l, 0].min() - t[:, 0, 0].min()) / 1e3 for l in range(n_layers)])
    tail = t[:, n_layers, :]
    return {"unit": "us since the layer's first CTA started; [min, mean, max] over CTAs, mean over layers 1..n-1",
            "events": {n: [round(float(x), 2) for x in acc[i]] for i, n in enumerate(names)},
            "layer_pitch_us": round(float(np.diff(starts).mean()), 2) if n_layers > 1 else None,
            "tail_us": round(float((tail[:, 3].max() - tail[:, 0].min()) / 1e3), 2)}


def run_ours(args, rank, world):
    import torch.distributed as dist
    import clusterfusionplus_b200 as cf

    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp = world
    if tp > 1:
        dist.init_process_group("nccl", device_id=dev)
    # started here so that nvidia-smi is up and printing by the time the timed loops run (they last tens of ms)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    H, NH, D, R, F, V = SHAPES[args.model]
    dims = cf.CfDims()
    dims.hidden, dims.heads, dims.head_dim, dims.rotary, dims.ffn, dims.vocab = H, NH, D, R, F, V
    layers, head, caches, max_seq = build_model(args, dev)
    if tp == 1:
        dec = cf.PythiaDecoder(dims, layers, head, caches, max_seq, use_graph=True)
        launches_per_token = 1
    else:
        loc_layers, loc_head, loc_caches = shard_model(cf, dims, layers, head, caches, rank, tp)
        if rank != 0:   # only rank 0 keeps the unsharded tensors (for the single-GPU comparison)
            layers = head = caches = None
            torch.cuda.empty_cache()
        dec = cf.TPDecoder(dims, loc_layers, loc_head, loc_caches, max_seq, use_graph=True, fused=(args.tp_mode == "fused"))
        launches_per_token = dec.launches_per_token
    K, W = args.steps, args.warmup

    def barrier():
        if tp > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: device time, everything resident
    dec.reset(args.ctx, 17)
    for _ in range(W):
        dec.step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    torch.cuda.nvtx.range_push("value_timed")
    e0.record()
    for _ in range(K):
        dec.step()
    e1.record()
    barrier()
    torch.cuda.nvtx.range_pop()
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1)
    status = cf.device_status()
    if tp > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    tpot_us = ms / K * 1e3
    mean_ctx = args.ctx + W + K / 2

    # ---- e2e: token id crosses the host every step (pinned buffers), copies timed
    pin_in = torch.zeros(1, dtype=torch.int32).pin_memory()
    pin_out = torch.zeros(1, dtype=torch.int32).pin_memory()
    dec.reset(args.ctx, 17)
    pin_in[0] = 17
    for _ in range(W):
        dec.token.copy_(pin_in, non_blocking=True)
        dec.step()
        pin_out.copy_(dec.token, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        pin_in[0] = int(pin_out[0])
    barrier()
    e0.record()
    w0 = time.perf_counter()
    for _ in range(K):
        dec.token.copy_(pin_in, non_blocking=True)
        dec.step()
        pin_out.copy_(dec.token, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        pin_in[0] = int(pin_out[0])
    e1.record()
    barrier()
    w1 = time.perf_counter()
    e2e_ms = max(e0.elapsed_time(e1), (w1 - w0) * 1e3)
    # clocks over both timed loops (the same launches back to back: the device-timed one alone can be shorter
    # than the sampling period)
    clocks = sampler.summary(t0, w1) if sampler else None
    if tp > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()
    status = status or cf.device_status()
    parity = None
    if tp > 1 and not args.no_parity:
        parity = tp_parity(cf, dist, args, dec, dims, layers, head, caches, max_seq, rank, tp, dev)
    timeline = phase_timeline(cf, dec, args, args.layers, barrier) if args.timeline else None
    if rank != 0:
        dec.close()
        if tp > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = hbm_peak()
    bytes_token = algorithmic_bytes_per_token(args.model, args.layers, mean_ctx, tp)
    achieved = bytes_token / (tpot_us * 1e-6) / 1e9
    traffic = None
    if tp == 1 and args.model == "6b9" and args.ctx == 4096 and args.layers == 32:
        traffic = NCU_TRAFFIC_BYTES_PER_TOKEN_6B9_4K
    metric = METRIC if (args.model == "6b9" and args.ctx == 4096) else f"Pythia-{args.model} B=1 decode TPOT (us) at {args.ctx} context"
    config = workload_config(args, tp)
    parity_ok = True
    if parity is not None:
        config["parity"] = parity
        parity_ok = (parity["ranks_agree"] and parity["equals_single_gpu"] and parity["hidden_within_tolerance"]
                     and parity["device_status"] == 0)
    line = {
        "metric": metric, "value": tpot_us, "unit": "us/token", "n_gpus": tp, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp16 (fp32 accumulate)", "data": "synthetic", "config": config,
        "clocks": clocks,
        "e2e": {"value": e2e_ms / K * 1e3, "unit": "us/token", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "gpu_launches": K * launches_per_token,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_source": peak_src, "bytes_per_launch_algorithmic": bytes_token,
                     "frac_of_8TBs_nominal": achieved / 8000.0, "per_gpu": tp > 1,
                     "kernel": "fused_decode_kernel (one launch per token)" if (tp == 1 or args.tp_mode == "fused") else
                               "fused_decode_kernel per layer + NCCL all-reduce (whole token timed)"},
        "launch": cf.launch_info(cf.CF_PYTHIA_6B9 if args.model == "6b9" else cf.CF_PYTHIA_2B8),
        "device_status": status,
    }
    if timeline is not None:
        line["timeline"] = timeline
    if tp == 1 and not args.no_read_ceiling:
        with_math, touch = read_ceiling_gbs(dev, H)
        line["roofline"]["read_ceiling_gbs"] = with_math
        line["roofline"]["read_ceiling_touch_only_gbs"] = touch
        line["roofline"]["frac_of_read_ceiling"] = achieved / with_math
        line["roofline"]["read_ceiling_how"] = ("one launch of the same persistent grid, TMA ring and row-GEMV consumers "
                                                "streaming a 3.2 GB fp16 matrix with no cross-CTA waits; best of 10")
        line["device_status"] = line["device_status"] or cf.device_status()
    if tp == 1 and not args.no_cpu_baseline:
        times, cores = oracle_tpot_us(args.model, args.layers, args.ctx, args.sample_layers, 5, 1)
        line["cpu_baseline"] = {
            "value": statistics.mean(times), "unit": "us/token", "cores": cores, "kind": "port",
            "sample": f"{args.sample_layers} of {args.layers} layers + LM head, 5 steps after 1 warm-up, fp32 torch oracle, "
                      f"layer time scaled x{args.layers / args.sample_layers:g}"}
    print(json.dumps(line), flush=True)
    dec.close()
    if tp > 1:
        dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit(f"tensor-parallel parity check failed: {json.dumps(parity)}")


def run_graph_step_api(args):
    """What a caller of the reference's own API gets (`--api graph_step`): the decode loop of the reference's
    tests/benchmark_decode_6b9.py:133-198 -- embedding lookup, one pythia_6b9_graph_decode_step per layer through
    per-layer graph contexts, torch final LayerNorm + LM head + arg-max -- with token id and sequence length kept
    on the device (graph_set_device_state) and the whole token captured once in a CUDA graph.  Same workload,
    metric and roofline arithmetic as the default line, which runs the whole token as ONE launch instead."""
    import clusterfusionplus_b200 as cf
    import torch.nn.functional as F

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    H, NH, D, R, Fd, V = SHAPES[args.model]
    pre = f"pythia_{args.model}_"
    create, step, destroy, set_state = (getattr(cf, pre + n) for n in
                                        ("create_graph_context", "graph_decode_step", "destroy_graph_context", "graph_set_device_state"))
    layers, head, caches, max_seq = build_model(args, dev)
    cos_t, sin_t = cf.rope_table(max_seq, R, dev)
    seq = torch.full((1,), args.ctx, dtype=torch.int32, device=dev)
    token = torch.full((1,), 17, dtype=torch.int64, device=dev)
    for l, (w, (k, v)) in enumerate(zip(layers, caches)):
        create(l, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], max_seq)
        set_state(l, seq, cos_t, sin_t)

    def one_token():
        h = head["embed_in"].index_select(0, token).contiguous()
        for l, (w, (k, v)) in enumerate(zip(layers, caches)):
            h, _, _ = step(l, h, w["ln_weight"], w["ln_bias"], w["qkv_bias"], w["o_bias"], cos_t[0], sin_t[0], k, v,
                           w["post_ln_weight"], w["post_ln_bias"], w["mlp_up_bias"], w["mlp_down_bias"], 0)
        h = F.layer_norm(h, (H,), head["final_ln_weight"], head["final_ln_bias"], eps=1e-5)
        logits = h @ head["embed_out"].t()
        token.copy_(torch.argmax(logits, dim=-1))
        seq.add_(1)

    K, W = args.steps, args.warmup
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        one_token()  # descriptor uploads happen here, outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        one_token()
    seq.fill_(args.ctx)
    token.fill_(17)
    for _ in range(W):
        graph.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(K):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.summary(t0, time.perf_counter())
    us = e0.elapsed_time(e1) / K * 1e3
    status = cf.device_status()
    peak, peak_src = hbm_peak()
    bytes_token = algorithmic_bytes_per_token(args.model, args.layers, args.ctx + W + K / 2)
    achieved = bytes_token / (us * 1e-6) / 1e9
    cfg = workload_config(args, 1)
    cfg["workload"] += f"; driven through the reference API: {args.layers} x graph_decode_step + torch embedding / final LayerNorm / LM head / arg-max per token"
    print(json.dumps({
        "metric": METRIC if (args.model == "6b9" and args.ctx == 4096) else f"Pythia-{args.model} B=1 decode TPOT (us) at {args.ctx} context",
        "value": us, "unit": "us/token", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": us / 1e3,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
        "data": "synthetic", "config": cfg, "clocks": clocks, "gpu_launches": K * args.layers,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": peak_src, "bytes_per_launch_algorithmic": bytes_token / args.layers,
                     "frac_of_8TBs_nominal": achieved / 8000.0,
                     "kernel": "fused_decode_kernel, one launch per layer (+ torch library kernels for the tail)"},
        "device_status": status,
    }), flush=True)
    for l in range(len(layers)):
        destroy(l)


def tensor_peak():
    """(TFLOP/s, source): the measured cuBLAS bf16 burst figure of this pool if the driver left one."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json, burst)"
    except Exception:
        return 1590.0, "fallback (1.59 PFLOP/s)"


def run_prefill(args):
    """Secondary line: prompt ingestion of --prefill-tokens positions through PythiaDecoder.prefill()
    (tensor-core GEMMs of this library + torch LayerNorm / RoPE / causal attention), and the four
    linear layers of a block timed alone for the tensor roofline."""
    import clusterfusionplus_b200 as cf
    from clusterfusionplus_b200.decoder import prefill_linear
    from clusterfusionplus_b200._lib import CF_ACT_GELU_TANH, CF_ACT_NONE, CfDims

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m = args.prefill_tokens
    H, NH, D, R, F, V = SHAPES[args.model]
    args.ctx = 0
    layers, head, caches, _ = build_model(args, dev)
    max_seq = caches[0][0].shape[0]
    if m + 1 > max_seq:
        caches = [(torch.zeros(m + 8, NH * D, dtype=torch.float16, device=dev),
                   torch.zeros(m + 8, NH * D, dtype=torch.float16, device=dev)) for _ in layers]
        max_seq = m + 8
    d = CfDims()
    d.hidden, d.heads, d.head_dim, d.rotary, d.ffn, d.vocab = H, NH, D, R, F, V
    dec = cf.PythiaDecoder(d, layers, head, caches, max_seq, use_graph=False)
    g = torch.Generator(device="cpu")
    g.manual_seed(7)
    prompt = torch.randint(0, V, (m + 1,), generator=g).tolist()  # prefill() leaves the last token to decode

    def timed(fn, reps, warm):
        for _ in range(warm):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ms_pass = timed(lambda: dec.prefill(prompt), args.steps, args.warmup)
    w = layers[0]
    x = rand_half((m, H), torch.Generator(device=dev), dev, std=1.0)
    xf = rand_half((m, F), torch.Generator(device=dev), dev, std=1.0)
    gemms = [(x, w["qkv_weight"], w["qkv_bias"], None, CF_ACT_NONE), (x, w["o_weight"], w["o_bias"], x, CF_ACT_NONE),
             (x, w["mlp_up_weight"], w["mlp_up_bias"], None, CF_ACT_GELU_TANH),
             (xf, w["mlp_down_weight"], w["mlp_down_bias"], x, CF_ACT_NONE)]
    ms_gemm = timed(lambda: [prefill_linear(*a) for a in gemms], max(args.steps, 5), args.warmup)
    flops = 2.0 * m * (3 * H * H + H * H + 2 * H * F)
    peak, src = tensor_peak()
    tf = flops / (ms_gemm * 1e-3) / 1e12
    print(json.dumps({
        "metric": "prompt ingestion throughput (tokens/s)", "value": m / (ms_pass * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_pass, "higher_is_better": True,
        "dtype": "fp16 operands, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"pythia-{args.model} shapes, {args.layers} layers, prompt of {m} tokens, batch 1"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                     "peak_source": src, "kernel": "the four linear layers of one block (QKV, O, MLP up + GELU, MLP down)",
                     "ms_per_block": ms_gemm, "traffic": None},
        "gemm_share_of_pass": ms_gemm * args.layers / ms_pass,
        "device_status": cf.device_status(),
    }))
    dec.close()


def run_llama_stack(args):
    """Secondary line: one decode step at batch 1 through a Llama-2-7B-shaped stack of --layers layers
    (attention block + SwiGLU MLP block per layer), every layer with its own --llama-ctx rows of KV cache.  The 2 x
    layers blocks of a step are launched one by one and replayed as one CUDA graph; --llama-one-launch runs them as ONE
    persistent launch (cf_batch_begin / cf_batch_end)."""
    import clusterfusionplus_b200 as cf

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    H, NH, D, F, S, L = 4096, 32, 128, 11008, args.llama_ctx, args.layers
    g = torch.Generator(device=dev)
    g.manual_seed(4321)
    layers = []
    for _ in range(L):
        layers.append(dict(
            weight_qkv=rand_half((3 * H, H), g, dev), weight_o=rand_half((H, H), g, dev),
            rms_input_weight=rand_half((H,), g, dev, 1.0), k_cache=rand_half((S, H), g, dev, std=1.0),
            v_cache=rand_half((S, H), g, dev, std=1.0), gate_up_weight=rand_half((2 * F, H), g, dev),
            down_weight=rand_half((H, F), g, dev), rms_post_weight=rand_half((H,), g, dev, 1.0)))
    ang = torch.rand(D // 2, generator=g, device=dev) * (2 * torch.pi)
    cos, sin = torch.cat([ang.cos(), ang.cos()]).contiguous(), torch.cat([ang.sin(), ang.sin()]).contiguous()
    x0, r0 = rand_half((1, H), g, dev, std=1.0), rand_half((1, H), g, dev, std=1.0)
    stack = cf.LlamaLayerStack(layers, eps=1e-5, one_launch=args.llama_one_launch)

    def step():
        stack.step(x0, r0, cos, sin)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()  # builds the per-layer descriptors (allocations) outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    sampler = ClockSampler(0)
    for _ in range(args.warmup):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.summary(t0, time.perf_counter())
    us = e0.elapsed_time(e1) / args.steps * 1e3
    per_layer = 2 * (3 * H * H + H * H + 3 * H * F) + 2 * 2 * S * H + 2 * (2 * H) + 2 * 2 * H * 4  # weights, KV, norms, x/res in-out
    peak, src = hbm_peak()
    gbs = per_layer * L / (us * 1e-6) / 1e9
    print(json.dumps({
        "metric": "Llama-2-7B-shaped layer stack, B=1 decode step (us)", "value": us, "unit": "us/token", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
        "dtype": "fp16 weights/KV, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"{L} layers x (attention block + SwiGLU MLP 4096-11008-4096), batch 1, {S} cached rows per layer",
                   "l2": "per-step working set far larger than L2"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "peak_source": src,
                     "algorithmic_bytes_per_step": per_layer * L, "traffic": None},
        "gpu_launches": (1 if args.llama_one_launch else 2 * L) * args.steps, "clocks": clocks, "device_status": cf.device_status(),
    }))


def run_llama_batch(args):
    """Secondary line (BASELINE config 5 at batch 4 / 16): one decode step of --batch sequences through a
    Llama-2-7B-shaped stack of --layers layers -- the batched, paged attention block (reference entry point
    llama_decoder_layer_batch_decode_sglang) followed by the batched SwiGLU MLP block -- 2 launches per
    layer replayed as one CUDA graph.  Every sequence has --llama-ctx cached rows per layer, scattered over
    a shuffled token pool."""
    import clusterfusionplus_b200 as cf

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    H, NH, D, F, S, L, B = 4096, 32, 128, 11008, args.llama_ctx, args.layers, args.batch
    g = torch.Generator(device=dev)
    g.manual_seed(4321)
    layers, pools = [], []
    n_rows = B * (S + 1)
    for _ in range(L):
        layers.append(dict(wqkv=rand_half((3 * H, H), g, dev), wo=rand_half((H, H), g, dev), g1=rand_half((H,), g, dev, 1.0),
                           wgu=rand_half((2 * F, H), g, dev), wd=rand_half((H, F), g, dev), g2=rand_half((H,), g, dev, 1.0)))
        pools.append((rand_half((n_rows, H), g, dev, std=1.0), rand_half((n_rows, H), g, dev, std=1.0)))
    perm = torch.randperm(n_rows, generator=torch.Generator().manual_seed(5)).to(torch.int32)
    indptr = torch.arange(0, B + 1, dtype=torch.int32) * (S + 1)
    indptr, indices = indptr.to(dev), perm.to(dev)
    kptrs = torch.tensor([p[0].data_ptr() for p in pools], dtype=torch.int64, device=dev)
    vptrs = torch.tensor([p[1].data_ptr() for p in pools], dtype=torch.int64, device=dev)
    positions = torch.full((B,), S, dtype=torch.int64, device=dev)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(S + 1, dtype=torch.float32), inv)
    cos_sin = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous().to(dev)
    x0, r0 = rand_half((B, H), g, dev, std=1.0), rand_half((B, H), g, dev, std=1.0)
    bufs = [torch.empty(B, H, dtype=torch.float16, device=dev) for _ in range(4)]

    def step():
        x, r = x0, r0
        for l, w in enumerate(layers):
            cf.llama_decoder_layer_batch_decode_sglang(bufs[0], bufs[1], x, r, w["wqkv"], w["wo"], indptr, indices, kptrs, vptrs, l,
                                                       w["g1"], 1e-5, positions, cos_sin)
            x, r = cf.llama_mlp_batch_sglang(bufs[0], bufs[1], w["wgu"], w["wd"], w["g2"], 1e-5)
        return x

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()  # scratch allocation and tensor maps outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    sampler = ClockSampler(0)
    for _ in range(args.warmup):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.summary(t0, time.perf_counter())
    us = e0.elapsed_time(e1) / args.steps * 1e3
    per_layer = 2 * (3 * H * H + H * H + 3 * H * F) + B * 2 * 2 * S * H + 2 * (2 * H) + B * 2 * H * 8  # weights, KV, norms, activations
    peak, src = hbm_peak()
    gbs = per_layer * L / (us * 1e-6) / 1e9
    print(json.dumps({
        "metric": "Llama-2-7B-shaped layer stack, batched decode step (us)", "value": us, "unit": "us/step", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
        "dtype": "fp16 weights/KV/activations, fp32 accumulate (tcgen05)", "data": "synthetic",
        "config": {"workload": f"{L} layers x (paged attention block + SwiGLU MLP 4096-11008-4096), batch {B}, {S} cached rows "
                               f"per sequence and layer in a shuffled token pool", "batch": B,
                   "l2": "per-step working set far larger than L2"},
        "tokens_per_s": B / (us * 1e-6),
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "peak_source": src,
                     "algorithmic_bytes_per_step": per_layer * L, "traffic": None,
                     "kernel": "llama_batch_kernel (tcgen05 skinny GEMMs + paged attention), 2 launches per layer"},
        "gpu_launches": 2 * L * args.steps, "clocks": clocks, "device_status": cf.device_status(),
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="6b9", choices=sorted(SHAPES))
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--sample-layers", type=int, default=2, help="layers the CPU oracle runs per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-read-ceiling", action="store_true",
                    help="skip the measurement of the kernel's own read-streaming ceiling (N = 1)")
    ap.add_argument("--no-parity", action="store_true",
                    help="N > 1: skip the comparison with a single-GPU decode of the same model (outside the timed regions)")
    ap.add_argument("--timeline", action="store_true",
                    help="add the device timeline of one token (phase stamps of every CTA, rank 0's view) to the line")
    ap.add_argument("--tp-mode", default="fused", choices=["fused", "nccl"],
                    help="N > 1: in-kernel all-reduce over peer memory (default) or one NCCL all-reduce per layer")
    ap.add_argument("--llama-ctx", type=int, default=0,
                    help="instead of Pythia decode: one step through a Llama-2-7B-shaped layer stack with this many "
                         "cached rows per layer (1 GPU, batch 1; a secondary line)")
    ap.add_argument("--api", default="decoder", choices=["decoder", "graph_step"],
                    help="decoder: the whole token as one launch (default); graph_step: the reference's per-layer "
                         "graph_decode_step API in the reference's decode loop, captured in a CUDA graph (1 GPU)")
    ap.add_argument("--batch", type=int, default=1,
                    help="with --llama-ctx: decode sequences per step; > 1 (or --llama-batched) uses the batched, paged blocks")
    ap.add_argument("--llama-one-launch", action="store_true", help="with --llama-ctx at batch 1: all blocks of a step as one launch")
    ap.add_argument("--llama-batched", action="store_true", help="with --llama-ctx: the batched, paged blocks even at batch 1")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help="instead of decode: time prompt ingestion of this many tokens (1 GPU; a secondary line)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.prefill_tokens > 0:
        run_prefill(args)
        return
    if args.llama_ctx > 0:
        if args.batch > 1 or args.llama_batched:
            run_llama_batch(args)
        else:
            run_llama_stack(args)
        return
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.api == "graph_step":
        if rank == 0:
            run_graph_step_api(args)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nnodes=1 "
                             "--nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...")
    run_ours(args, rank, world)


if __name__ == "__main__":
    main()
