#!/usr/bin/env python
"""Benchmark of the KV-cache hot path: fused RoPE + K/V append + paged GQA flash-decode.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c2|c2-paged|c3|c3-small|c4|c5]

Workload (default `c3`, the batched paged-decode configuration the headline metric is quoted on):
Qwen2.5-3B shape, 36 layers, 16 q heads / 2 kv heads, head_dim 128, batch 64, per-sequence
context lengths uniform in [512, 16384] from the seed, page size 16, page table a seeded random
permutation of a shared f16 page pool (one K and one V pool per layer).  A step appends one
token per sequence in every layer and attends over the whole context: 36 launches of the fused
kernel.  Inputs are synthetic N(0,1) f16; no model weights are involved.

With N > 1 (launched by torchrun, one rank per GPU) every rank owns its own batch of 64
sequences (seed + rank) and its own pools: sequences are independent, so there is no data-path
collective and the scaling is weak.  torch.distributed (NCCL) is used for the barrier and the
max-over-ranks of the device time only.

`--impl reference` times the CPU restatement of the reference's math (the oracle; the reference
itself is Rust + Metal and cannot run here) on the host cores, one layer per step, and scales
to the full step.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: layers, Hq, Hkv, D, batch, len_lo, len_hi, page_size, theta, rope_mode
    "c3": dict(layers=36, n_heads=16, n_kv_heads=2, head_dim=128, batch=64, lo=512, hi=16384, page_size=16,
               theta=1e6, rope_mode=0,
               name="batched paged decode, Qwen2.5-3B shape: 36 layers, 16q/2kv heads, D128, batch 64, "
                    "ctx U[512,16384], page 16, fused rope+append+decode"),
    "c3-kv8": dict(layers=36, n_heads=16, n_kv_heads=2, head_dim=128, batch=64, lo=512, hi=16384, page_size=16,
                   theta=1e6, rope_mode=0, kv8=True,
                   name="batched paged decode on the 8-bit cache (FP8 E4M3 + one f32 scale per row), Qwen2.5-3B shape: "
                        "36 layers, 16q/2kv heads, D128, batch 64, ctx U[512,16384], page 16, fused rope+quantising "
                        "append+decode"),
    "c3-kv8-small": dict(layers=4, n_heads=16, n_kv_heads=2, head_dim=128, batch=64, lo=512, hi=16384, page_size=16,
                         theta=1e6, rope_mode=0, kv8=True, name="c3-kv8 with 4 layers (profiling case)"),
    "c3-small": dict(layers=4, n_heads=16, n_kv_heads=2, head_dim=128, batch=64, lo=512, hi=16384, page_size=16,
                     theta=1e6, rope_mode=0, name="c3 with 4 layers (profiling case)"),
    "c2-paged": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, batch=1, lo=8191, hi=8191, page_size=64,
                     theta=5e5, rope_mode=1,
                     name="Llama-3.2-3B shape decode step: 28 layers, 24q/8kv heads, D128, batch 1, ctx 8192, "
                          "cache as 64-token pages in order, one fused launch per layer"),
    # the batch-1 step on the 8-bit cache: pages in order, the library's own plan (cluster form), CUDA-graph replay
    "c2-kv8": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, batch=1, lo=8191, hi=8191, page_size=64,
                   theta=5e5, rope_mode=1, kv8=True, auto_plan=True, graph=True,
                   name="Llama-3.2-3B shape decode step on the 8-bit cache (FP8 E4M3 + one f32 scale per row): 28 layers, "
                        "24q/8kv heads, D128, batch 1, ctx 8192, 64-token pages in order, one fused launch per layer, "
                        "CUDA-graph replay"),
}
LONG_CONTEXT = {
    # sequence-sharded single-sequence decode (strong scaling): pages of ONE sequence are cut into
    # contiguous ranges over the ranks; per layer one all-gather of (acc, m, l) and the merge.
    "c5": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, kv_len=131072, page_size=64, theta=5e5, rope_mode=1,
               name="long-context single-sequence decode, Llama-3.2-3B shape: 28 layers, 24q/8kv heads, D128, "
                    "131072 cached tokens, page 64, sequence-sharded with (O,m,l) all-gather + merge"),
    # c5 on the 8-bit cache (the same three exchange routes)
    "c5-kv8": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, kv_len=131072, page_size=64, theta=5e5, rope_mode=1,
                   kv8=True,
                   name="long-context single-sequence decode on the 8-bit cache (FP8 E4M3 + one f32 scale per row), "
                        "Llama-3.2-3B shape: 28 layers, 24q/8kv heads, D128, 131072 cached tokens, page 64, "
                        "sequence-sharded with (O,m,l) all-gather + merge"),
    "c5-kv8-32k": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, kv_len=32768, page_size=64, theta=5e5, rope_mode=1,
                       kv8=True, name="c5-32k on the 8-bit cache (the per-GPU shape of c5-kv8 at 8 GPUs, on 2)"),
    "c5-small": dict(layers=4, n_heads=24, n_kv_heads=8, head_dim=128, kv_len=131072, page_size=64, theta=5e5,
                     rope_mode=1, name="c5 with 4 layers (test case)"),
    # the per-GPU shape of c5 at 8 GPUs (16384 tokens per rank: short launches, cluster form) on 2 and on 4 GPUs
    "c5-32k": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, kv_len=32768, page_size=64, theta=5e5, rope_mode=1,
                   name="long-context single-sequence decode, Llama-3.2-3B shape, 32768 cached tokens, page 64, sequence-sharded"),
    "c5-64k": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, kv_len=65536, page_size=64, theta=5e5, rope_mode=1,
                   name="long-context single-sequence decode, Llama-3.2-3B shape, 65536 cached tokens, page 64, sequence-sharded"),
}
SEED = 0x5EED
METRIC = "kv_append_decode_attn_tokens_per_s"
# DRAM bytes moved by the decode kernel per algorithmic byte: dram__bytes_read.sum + dram__bytes_write.sum of
# one ncu capture of a 4-layer C3 step over the algorithmic bytes of the same launch.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0099


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def make_lengths(w, seed):
    rng = np.random.default_rng(seed)
    cached = rng.integers(w["lo"], w["hi"] + 1, size=w["batch"]).astype(np.uint32)
    return cached, cached + 1  # cached tokens, kv_len after the append


def make_page_table(w, kv_lens, seed):
    P = w["page_size"]
    pages = (kv_lens + P - 1) // P
    n_pages = int(pages.sum())
    rng = np.random.default_rng(seed + 1)
    shuffle = w["batch"] > 1
    perm = rng.permutation(n_pages).astype(np.uint32) if shuffle else np.arange(n_pages, dtype=np.uint32)
    stride = int(pages.max())
    table = np.zeros((w["batch"], stride), np.uint32)
    o = 0
    for b in range(w["batch"]):
        n = int(pages[b])
        table[b, :n] = perm[o:o + n]
        o += n
    return table, n_pages


def algorithmic_bytes_per_layer(w, kv_lens):
    """K and V read once per KV head (incl. the new row) + new k,v read + cache row write + q read,
    out write + cos/sin row + page ids."""
    hq, hkv, d, P = w["n_heads"], w["n_kv_heads"], w["head_dim"], w["page_size"]
    row = d + 4 if w.get("kv8") else d * 2  # bytes of a cached row: e4m3 bytes + its f32 scale, or f16
    total = 0
    for L in kv_lens.astype(np.int64):
        total += 2 * hkv * L * row + 2 * hkv * d * 2 + 2 * hkv * row + 2 * hq * d * 2 + 2 * (d // 2) * 2
        total += 4 * ((L + P - 1) // P)
    return int(total)


def config_of(w):
    """The `config` object of a batched-decode line: the same for this arm and the reference arm (rank 0's
    figures; rank r draws its lengths and page table from seed + r)."""
    cached, kv_lens = make_lengths(w, SEED)
    P = w["page_size"]
    n_pages = int(((kv_lens + P - 1) // P).sum())
    pool_gb = 2 * w["layers"] * n_pages * w["n_kv_heads"] * P * (w["head_dim"] + 4 if w.get("kv8") else w["head_dim"] * 2) / 1e9
    return {"workload": w["name"], "layers": w["layers"], "batch_per_gpu": w["batch"],
            "tokens_cached_per_gpu": int(cached.sum()), "pages_per_layer": n_pages, "seed": SEED,
            "seed_rule": "rank r uses seed + r", "l2": "inputs larger than L2 (KV pools %.1f GB per GPU)" % pool_gb}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.2] or [l for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            f = [x.strip() for x in r.split(",")]
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- ours ---

def apply_options(mfk, f, args):
    """Library options that a run may override from the command line."""
    if getattr(args, "plan_item_cost", 0):
        f.set_option(mfk.OPTION_PLAN_ITEM_COST, args.plan_item_cost)
    if getattr(args, "decode_stages", 0):
        f.set_option(mfk.OPTION_DECODE_STAGES, args.decode_stages)


def run_ours(args, w):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    rank, world, local = rank_setup()
    dev = torch.device("cuda", torch.cuda.current_device())
    mfk = importlib.import_module("test-burn_b200")  # raises if the CUDA library is missing

    layers, hq, hkv, d, B, P = w["layers"], w["n_heads"], w["n_kv_heads"], w["head_dim"], w["batch"], w["page_size"]
    seed = SEED + rank
    cached, kv_lens = make_lengths(w, seed)
    table, n_pages = make_page_table(w, kv_lens, seed)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    pool_elems = n_pages * hkv * P * d
    kv8 = bool(w.get("kv8"))
    if kv8:
        # bytes of finite E4M3 values (exponent field below 15) with random signs; scales of N(0,1) rows (amax / 448)
        def fp8_pool():
            t = torch.randint(0, 0x78, (pool_elems,), dtype=torch.uint8, device=dev, generator=gen)
            return t | (torch.randint(0, 2, (pool_elems,), dtype=torch.uint8, device=dev, generator=gen) << 7)

        k_pools = [fp8_pool() for _ in range(layers)]
        v_pools = [fp8_pool() for _ in range(layers)]
        k_scales = [torch.full((pool_elems // d,), 3.5 / 448, dtype=torch.float32, device=dev) for _ in range(layers)]
        v_scales = [torch.full((pool_elems // d,), 3.5 / 448, dtype=torch.float32, device=dev) for _ in range(layers)]
    else:
        k_pools = [torch.empty(pool_elems, dtype=torch.float16, device=dev).normal_(generator=gen) for _ in range(layers)]
        v_pools = [torch.empty(pool_elems, dtype=torch.float16, device=dev).normal_(generator=gen) for _ in range(layers)]
    d_table = torch.from_numpy(table.view(np.int32)).to(dev)
    d_lens = torch.from_numpy(kv_lens.view(np.int32)).to(dev)
    cos_np, sin_np = mfk.rope_tables(w["theta"], d, int(kv_lens.max()))
    d_cos = torch.from_numpy(cos_np.view(np.float16)).to(dev)
    d_sin = torch.from_numpy(sin_np.view(np.float16)).to(dev)
    # per-layer step inputs: host (pinned) and device copies
    cpu_gen = torch.Generator().manual_seed(seed)
    h_q = torch.randn((layers, B, hq * d), generator=cpu_gen).half().pin_memory()
    h_k = torch.randn((layers, B, hkv * d), generator=cpu_gen).half().pin_memory()
    h_v = torch.randn((layers, B, hkv * d), generator=cpu_gen).half().pin_memory()
    h_out = torch.empty((layers, B, hq * d), dtype=torch.float16).pin_memory()
    h_table = torch.from_numpy(table.view(np.int32)).pin_memory()
    h_lens = torch.from_numpy(kv_lens.view(np.int32)).pin_memory()
    d_q, d_k, d_v = h_q.to(dev), h_k.to(dev), h_v.to(dev)
    d_out = torch.empty((layers, B, hq * d), dtype=torch.float16, device=dev)

    stream = torch.cuda.Stream(device=dev)
    copy_in, copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    f = mfk.Foundry(dev.index, stream.cuda_stream)
    apply_options(mfk, f, args)
    if not args.no_overlap:
        f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 1)
    if kv8:
        plan = f.decode_plan(kv_lens, n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P,
                             max_ctas=0 if w.get("auto_plan") else 2 * torch.cuda.get_device_properties(dev).multi_processor_count)
        descs = [mfk.paged_kv8(k_pools[i].view(n_pages, hkv, P, d), v_pools[i].view(n_pages, hkv, P, d),
                               k_scales[i].view(n_pages, hkv, P), v_scales[i].view(n_pages, hkv, P), d_table, d_lens,
                               n_kv_heads=hkv, page_size=P) for i in range(layers)]
        decode = f.paged_decode_kv8
    else:
        plan = f.decode_plan(kv_lens, n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P)
        descs = [mfk.paged_kv(k_pools[i].view(n_pages, hkv, P, d), v_pools[i].view(n_pages, hkv, P, d), d_table, d_lens,
                              n_kv_heads=hkv, page_size=P, head_dim=d) for i in range(layers)]
        decode = f.paged_decode
    scale = 1.0 / math.sqrt(d)

    def device_step():
        for i in range(layers):
            decode(plan, descs[i], d_q[i], d_out[i], n_heads=hq, k=d_k[i], v=d_v[i], cos=d_cos, sin=d_sin,
                           rope=True, rope_mode=w["rope_mode"], append=True, scale=scale)

    # End-to-end step: host inputs -> device -> host results, through the same C-ABI calls.  The page
    # table, lengths and work plan are rebuilt from host state each step as a serving loop would; per
    # layer the q/k/v rows go up and the attention output comes back; the KV pools are cache state
    # and stay resident.  Uploads and downloads run on copy streams, ordered by events.
    # q, k and v rows of a layer travel as ONE pinned block and one copy
    nq, nk = B * hq * d, B * hkv * d
    h_qkv = torch.empty((layers, nq + 2 * nk), dtype=torch.float16).pin_memory()
    h_qkv[:, :nq] = h_q.view(layers, -1)
    h_qkv[:, nq:nq + nk] = h_k.view(layers, -1)
    h_qkv[:, nq + nk:] = h_v.view(layers, -1)
    # Layers travel in groups: one upload and one download per group and slot, two slots in rotation.
    # Every event wait on the launch stream breaks the programmatic overlap of two launches, so the
    # fewer the better; the group size keeps a group's transfers well inside its compute time.
    GROUP = max(1, min(args.e2e_group, layers))
    # the first upload and the last download are the two transfers nothing hides: one layer each
    bounds = [0]
    if layers > 2 and GROUP > 1:
        bounds.append(1)
        while bounds[-1] + GROUP < layers - 1:
            bounds.append(bounds[-1] + GROUP)
        if bounds[-1] < layers - 1:
            bounds.append(layers - 1)
        bounds.append(layers)
    else:
        while bounds[-1] < layers:
            bounds.append(min(layers, bounds[-1] + GROUP))
    n_groups = len(bounds) - 1
    e2e_qkv = torch.empty((2, GROUP, nq + 2 * nk), dtype=torch.float16, device=dev)
    e2e_q = [[e2e_qkv[s, j, :nq].view(B, hq * d) for j in range(GROUP)] for s in range(2)]
    e2e_k = [[e2e_qkv[s, j, nq:nq + nk].view(B, hkv * d) for j in range(GROUP)] for s in range(2)]
    e2e_v = [[e2e_qkv[s, j, nq + nk:].view(B, hkv * d) for j in range(GROUP)] for s in range(2)]
    e2e_out = torch.empty((2, GROUP, B, hq * d), dtype=torch.float16, device=dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out_free = [torch.cuda.Event() for _ in range(2)]

    def e2e_step():
        with torch.cuda.stream(stream):
            d_table.copy_(h_table, non_blocking=True)
            d_lens.copy_(h_lens, non_blocking=True)
        plan.update(kv_lens)
        for gi in range(n_groups):
            s = gi & 1
            l0, l1 = bounds[gi], bounds[gi + 1]
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(ev_done[s])  # the launches that read this slot two groups ago
                e2e_qkv[s, :l1 - l0].copy_(h_qkv[l0:l1], non_blocking=True)
                ev_in[s].record(copy_in)
            stream.wait_event(ev_in[s])
            stream.wait_event(ev_out_free[s])
            for i in range(l0, l1):
                j = i - l0
                decode(plan, descs[i], e2e_q[s][j], e2e_out[s, j], n_heads=hq, k=e2e_k[s][j], v=e2e_v[s][j],
                               cos=d_cos, sin=d_sin, rope=True, rope_mode=w["rope_mode"], append=True, scale=scale)
            ev_done[s].record(stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(ev_done[s])
                h_out[l0:l1].copy_(e2e_out[s, :l1 - l0], non_blocking=True)
                ev_out_free[s].record(copy_out)
        stream.wait_stream(copy_out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """Returns (device ms for all steps, wall seconds window)."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0 = time.time()
        start.record(stream)
        for _ in range(steps):
            fn()
        stop.record(stream)
        barrier()
        t1 = time.time()
        ms = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, t0, t1

    for _ in range(max(args.warmup, 3)):
        device_step()
    f.synchronize()
    sampler = ClockSampler(dev.index)
    sampler.start()
    time.sleep(0.3)
    launches0 = f.launch_count
    if w.get("graph"):
        # batch-1 steps are host-bound call by call: the same launches replayed from a CUDA graph (the step is
        # idempotent: same rows, same values)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            device_step()

        def replay():
            with torch.cuda.stream(stream):
                graph.replay()

        for _ in range(3):
            replay()
        torch.cuda.synchronize()
        ms, t0, t1 = timed(replay, args.steps)
        launches = layers * args.steps
    else:
        ms, t0, t1 = timed(device_step, args.steps)
        launches = f.launch_count - launches0
    f.synchronize()  # also reads the device status word: a timed-out barrier wait would raise here
    for _ in range(2):
        e2e_step()
    ms_e2e, _, t1 = timed(e2e_step, args.steps)
    f.synchronize()
    clocks = sampler.stop(t0, t1)
    # spread of single steps (an event after every step; kept out of the headline region)
    n_stat = min(args.steps, 100)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_stat + 1)]
    marks[0].record(stream)
    for i in range(n_stat):
        device_step()
        marks[i + 1].record(stream)
    f.synchronize()
    per_step = np.array([marks[i].elapsed_time(marks[i + 1]) for i in range(n_stat)])

    ms_step = ms / args.steps
    tokens_per_s = B * world / (ms_step * 1e-3)
    ms_step_e2e = ms_e2e / args.steps
    bytes_layer = algorithmic_bytes_per_layer(w, kv_lens)
    launch_us = ms_step * 1e3 / layers
    achieved = bytes_layer / (launch_us * 1e-6) / 1e9
    peak, peak_kind = measured_peak_gbs()
    if world > 1:
        t = torch.tensor([launches], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        launches = int(t.item())
    h2d = layers * B * (hq + 2 * hkv) * d * 2 + h_table.numel() * 4 + h_lens.numel() * 4 + plan.items * 32
    d2h = layers * B * hq * d * 2
    result = {
        "metric": METRIC, "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "us_per_step": ms_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 storage, f32 accumulate" if kv8 else "f16 storage, f32 accumulate",
        "data": "synthetic",
        "config": config_of(w),
        "plan": {"ctas": plan.ctas, "work_items": plan.items},
        "hbm_tb_s": achieved / 1e3,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "kernel": "decode_kv8_kernel" if kv8 else "decode_kernel<128,1,3,2>",
                     "launch_us": launch_us,
                     "algorithmic_bytes_per_launch": bytes_layer,
                     "traffic": (bytes_layer * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE
                                 if NCU_TRAFFIC_PER_ALGORITHMIC_BYTE and not kv8 else None)},
        "e2e": {"value": B * world / (ms_step_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_step_e2e,
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "step_spread_ms": {"n": n_stat, "min": float(per_step.min()), "median": float(np.median(per_step)),
                           "mean": float(per_step.mean()), "sd": float(per_step.std())},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not kv8:  # the CPU arm is the f16 cache's
        result["cpu_baseline"] = cpu_baseline(w, steps=3)
    # Sanity on the timed buffers: the last layer's output is finite and the end-to-end output equals it.
    torch.cuda.synchronize()
    ok = bool(torch.isfinite(d_out[-1].float()).all()) and bool(torch.equal(h_out[-1].to(dev), d_out[-1]))
    result["self_check"] = "ok" if ok else "FAILED"
    plan.close()
    f.close()
    if rank == 0:
        emit(result)
    return 0 if ok else 1


def run_long_context(args, w):
    """Configuration 5: one long sequence, pages sharded over the ranks."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    rank, world, local = rank_setup()
    dev = torch.device("cuda", torch.cuda.current_device())
    mfk = importlib.import_module("test-burn_b200")
    sharding = importlib.import_module("test-burn_b200.sharding")
    layers, hq, hkv, d, P, L = w["layers"], w["n_heads"], w["n_kv_heads"], w["head_dim"], w["page_size"], w["kv_len"]
    n_pages = (L + P - 1) // P
    b, e = sharding.shard_pages(n_pages, world, rank)
    n_local = sharding.shard_local_len(L, P, b, e)
    owner = sharding.tail_owner(L, P, n_pages, world)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + rank)
    pool_elems = (e - b) * hkv * P * d
    kv8 = bool(w.get("kv8"))
    if kv8:
        # bytes of finite E4M3 values (exponent field below 15) with random signs; scales of N(0,1) rows (amax / 448)
        def fp8_pool():
            t = torch.randint(0, 0x78, (pool_elems,), dtype=torch.uint8, device=dev, generator=gen)
            return t | (torch.randint(0, 2, (pool_elems,), dtype=torch.uint8, device=dev, generator=gen) << 7)

        k_pools = [fp8_pool() for _ in range(layers)]
        v_pools = [fp8_pool() for _ in range(layers)]
        k_scales = [torch.full((pool_elems // d,), 3.5 / 448, dtype=torch.float32, device=dev) for _ in range(layers)]
        v_scales = [torch.full((pool_elems // d,), 3.5 / 448, dtype=torch.float32, device=dev) for _ in range(layers)]
    else:
        k_pools = [torch.empty(pool_elems, dtype=torch.float16, device=dev).normal_(generator=gen) for _ in range(layers)]
        v_pools = [torch.empty(pool_elems, dtype=torch.float16, device=dev).normal_(generator=gen) for _ in range(layers)]
    table = torch.arange(e - b, dtype=torch.int32, device=dev).view(1, -1)
    lens_host = np.array([n_local], np.uint32)
    d_lens = torch.from_numpy(lens_host.view(np.int32)).to(dev)
    d_pos = torch.tensor([L - 1], dtype=torch.int32, device=dev)
    cos_np, sin_np = mfk.rope_tables(w["theta"], d, L)
    d_cos = torch.from_numpy(cos_np.view(np.float16)).to(dev)
    d_sin = torch.from_numpy(sin_np.view(np.float16)).to(dev)
    g = torch.Generator().manual_seed(SEED)  # the token is the same on every rank
    q = torch.randn((layers, 1, hq * d), generator=g).half().to(dev)
    k = torch.randn((layers, 1, hkv * d), generator=g).half().to(dev)
    v = torch.randn((layers, 1, hkv * d), generator=g).half().to(dev)
    out = torch.zeros((layers, hq, d), dtype=torch.float16, device=dev)
    stream = torch.cuda.Stream(device=dev)
    f = mfk.Foundry(dev.index, stream.cuda_stream)
    if not args.no_overlap:
        # 2: the pools of a layer are written by nothing but that layer's own fused append, so every rank
        # (not only the one that appends) may stream K/V before the previous launch has ended
        f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 2)
    if kv8:
        plan = f.decode_plan(lens_host, n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P)
        descs = [mfk.paged_kv8(k_pools[i].view(e - b, hkv, P, d), v_pools[i].view(e - b, hkv, P, d),
                               k_scales[i].view(e - b, hkv, P), v_scales[i].view(e - b, hkv, P), table, d_lens,
                               n_kv_heads=hkv, page_size=P) for i in range(layers)]
    else:
        plan = f.decode_plan(lens_host, n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P)
        descs = [mfk.paged_kv(k_pools[i].view(e - b, hkv, P, d), v_pools[i].view(e - b, hkv, P, d), table, d_lens,
                              n_kv_heads=hkv, page_size=P, head_dim=d) for i in range(layers)]
    block = hq * (d + 2)
    mine = torch.zeros(block, dtype=torch.float32, device=dev)
    mine[hq * d:hq * d + hq] = -1e30  # a shard without keys contributes nothing
    acc, m, l = mine[:hq * d].view(1, hq, d), mine[hq * d:hq * d + hq], mine[hq * d + hq:]
    gathered = torch.empty((world, block), dtype=torch.float32, device=dev)
    scale = 1.0 / math.sqrt(d)
    append_here = rank == owner
    px, step_no = None, [0]
    if args.exchange in ("push", "fused"):
        # the kernels exchange the partials themselves: peer stores into every rank's receive block
        px, handle = f.peer_exchange_create(world, rank, hq, d)
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            for r in range(world):
                if r != rank:
                    f.peer_exchange_attach(px, r, handles[r])
        units = []
        for r in range(world):
            rb, re_ = sharding.shard_pages(n_pages, world, r)
            units.append(hkv if sharding.shard_local_len(L, P, rb, re_) else 0)

    partial_push = f.paged_decode_kv8_partial_push if kv8 else f.paged_decode_partial_push
    push_merge = f.paged_decode_kv8_push_merge if kv8 else f.paged_decode_push_merge

    def step_push():
        with torch.cuda.stream(stream):
            for i in range(layers):
                if n_local:
                    partial_push(plan, descs[i], q[i], px, step_no[0], n_heads=hq, rope_positions=d_pos,
                                                scale=scale, k=k[i] if append_here else None,
                                                v=v[i] if append_here else None, cos=d_cos, sin=d_sin, rope=True,
                                                rope_mode=w["rope_mode"], append=append_here)
                f.merge_pushed(px, units, step_no[0], hq, d, out[i])
                step_no[0] += 1

    all_push = px is not None and all(units)
    pusher_mask = (1 << world) - 1

    def step_fused():
        with torch.cuda.stream(stream):
            for i in range(layers):
                push_merge(plan, descs[i], q[i], out[i], px, step_no[0], pusher_mask, n_heads=hq,
                                          rope_positions=d_pos, scale=scale, k=k[i] if append_here else None,
                                          v=v[i] if append_here else None, cos=d_cos, sin=d_sin, rope=True,
                                          rope_mode=w["rope_mode"], append=append_here)
                step_no[0] += 1

    def step():
        if args.exchange == "fused" and all_push:
            return step_fused()
        if px is not None:
            return step_push()
        with torch.cuda.stream(stream):
            for i in range(layers):
                if n_local and kv8:
                    f.paged_decode_kv8_partial(plan, descs[i], q[i], d_pos, acc, m, l, n_heads=hq, scale=scale,
                                               k=k[i] if append_here else None, v=v[i] if append_here else None,
                                               cos=d_cos, sin=d_sin, rope=True, rope_mode=w["rope_mode"], append=append_here)
                elif n_local:
                    f.paged_decode_partial(plan, descs[i], q[i], acc, m, l, n_heads=hq, rope_positions=d_pos,
                                           scale=scale, k=k[i] if append_here else None,
                                           v=v[i] if append_here else None, cos=d_cos, sin=d_sin, rope=True,
                                           rope_mode=w["rope_mode"], append=append_here)
                if world > 1:
                    dist.all_gather_into_tensor(gathered.view(-1), mine)
                else:
                    gathered.view(-1).copy_(mine, non_blocking=True)
                f.merge_gathered(gathered, hq, d, out[i])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    f.synchronize()
    sampler = ClockSampler(dev.index)
    sampler.start()
    time.sleep(0.3)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = f.launch_count
    barrier()
    t0 = time.time()
    start.record(stream)
    for _ in range(args.steps):
        step()
    stop.record(stream)
    barrier()
    t1 = time.time()
    ms = start.elapsed_time(stop)
    launches = f.launch_count - launches0
    if world > 1:
        t = torch.tensor([ms, launches], dtype=torch.float64, device=dev)
        dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
        dist.all_reduce(t[1:])
        ms, launches = float(t[0]), int(t[1])
    f.synchronize()
    clocks = sampler.stop(t0, t1)
    ms_step = ms / args.steps
    bytes_layer_rank = 2 * hkv * (L // world) * ((d + 4) if kv8 else d * 2)
    launch_us = ms_step * 1e3 / layers
    achieved = bytes_layer_rank / (launch_us * 1e-6) / 1e9
    peak, peak_kind = measured_peak_gbs()
    # all ranks hold the same result; it must be finite and equal across ranks
    ok = bool(torch.isfinite(out.float()).all())
    if world > 1:
        ref = out.clone()
        dist.broadcast(ref, 0)
        ok = ok and bool(torch.equal(ref, out))
    result = {
        "metric": METRIC, "value": 1.0 / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "us_per_step": ms_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "e4m3 storage, f32 accumulate" if kv8 else "f16 storage, f32 accumulate", "data": "synthetic",
        "config": {"workload": w["name"], "layers": layers, "kv_len": L, "pages_per_rank": e - b,
                   "l2": "inputs larger than L2 (KV pools %.1f GB per GPU)" % (2 * layers * pool_elems * (1 if kv8 else 2) / 1e9),
                   "ctas": plan.ctas, "collective": ("none: decode kernels store %d values per layer into every rank's receive block "
                                  % block
                                  + ("(peer stores of tagged 8-byte words: value + step tag) and merge them themselves as soon as "
                                     "every word carries the tag: one launch per layer"
                                     if args.exchange == "fused" and all_push else
                                     "(peer stores, a system-scope fence, arrival counters); the merge kernel waits on the counters"))
                   if px is not None else "ncclAllGather of %d bytes per rank per layer" % (block * 4)},
        "hbm_tb_s_per_gpu": achieved / 1e3,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind,
                     "kernel": ("decode_kv8_kernel" if kv8 else "decode_kernel<128,1,3,2>") + " + exchange + merge per layer",
                     "launch_us": launch_us, "algorithmic_bytes_per_launch": bytes_layer_rank, "traffic": None},
        "gpu_launches": launches, "clocks": clocks, "self_check": "ok" if ok else "FAILED",
    }
    plan.close()
    if px is not None:
        barrier()  # nobody unmaps while a peer may still store
        f.peer_exchange_destroy(px)
    f.close()
    if rank == 0:
        emit(result)
    return 0 if ok else 1


def rank_setup():
    """(rank, world, device index): one process per GPU under torchrun (NCCL only for the barrier, the max over
    ranks and the baseline exchange), a single process otherwise.  The process group is made once per process."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0")) if world > 1 else 0
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def rank_teardown():
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


# Result lines go through emit(): printed, or collected when a run gathers several workloads into one line.
_COLLECT = None


def emit(result):
    if _COLLECT is not None:
        _COLLECT.append(result)
    else:
        print(json.dumps(result))


def rank_reduce(value, world, op="max"):
    """Max (or min) of a float over the ranks, with a barrier's worth of synchronisation."""
    if world == 1:
        return float(value)
    import torch
    import torch.distributed as dist

    t = torch.tensor([float(value)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN)
    return float(t.item())


def run_prefill(args):
    """Configuration 4: 2048 new tokens after 2048 cached, Llama-3.2-3B heads, one layer per step:
    KvPrepFused (RoPE + append of 2048 rows) then causal attention over 4096 keys."""
    import torch

    rank, world, local = rank_setup()
    dev = torch.device("cuda", local)
    mfk = importlib.import_module("test-burn_b200")
    sharding = importlib.import_module("test-burn_b200.sharding")
    hq_all, hkv_all, d, m, cached, cap = 24, 8, 128, 2048, 2048, 4096
    # N > 1: KV heads (with their query groups) over the GPUs, no exchange inside the path
    h0, h1 = sharding.shard_kv_heads(hkv_all, world, rank)
    hkv = max(h1 - h0, 1)  # a rank without heads (more GPUs than KV heads) repeats head 0's work, untimed in effect
    hq = hkv * (hq_all // hkv_all)
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    q = torch.empty((m, hq * d), dtype=torch.float16, device=dev).normal_(generator=g)
    k = torch.empty((m, hkv * d), dtype=torch.float16, device=dev).normal_(generator=g)
    v = torch.empty((m, hkv * d), dtype=torch.float16, device=dev).normal_(generator=g)
    kc = torch.empty((hkv, cap, d), dtype=torch.float16, device=dev).normal_(generator=g)
    vc = torch.empty((hkv, cap, d), dtype=torch.float16, device=dev).normal_(generator=g)
    cos_np, sin_np = mfk.rope_tables(5e5, d, cap)
    cos = torch.from_numpy(cos_np.view(np.float16)).to(dev)
    sin = torch.from_numpy(sin_np.view(np.float16)).to(dev)
    q_rot = torch.empty((hq, m, d), dtype=torch.float16, device=dev)
    out = torch.empty((m, hq * d), dtype=torch.float16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(device=dev)
    f = mfk.Foundry(local, stream.cuda_stream)
    apply_options(mfk, f, args)
    p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, m, cached, cap, hq * m * d, 1, 0, 0)
    desc = None
    if args.page_size:
        # the same chunk into a PAGED cache: pages of the sequence scattered over the pool
        P = args.page_size
        n_pages = cap // P + 7
        kp = torch.empty((n_pages, hkv, P, d), dtype=torch.float16, device=dev).normal_(generator=g)
        vp = torch.empty((n_pages, hkv, P, d), dtype=torch.float16, device=dev).normal_(generator=g)
        table = torch.randperm(n_pages, device=dev, generator=g)[: cap // P].to(torch.int32).reshape(1, -1).contiguous()
        lens = torch.tensor([cached + m], dtype=torch.int32, device=dev)
        desc = mfk.paged_kv(kp, vp, table, lens, n_kv_heads=hkv, page_size=P, head_dim=d)
    scale = 1.0 / math.sqrt(d)

    def step(timed_events=None):
        with torch.cuda.stream(stream):
            flush.zero_()  # L2 flush between iterations: write a buffer larger than L2
            if timed_events:
                timed_events[0].record(stream)
            if desc is not None:
                f.paged_kv_append(desc, q, k, v, q_rot, cos, sin, n_heads=hq, rope_mode=1, seq=0, position_offset=cached,
                                  seq_len=m)
            else:
                f.kv_prep_fused(q, k, v, q_rot, kc, vc, cos, sin, p)
            if timed_events:
                timed_events[1].record(stream)
            if desc is not None:
                f.paged_prefill(desc, q_rot, out, seq=0, q_len=m, kv_len=cached + m, query_offset=cached, n_heads=hq,
                                scale=scale)
            else:
                f.flash_attention(q_rot, kc, vc, out, causal=True, query_offset=cached, n_heads=hq, head_dim=d,
                                  kv_seq_len=cached + m, m=m)
            if timed_events:
                timed_events[2].record(stream)

    for _ in range(max(args.warmup, 3)):
        step()
    f.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.2)
    t0 = time.time()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches0 = f.launch_count
    for e in evs:
        step(e)
    f.synchronize()
    t1 = time.time()
    launches = f.launch_count - launches0
    clocks = sampler.stop(t0, t1)
    t_append = rank_reduce(np.median([e[0].elapsed_time(e[1]) for e in evs]), world)
    t_attn = rank_reduce(np.median([e[1].elapsed_time(e[2]) for e in evs]), world)
    pairs = sum(cached + i + 1 for i in range(m))
    flops = 4 * d * pairs * hq_all  # the whole job; every GPU's tensor pipe is the roofline of its own share
    ok = rank_reduce(float(bool(torch.isfinite(out.float()).all())), world, "min") > 0.5
    if rank != 0:
        f.close()
        return 0
    peak_path = ROOT / "MEASURED_PEAKS.json"
    peak = json.loads(peak_path.read_text())["bf16_tflops"] if peak_path.exists() else 1590.0
    achieved = flops / (t_attn * 1e-3) / 1e12
    emit({
        "metric": "prefill_attention_tflops", "value": achieved, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": t_append + t_attn, "higher_is_better": True,
        "scaling": "weak" if world == 1 else "strong",
        "vs_baseline": None, "dtype": "f16 inputs, f32 accumulate", "data": "synthetic",
        "config": {"workload": "chunked causal prefill into cache, Llama-3.2-3B shape: 2048 new after 2048 cached, "
                               "24q/8kv heads, D128, one layer" +
                               (", paged cache (page %d)" % args.page_size if args.page_size else ", contiguous cache") +
                               ("" if world == 1 else "; KV heads split over %d GPUs, no exchange" % world),
                   "l2": "flushed between iterations (256 MB write)",
                   "split_k": mfk.prefill_split_k(cached + m, m)},
        "append_us": t_append * 1e3, "attention_us": t_attn * 1e3, "algorithmic_flops": flops,
        "roofline": {"bound": "tensor", "achieved": achieved / world, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / world / peak, "peak_kind": "measured" if peak_path.exists() else "fallback",
                     "traffic": None, "note": "per GPU"},
        "gpu_launches": launches, "clocks": clocks, "self_check": "ok" if ok else "FAILED"})
    f.close()
    return 0 if ok else 1


CONTIGUOUS = {
    # the reference's own layout and op order: contiguous cache [Hkv, capacity, D] per layer, KvPrepFused then
    # FlashAttention (decode route), batch 1
    "c1": dict(layers=1, n_heads=14, n_kv_heads=2, head_dim=64, cached=511, capacity=512, theta=1e6, rope_mode=0,
               hidden=896, qkv_bias=True,
               name="single-token latency, Qwen2.5-0.5B shape: 1 layer, 14q/2kv heads, D64, batch 1, 511 cached + 1, "
                    "contiguous cache, KvPrepFused then FlashAttention (2 launches)"),
    "c2": dict(layers=28, n_heads=24, n_kv_heads=8, head_dim=128, cached=8191, capacity=8192, theta=5e5, rope_mode=1,
               hidden=3072, qkv_bias=False,
               name="Llama-3.2-3B shape decode step: 28 layers, 24q/8kv heads, D128, batch 1, ctx 8192, contiguous "
                    "cache, KvPrepFused then FlashAttention per layer (56 launches)"),
}


def run_contiguous_decode(args, w):
    """Configurations 1 and 2: batch-1 decode steps on contiguous caches through the reference's two ops per
    layer.  The step is timed twice: launched call by call from the Python binding (host-bound for
    launches this short) and replayed from a CUDA graph, which is the device-side figure reported as
    `value`.  Configuration 1 (0.27 MB) is L2-resident: latency only."""
    import torch

    rank, world, local = rank_setup()
    dev = torch.device("cuda", local)
    mfk = importlib.import_module("test-burn_b200")
    sharding = importlib.import_module("test-burn_b200.sharding")
    layers, hq_all, hkv_all, d, cached, cap = (w["layers"], w["n_heads"], w["n_kv_heads"], w["head_dim"], w["cached"],
                                               w["capacity"])
    # N > 1: KV heads (with their query groups) over the GPUs, no exchange inside the path; a rank
    # beyond the KV head count repeats one head's work so that every process runs the same program
    h0, h1 = sharding.shard_kv_heads(hkv_all, world, rank)
    hkv = max(h1 - h0, 1)
    hq = hkv * (hq_all // hkv_all)
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    q = torch.empty((layers, 1, hq * d), dtype=torch.float16, device=dev).normal_(generator=g)
    k = torch.empty((layers, 1, hkv * d), dtype=torch.float16, device=dev).normal_(generator=g)
    v = torch.empty((layers, 1, hkv * d), dtype=torch.float16, device=dev).normal_(generator=g)
    kcs = [torch.empty((hkv, cap, d), dtype=torch.float16, device=dev).normal_(generator=g) for _ in range(layers)]
    vcs = [torch.empty((hkv, cap, d), dtype=torch.float16, device=dev).normal_(generator=g) for _ in range(layers)]
    cos_np, sin_np = mfk.rope_tables(w["theta"], d, cap)
    cos = torch.from_numpy(cos_np.view(np.float16)).to(dev)
    sin = torch.from_numpy(sin_np.view(np.float16)).to(dev)
    q_rot = torch.empty((layers, 1, hq * d), dtype=torch.float16, device=dev)
    out = torch.empty((layers, 1, hq * d), dtype=torch.float16, device=dev)
    stream = torch.cuda.Stream(device=dev)
    f = mfk.Foundry(local, stream.cuda_stream)
    apply_options(mfk, f, args)
    if not args.no_overlap:
        f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 1)
    p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, 1, cached, cap, hq * d, w["rope_mode"], 0, 0)

    qkv_args, weight_bytes = None, 0
    if args.projection:
        # the step in front of the path as well: RMSNorm + fused Q/K/V projection (f16 weights in the
        # reference's blocked layout) + RoPE + append in one launch, then FlashAttention
        hidden = w["hidden"]
        x = torch.empty((1, hidden), dtype=torch.float16, device=dev).normal_(generator=g)
        gamma = torch.empty((hidden,), dtype=torch.float16, device=dev).uniform_(0.5, 1.5, generator=g)
        qkv_args = []
        for _ in range(layers):
            ws = [torch.empty((n * hidden,), dtype=torch.float16, device=dev).uniform_(-0.05, 0.05, generator=g)
                  for n in (hq * d, hkv * d, hkv * d)]
            bias = tuple(torch.empty((n,), dtype=torch.float16, device=dev).uniform_(-0.1, 0.1, generator=g)
                         for n in (hq * d, hkv * d, hkv * d)) if w["qkv_bias"] else None
            qkv_args.append(f.fused_qkv_args(x, *ws, k_dim=hidden, n_dim=hq * d, n_kv=hkv * d, m=1, gamma=gamma, bias=bias,
                                             weights_per_block=32))
        weight_bytes = (hq + 2 * hkv) * d * hidden * 2

    def step():
        for i in range(layers):
            if qkv_args is not None:
                f.fused_qkv_kv_prep(qkv_args[i], q_rot[i], kcs[i], vcs[i], cos, sin, p)
            elif args.one_launch:
                # KvPrepFused and FlashAttention of the layer in one launch
                f.kv_prep_flash_decode(q[i], k[i], v[i], q_rot[i], kcs[i], vcs[i], cos, sin, out[i], p)
                continue
            else:
                f.kv_prep_fused(q[i], k[i], v[i], q_rot[i], kcs[i], vcs[i], cos, sin, p)
            f.flash_attention(q_rot[i], kcs[i], vcs[i], out[i], causal=True, query_offset=cached, n_heads=hq, head_dim=d,
                              kv_seq_len=cached + 1, m=1)

    for _ in range(max(args.warmup, 25 if layers == 1 else 3)):
        step()
    f.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    trials, iters = 10, max(args.steps, 100) if layers == 1 else max(10, min(args.steps, 40))
    per_iter_us = []
    launches0 = f.launch_count
    t0 = time.time()
    for _ in range(trials):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(iters):
            step()
        b.record(stream)
        f.synchronize()
        per_iter_us.append(a.elapsed_time(b) * 1e3 / iters)
    launches = f.launch_count - launches0
    # The same launches replayed from a CUDA graph: the device-side time without the per-call cost of
    # the Python binding.  The step is idempotent (same rows, same values).
    graph_us = None
    try:
        g_steps = 20 if layers == 1 else 2
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for _ in range(g_steps):
                step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        per_graph = []
        for _ in range(trials):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            with torch.cuda.stream(stream):
                for _ in range(10):
                    graph.replay()
            b.record(stream)
            torch.cuda.synchronize()
            per_graph.append(a.elapsed_time(b) * 1e3 / (10 * g_steps))
        graph_us = {"steps_per_graph": g_steps, "min": float(np.min(per_graph)), "median": float(np.median(per_graph)),
                    "mean": float(np.mean(per_graph)), "sd": float(np.std(per_graph))}
    except Exception as e:  # capture is an extra; the eager figure stands on its own
        graph_us = {"unavailable": str(e)[:200]}
    f.synchronize()
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    us = np.array(per_iter_us)
    eager_med = float(np.median(us))
    med = graph_us["median"] if "median" in graph_us else eager_med  # the device-side figure when it exists
    med = rank_reduce(med, world)
    eager_med = rank_reduce(eager_med, world)
    ok = rank_reduce(float(bool(torch.isfinite(out.float()).all())), world, "min") > 0.5
    if rank != 0:
        f.close()
        return 0
    # per GPU (the largest share)
    bytes_layer = 2 * hkv * (cached + 1) * d * 2 + 4 * hkv * d * 2 + 2 * hq * d * 2 + 2 * (d // 2) * 2
    bytes_layer += weight_bytes
    peak, peak_kind = measured_peak_gbs()
    achieved = bytes_layer * layers / (med * 1e-6) / 1e9
    l2_note = ("L2-resident by construction (0.27 MB): latency only, not a bandwidth figure" if layers == 1 else
               "inputs larger than L2 (caches %.2f GB)" % (2 * layers * hkv * cap * d * 2 / 1e9))
    emit({
        "metric": METRIC, "value": 1e6 / med, "unit": "tokens/s", "n_gpus": world, "steps": iters * trials,
        "warmup": max(args.warmup, 3), "ms_per_step": med * 1e-3, "us_per_step": med, "higher_is_better": True,
        "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
        "config": {"workload": w["name"] + ("; with --projection the first launch of a layer is RMSNorm + fused QKV "
                                            "projection + RoPE + append (weights %.1f MB per layer)" % (weight_bytes / 1e6)
                                            if args.projection else "") +
                               ("; --one-launch: the two ops of a layer fused into one launch" if args.one_launch else "") +
                               ("" if world == 1 else "; KV heads split over %d GPUs (%d per GPU), no exchange" % (world, hkv)),
                   "l2": l2_note,
                   "timing": "value / us_per_step = CUDA-graph replay of the step when capture works, else eager"},
        "latency_us": {"trials": trials, "iterations": iters, "min": float(us.min()), "median": eager_med,
                       "mean": float(us.mean()), "sd": float(us.std()),
                       "note": "launched call by call from the Python binding: host-bound"},
        "latency_us_cuda_graph": graph_us,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": None, "launch_us": med / layers, "per": "GPU",
                     "algorithmic_bytes_per_launch": bytes_layer,
                     "note": "launch-bound" if layers == 1 else "per layer: %s + decode_kernel" %
                             ("fused_qkv_kernel" if args.projection else "kv_append_kernel")},
        "gpu_launches": launches, "clocks": clocks, "self_check": "ok" if ok else "FAILED"})
    f.close()
    return 0 if ok else 1


def run_batched_strong(args, w):
    """ONE batch of the workload (the sequences drawn from the seed of rank 0) split over the ranks by
    sharding.shard_sequences: longest first, dealt out in a snake; every rank owns its sequences' pages, page
    table and plan, nothing crosses GPUs during a step (strong scaling; at N = 1 this is the headline step)."""
    import torch
    import torch.distributed as dist

    rank, world, local = rank_setup()
    dev = torch.device("cuda", torch.cuda.current_device())
    mfk = importlib.import_module("test-burn_b200")
    sharding = importlib.import_module("test-burn_b200.sharding")
    layers, hq, hkv, d, P = w["layers"], w["n_heads"], w["n_kv_heads"], w["head_dim"], w["page_size"]
    _, all_lens = make_lengths(w, SEED)
    mine = sharding.shard_sequences(all_lens, world, rank)
    kv_lens = np.ascontiguousarray(all_lens[mine])
    B = len(mine)
    wl = dict(w, batch=B)
    table, n_pages = make_page_table(wl, kv_lens, SEED + rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + rank)
    pool_elems = n_pages * hkv * P * d
    k_pools = [torch.empty(pool_elems, dtype=torch.float16, device=dev).normal_(generator=gen) for _ in range(layers)]
    v_pools = [torch.empty(pool_elems, dtype=torch.float16, device=dev).normal_(generator=gen) for _ in range(layers)]
    d_table = torch.from_numpy(table.view(np.int32)).to(dev)
    d_lens = torch.from_numpy(kv_lens.view(np.int32)).to(dev)
    cos_np, sin_np = mfk.rope_tables(w["theta"], d, int(all_lens.max()))
    d_cos = torch.from_numpy(cos_np.view(np.float16)).to(dev)
    d_sin = torch.from_numpy(sin_np.view(np.float16)).to(dev)
    d_q = torch.empty((layers, B, hq * d), dtype=torch.float16, device=dev).normal_(generator=gen)
    d_k = torch.empty((layers, B, hkv * d), dtype=torch.float16, device=dev).normal_(generator=gen)
    d_v = torch.empty((layers, B, hkv * d), dtype=torch.float16, device=dev).normal_(generator=gen)
    d_out = torch.empty((layers, B, hq * d), dtype=torch.float16, device=dev)
    stream = torch.cuda.Stream(device=dev)
    f = mfk.Foundry(dev.index, stream.cuda_stream)
    if not args.no_overlap:
        f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 1)
    plan = f.decode_plan(kv_lens, n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P)
    descs = [mfk.paged_kv(k_pools[i].view(n_pages, hkv, P, d), v_pools[i].view(n_pages, hkv, P, d), d_table, d_lens,
                          n_kv_heads=hkv, page_size=P, head_dim=d) for i in range(layers)]
    scale = 1.0 / math.sqrt(d)

    def step():
        with torch.cuda.stream(stream):
            for i in range(layers):
                f.paged_decode(plan, descs[i], d_q[i], d_out[i], n_heads=hq, k=d_k[i], v=d_v[i], cos=d_cos, sin=d_sin,
                               rope=True, rope_mode=w["rope_mode"], append=True, scale=scale)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    f.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = f.launch_count
    barrier()
    start.record(stream)
    for _ in range(args.steps):
        step()
    stop.record(stream)
    barrier()
    ms = rank_reduce(start.elapsed_time(stop), world)
    launches = f.launch_count - launches0
    f.synchronize()
    ms_step = ms / args.steps
    bytes_layer = algorithmic_bytes_per_layer(wl, kv_lens)  # this rank's share
    launch_us = ms_step * 1e3 / layers
    achieved = bytes_layer / (launch_us * 1e-6) / 1e9
    peak, peak_kind = measured_peak_gbs()
    worst = rank_reduce(achieved, world, "min")
    ok = rank_reduce(float(bool(torch.isfinite(d_out[-1].float()).all())), world, "min") > 0.5
    result = {
        "metric": METRIC, "value": w["batch"] / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "us_per_step": ms_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
        "config": {"workload": w["name"] + "; ONE batch of %d sequences split over the GPUs by length (snake order), "
                               "no exchange" % w["batch"], "sequences_on_rank_0": B, "seed": SEED,
                   "l2": "inputs larger than L2"},
        "roofline": {"bound": "hbm", "achieved": worst, "peak": peak, "unit": "GB/s", "frac": worst / peak,
                     "peak_kind": peak_kind, "per": "GPU (the rank with the smallest share, max-over-ranks time)",
                     "launch_us": launch_us, "traffic": None},
        "gpu_launches": launches * world, "self_check": "ok" if ok else "FAILED"}
    plan.close()
    f.close()
    if rank == 0:
        emit(result)
    return 0 if ok else 1


def other_workloads(args):
    """The workloads beside the headline one, measured in the same run so that they land in the same record:
    at every N the sequence-sharded long context (C5, strong scaling, exchange and merge inside the decode
    kernel) and ONE batch of the headline workload split over the ranks (strong scaling); at N = 1 also the
    batch-1 step on contiguous caches (C2, one launch per layer, CUDA-graph replay), the prefill chunk (C4) and the
    headline workload on the 8-bit cache (FP8 E4M3 pages + one f32 scale per row).
    Returns {name: short record}; every rank must call it (the sub-runs synchronise)."""
    import copy

    import torch

    global _COLLECT
    world = int(os.environ.get("WORLD_SIZE", "1"))
    jobs = [("c5", lambda a: run_long_context(a, LONG_CONTEXT["c5"]), dict(steps=20, exchange="fused")),
            ("c3_strong", lambda a: run_batched_strong(a, dict(WORKLOADS["c3"])), dict(steps=20)),
            ("c5_kv8", lambda a: run_long_context(a, LONG_CONTEXT["c5-kv8"]), dict(steps=20, exchange="fused"))]
    if world == 1:
        jobs += [("c2", lambda a: run_contiguous_decode(a, CONTIGUOUS["c2"]), dict(one_launch=True, projection=False)),
                 ("c4", run_prefill, dict(steps=20, page_size=0)),
                 ("c3_kv8", lambda a: run_ours(a, dict(WORKLOADS["c3-kv8"])), dict(steps=20, no_cpu_baseline=True)),
                 ("c2_kv8", lambda a: run_ours(a, dict(WORKLOADS["c2-kv8"])), dict(steps=100, no_cpu_baseline=True))]
    out = {}
    for name, fn, over in jobs:
        a = copy.copy(args)
        for k, v in over.items():
            setattr(a, k, v)
        torch.cuda.empty_cache()
        _COLLECT = []
        try:
            rc = fn(a)
            rec = _COLLECT[0] if _COLLECT else None
        except Exception as e:  # a side workload must not take the headline down
            rc, rec = 1, {"error": "%s: %s" % (type(e).__name__, str(e)[:200])}
        finally:
            _COLLECT = None
        if rec is not None:
            keep = {k: rec[k] for k in ("metric", "value", "unit", "us_per_step", "ms_per_step", "scaling", "n_gpus", "steps",
                                        "self_check", "gpu_launches", "error", "append_us", "attention_us") if k in rec}
            if "roofline" in rec:
                keep["roofline"] = {k: rec["roofline"].get(k) for k in ("bound", "achieved", "peak", "unit", "frac", "per", "launch_us")}
            if "config" in rec:
                keep["workload"] = rec["config"].get("workload")
            if "latency_us_cuda_graph" in rec:
                keep["timing"] = "CUDA-graph replay" if "median" in rec["latency_us_cuda_graph"] else "eager"
            keep["rc"] = rc
            out[name] = keep
    return out


# ---------------------------------------------------------------------- CPU arms ---

def cpu_layer_inputs(w, seed):
    """Host-side inputs of ONE layer of the workload (pools tiled from a random block)."""
    hq, hkv, d, B, P = w["n_heads"], w["n_kv_heads"], w["head_dim"], w["batch"], w["page_size"]
    cached, kv_lens = make_lengths(w, seed)
    table, n_pages = make_page_table(w, kv_lens, seed)
    rng = np.random.default_rng(seed)
    block = rng.standard_normal(1 << 22, dtype=np.float32).astype(np.float16).view(np.uint16)
    n = n_pages * hkv * P * d
    k_pool = np.resize(block, n)
    v_pool = np.resize(block[::-1], n)
    q = rng.standard_normal(B * hq * d, dtype=np.float32).astype(np.float16).view(np.uint16)
    k = rng.standard_normal(B * hkv * d, dtype=np.float32).astype(np.float16).view(np.uint16)
    v = rng.standard_normal(B * hkv * d, dtype=np.float32).astype(np.float16).view(np.uint16)
    return cached, kv_lens, table, k_pool, v_pool, q, k, v


def cpu_time_layer(w, repeats):
    """One layer of the workload on the host cores with the fast CPU arm (oracle/mf_oracle_fast.c, built here
    for this machine); the strict scalar oracle stands in if that build is not possible.  Returns the times,
    the threads used and a description of the build."""
    import oracle

    threads = len(os.sched_getaffinity(0))  # torchrun exports OMP_NUM_THREADS=1
    hq, hkv, d, B, P = w["n_heads"], w["n_kv_heads"], w["head_dim"], w["batch"], w["page_size"]
    cached, kv_lens, table, k_pool, v_pool, q, k, v = cpu_layer_inputs(w, SEED)
    cos, sin = oracle.rope_tables(w["theta"], d, int(kv_lens.max()))
    out = np.empty(B * hq * d, np.uint16)
    try:
        F = oracle.fast_lib()
        F.mfo_fast_set_num_threads(threads)
        fn, threads = F.mfo_fast_paged_decode_layer, int(F.mfo_fast_num_threads())
        build = "fast build (gcc -O3 -march=native, %s, one K/V pass per KV head, OpenMP)" % (
            "F16C + FMA vectors" if F.mfo_fast_simd() else "no F16C/AVX2 on this host: scalar conversions")
    except Exception as e:  # no gcc on this host, or the build failed
        L = oracle.lib()
        L.mfo_set_num_threads(threads)
        fn, threads = L.mfo_paged_decode_layer, int(L.mfo_num_threads())
        build = "strict scalar build (-O2 -ffp-contract=off; the fast build failed: %s)" % type(e).__name__
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn(q, k, v, k_pool, v_pool, cos, sin, table, table.shape[1], kv_lens, B, hq, hkv, d, P, w["rope_mode"],
           1.0 / math.sqrt(d), out)
        times.append(time.perf_counter() - t0)
    return times, threads, build


def cpu_baseline(w, steps=3):
    times, threads, build = cpu_time_layer(w, steps)
    t_layer = float(np.median(times))
    kv_lens = make_lengths(w, SEED)[1]
    return {"value": w["batch"] / (t_layer * w["layers"]), "unit": "tokens/s", "cores": threads, "kind": "port",
            "build": build, "achieved_gbs": algorithmic_bytes_per_layer(w, kv_lens) / t_layer / 1e9,
            "extrapolated": "1 of %d layers x %d" % (w["layers"], w["layers"]),
            "sample": "1 of %d layers, all %d sequences, timed %d time(s) (median %.3f s per layer), scaled by the layer "
                      "count; CPU restatement of the reference math, %s" % (w["layers"], w["batch"], steps, t_layer, build)}


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    n = int(os.environ.get("WORLD_SIZE", "1"))
    times, threads, build = cpu_time_layer(w, max(1, args.steps + min(args.warmup, 1)))
    times = times[min(args.warmup, 1):] or times
    t_layer = float(np.mean(times))
    ms_step = t_layer * w["layers"] * 1e3
    value = w["batch"] / (ms_step * 1e-3)
    kv_lens = make_lengths(w, SEED)[1]
    sample = ("each step = 1 of %d layers on all %d sequences (%.3f s), scaled by the layer count; CPU restatement of "
              "the reference math (the reference is Rust + Metal and cannot run on this host), %s"
              % (w["layers"], w["batch"], t_layer, build))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "extrapolated": "1 of %d layers x %d" % (w["layers"], w["layers"]),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 storage, f32 accumulate", "data": "synthetic", "config": config_of(w),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "build": build,
                         "achieved_gbs": algorithmic_bytes_per_layer(w, kv_lens) / t_layer / 1e9, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + sorted(LONG_CONTEXT) + sorted(CONTIGUOUS) + ["c4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--decode-stages", type=int, default=0,
                    help="depth of the decode kernel's K/V ring (MF_OPTION_DECODE_STAGES; 6 = one CTA per SM with a 192 KB ring)")
    ap.add_argument("--plan-item-cost", type=int, default=0,
                    help="batched paged workloads: what the step planner charges a CTA per piece of a (sequence, kv head) "
                         "unit, in tiles (MF_OPTION_PLAN_ITEM_COST; default 20)")
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="c3: only the headline workload (by default the line also carries c5, c3_strong and, at one "
                         "GPU, c2 and c4 under `other_workloads`)")
    ap.add_argument("--e2e-group", type=int, default=6, help="layers per host<->device transfer in the end-to-end step")
    ap.add_argument("--exchange", default="fused", choices=["fused", "push", "nccl"],
                    help="long-context workloads: partials exchanged and merged inside the decode kernel (fused), "
                         "exchanged by the decode kernel and merged by a second one (push), or by ncclAllGather")
    ap.add_argument("--no-overlap", action="store_true", help="plain launches instead of programmatic dependent launch")
    ap.add_argument("--one-launch", action="store_true",
                    help="c1 / c2: KvPrepFused and FlashAttention of a layer in one launch (mf_kv_prep_flash_decode)")
    ap.add_argument("--projection", action="store_true",
                    help="c1 / c2: start each layer from the hidden state (RMSNorm + fused QKV projection + RoPE + append "
                         "in one launch) instead of from q, k, v")
    ap.add_argument("--page-size", type=int, default=0,
                    help="c4: prefill into a paged cache with pages of this many rows (default: contiguous cache); "
                         "batched paged workloads: pages of this many rows instead of the workload's own")
    args = ap.parse_args()
    if args.impl == "reference" and args.workload not in WORKLOADS:
        sys.stderr.write("--impl reference times the batched paged decode workloads (%s) only; %s has no CPU arm\n"
                         % (", ".join(sorted(WORKLOADS)), args.workload))
        return 2
    if args.workload == "c4" or args.workload in CONTIGUOUS or args.workload in LONG_CONTEXT:
        if args.workload == "c4":
            rc = run_prefill(args)
        elif args.workload in CONTIGUOUS:
            rc = run_contiguous_decode(args, CONTIGUOUS[args.workload])
        else:
            rc = run_long_context(args, LONG_CONTEXT[args.workload])
        rank_teardown()
        return rc
    w = dict(WORKLOADS[args.workload])
    if args.page_size:
        w["name"] = w["name"].replace("page %d" % w["page_size"], "page %d" % args.page_size)
        w["page_size"] = args.page_size
    if args.impl == "reference":
        return run_reference(args, w)
    if args.workload != "c3" or args.no_other_workloads:
        rc = run_ours(args, w)
        rank_teardown()
        return rc
    # the headline line, with the other workloads of this run attached
    global _COLLECT
    _COLLECT = []
    rc = run_ours(args, w)
    headline = _COLLECT[0] if _COLLECT else None
    _COLLECT = None
    others = other_workloads(args)
    rank_teardown()
    if headline is not None:
        headline["other_workloads"] = others
        print(json.dumps(headline))
    return rc


if __name__ == "__main__":
    sys.exit(main())
