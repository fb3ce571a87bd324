#!/usr/bin/env python
"""Benchmark of the tree-attention decode operator.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3] [--impl reference]

A step is one call of flash_decoding_attention on one synthetic job.  At N GPUs (one process per
GPU under torch.distributed.run) ONE job is partitioned, never replicated:

  batched jobs (cfg2, cfg3, cfg5)   the job's sequences are dealt to the ranks by total KV length
                                    (dist.shard_batch); every (sequence, KV head) is independent,
                                    so there is no collective on the data path
  one long sequence (cfg4)          a contiguous KV range per rank, partial (O, LSE) per rank, one
                                    exchange-merge kernel per rank over peer-mapped memory
                                    (--exchange nccl: one all-gather + merge kernel)

so scaling is strong: value = calls of the WHOLE job per second of the slowest rank.  Prints ONE
JSON line (rank 0).  The headline workload is --workload (default cfg3); `per_config` carries the
same measurements for the other performance configurations.

Keys beyond the basic contract:
  roofline      dominant kernel (stage 1) of the slowest rank: algorithmic KV bytes (or flops) of
                its launch / its CUDA-event duration, against the measured peak
  cpu_baseline  the fp32 CPU oracle timed on this box's host cores (reported baseline only)
  e2e           same metric through the public Python call with the step's inputs (q, tree K/V,
                mask, lengths) copied from pinned host memory and the result copied back inside
                the timed region; median of 5 regions of K steps; the KV cache, which is decode
                state that lives in HBM across steps, is resident
  max_abs_out / max_abs_lse   the timed call's result against the fp32 oracle evaluated on the GPU,
                outside the timed regions (oracle as checker only)
  triton_gpu    the reference's own Triton kernels timed on this GPU by baseline/triton_reference.py
                when baseline/_ref/ is present (N = 1 only)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

PERF_CONFIGS = ["cfg2", "cfg3", "cfg4", "cfg5"]
REGIONS = 5  # timed regions of K steps each; the median is reported

# dram__bytes_read.sum + dram__bytes_write.sum of one stage-1 launch divided by its algorithmic KV
# bytes, from the ncu captures summarised under profiles/ (smaller batches for cfg3 / cfg5: traffic
# grows in proportion to the KV rows a launch streams)
NCU_TRAFFIC_RATIO = {
    "cfg2": (1.089, "profiles/stage1_umma_cfg2.md (one full-size launch)"),
    "cfg3": (1.046, "profiles/stage1_umma_cfg2.md (cfg3 at batch 8, scaled by KV bytes)"),
    "cfg4": (1.016, "profiles/stage1_umma_cfg2.md (one full-size launch)"),
    "cfg5": (1.011, "profiles/stage1_mma_cfg5.md (cfg5 at batch 16, scaled by KV bytes)"),
}


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", 1400.0)), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# CPU legs: the fp32 oracle port on the host cores (reported baseline; the reference arm)
# ---------------------------------------------------------------------------------------------

def _cpu_sample(w, lens, budget_s):
    """Chooses the sequences a bounded CPU sample runs on: the oracle is timed on one sequence, then
    as many sequences (in batch order) as fit `budget_s` are taken.  Returns (args of the oracle call
    on the sample, fraction of the job's KV rows it covers, description)."""
    from flash_tree_attn_b200.workloads import make_inputs
    from oracle.tree_attention_oracle import tree_attention_oracle  # timed CPU baseline

    def call_args(seqs):
        inp = make_inputs(w, "cpu", lens=lens, seqs=seqs)
        return (inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
                inp["kv_seq_len"], None, w.G)

    a = call_args([0])
    tree_attention_oracle(*a)  # thread pool, allocator
    t0 = time.perf_counter()
    tree_attention_oracle(*a)
    t_row = (time.perf_counter() - t0) / max(1, lens[0])  # seconds per KV row of one sequence
    seqs, rows = [], 0
    for b in range(w.B):
        if seqs and (rows + lens[b]) * t_row > budget_s:
            break
        seqs.append(b)
        rows += lens[b]
    frac = rows / max(1, sum(lens))
    what = (f"all {w.B} sequences of {w.name}" if len(seqs) == w.B else
            f"sequences 0..{len(seqs) - 1} of {w.B} of {w.name} ({100 * frac:.1f} % of its KV rows; calls/s scaled by that share)")
    return (a if seqs == [0] else call_args(seqs)), frac, what


def cpu_baseline(w, lens, budget_s=12.0):
    """calls/s of the fp32 CPU oracle (oracle/tree_attention_oracle.py) for the whole job, from a
    bounded sample (about 10-30 s of CPU work)."""
    from oracle.tree_attention_oracle import tree_attention_oracle  # timed CPU baseline

    torch.set_num_threads(os.cpu_count() or 1)
    a, frac, what = _cpu_sample(w, lens, budget_s)
    n, t0 = 0, time.perf_counter()
    while True:
        tree_attention_oracle(*a)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= 10.0 or n >= 200:
            break
    return {"value": n * frac / dt, "unit": "calls/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n} pass(es) of the fp32 CPU oracle over {what}"}


def reference_arm(args, w):
    """--impl reference: the CPU oracle (a port of the reference's dense checker,
    flash_tree_attn.py:388-397, ragged- and GQA-aware) on all host cores; each step is a bounded
    sample of the job.  Under torch.distributed.run rank 0 alone runs it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from flash_tree_attn_b200.workloads import draw_lengths
    from oracle.tree_attention_oracle import tree_attention_oracle

    torch.set_num_threads(os.cpu_count() or 1)  # torch.distributed.run exports OMP_NUM_THREADS=1
    lens = draw_lengths(w)
    a, frac, what = _cpu_sample(w, lens, 90.0 / max(1, args.steps + min(args.warmup, 3)))
    for _ in range(max(1, min(args.warmup, 3))):
        tree_attention_oracle(*a)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tree_attention_oracle(*a)
    dt = time.perf_counter() - t0
    val = args.steps * frac / dt
    world = int(os.environ.get("WORLD_SIZE", "1"))
    print(json.dumps({
        "impl": "reference", "metric": "tree_attn_calls_per_s", "value": val, "unit": "calls/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, lens, world),
        "cpu_baseline": {"value": val, "unit": "calls/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"each step: the fp32 CPU oracle over {what}"},
        "e2e": {"value": val, "unit": "calls/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------
# helpers of the GPU arm
# ---------------------------------------------------------------------------------------------

class Env:
    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def reduce(self, values, op="max"):
        """Element-wise max (or sum) over ranks of a list of floats."""
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.SUM)
        return [float(x) for x in t]

    def gather(self, values):
        """[world][len(values)] floats, on every rank."""
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.dist is None:
            return [[float(x) for x in t]]
        out = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [[float(x) for x in o] for o in out]


def workload_config(w, lens, world=1, extra=None):
    cfg = {
        "workload": f"{w.name}: B={w.B} H={w.H} kv_group_num={w.G} D={w.D} q_len={w.Q} "
                    f"{str(w.dtype).split('.')[-1]} ctx={w.ctx} lens={w.lens} tree={w.tree} block_size={w.block_size}",
        "sum_kv_len": int(sum(lens)),
        "parallelism": ("one GPU" if world == 1 else
                        (f"one job, KV range split over {world} GPUs" if (w.B == 1 and w.lens == "full") else
                         f"one job, its {w.B} sequences dealt to {world} GPUs by KV length" +
                         (", KV heads split where sequences run out" if w.B < world else "") + ", no collective")),
        "l2": ("inputs larger than L2: the KV rows one call streams exceed the 126 MB L2, no flush needed"
               if 2 * 2 * w.D * (w.H // w.G) * sum(lens) / world > (126 << 20) else
               "inputs smaller than L2 and not flushed between iterations: a launch-latency figure, not a bandwidth one"),
    }
    if extra:
        cfg.update(extra)
    return cfg


def timed_regions(env, fn, steps, regions=REGIONS):
    """`regions` regions of exactly `steps` calls of fn, each bracketed by barrier + synchronise;
    per region the max over ranks; returns (median ms per region, all region times)."""
    ms = []
    for _ in range(regions):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        env.barrier()
        ms.append(e0.elapsed_time(e1))
    ms = env.reduce(ms, "max")
    return statistics.median(ms), ms


def local_loop_ms(fn, steps, rest_s=0.25):
    """ms per call of `steps` back-to-back calls on this rank (CUDA events).  A kernel timed alone is
    compared with the burst peak, so the GPU first rests for `rest_s`: after the timed regions' tens of
    milliseconds of load the power management holds the SM clock down for a while (1965 -> ~1550 MHz)."""
    torch.cuda.synchronize()
    time.sleep(rest_s)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(steps):
        fn()
    s1.record()
    torch.cuda.synchronize()
    return s0.elapsed_time(s1) / steps


def oracle_errors(env, out, lse, inp, G):
    """max-abs error of (out, lse) against the fp32 oracle evaluated on this rank's GPU, max over
    ranks.  Checker only: nothing here is timed."""
    from oracle.tree_attention_oracle import tree_attention_oracle  # checker, outside the timed regions

    if out is None:
        return env.reduce([0.0, 0.0, 0.0], "max")
    ora = tree_attention_oracle(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"],
                                inp["mask"], inp["kv_seq_len"], None, G)
    err = (out.float() - ora["out"]).abs()
    eo = err.max().item()
    # beyond the rounding of the output itself (half a unit in the last place of its dtype)
    half_ulp = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}.get(out.dtype, 0.0)
    ex = (err - half_ulp * ora["out"].abs()).max().item()
    el = (lse - ora["lse"]).abs().max().item()
    del ora, err
    return env.reduce([eo, el, ex], "max")


class E2E:
    """A serving loop through the public call: step i's inputs are copied host->device on one stream
    while step i-1 computes on another and step i-2's result goes device->host on a third (two
    staging sets).  Every step's copies and its call are inside the timed region."""

    NAMES = ["q", "current_k", "current_v", "mask", "kv_seq_len"]
    NBUF = 2

    def __init__(self, env, inp, out_shape, out_dtype, call):
        self.env, self.call = env, call
        dev = env.dev
        # one pinned blob per step holds all of the step's inputs (256-byte aligned sections), so a
        # step costs one host->device copy; the device-side tensors are views into the staging blob
        offs, total = {}, 0
        for n in self.NAMES:
            offs[n] = total
            total += -(-(inp[n].numel() * inp[n].element_size()) // 256) * 256
        self.h2d = total
        self.host_blob = torch.empty(total, dtype=torch.uint8).pin_memory()
        self.dev_blob = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(self.NBUF)]

        def views(blob):
            out = {}
            for n in self.NAMES:
                nb = inp[n].numel() * inp[n].element_size()
                out[n] = blob[offs[n]:offs[n] + nb].view(inp[n].dtype).view(inp[n].shape)
            return out

        for n, v in views(self.host_blob).items():
            v.copy_(inp[n].cpu())
        self.stage = [views(b) for b in self.dev_blob]
        self.out_host = [torch.empty(out_shape, dtype=out_dtype).pin_memory() for _ in range(self.NBUF)]
        self.d2h = self.out_host[0].numel() * self.out_host[0].element_size()
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.s_cmp = torch.cuda.current_stream(dev)
        self.ev_in = [torch.cuda.Event() for _ in range(self.NBUF)]
        self.ev_cmp = [torch.cuda.Event() for _ in range(self.NBUF)]
        self.ev_out = [torch.cuda.Event() for _ in range(self.NBUF)]

    def step(self, i):
        b = i % self.NBUF
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.ev_cmp[b])  # the call that last read this staging set has finished
            self.dev_blob[b].copy_(self.host_blob, non_blocking=True)
            self.ev_in[b].record(self.s_in)
        self.s_cmp.wait_event(self.ev_in[b])
        o = self.call(self.stage[b])
        self.ev_cmp[b].record(self.s_cmp)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_cmp[b])
            self.s_out.wait_event(self.ev_out[b])
            self.out_host[b].copy_(o, non_blocking=True)
            o.record_stream(self.s_out)
            self.ev_out[b].record(self.s_out)

    def region(self, n_steps):
        self.env.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(self.s_cmp)
        for i in range(n_steps):
            self.step(i)
        for b in range(self.NBUF):  # the region ends when the last results are in host memory
            self.s_cmp.wait_event(self.ev_out[b])
        t1.record(self.s_cmp)
        self.env.barrier()
        return t0.elapsed_time(t1)

    def measure(self, steps, regions=REGIONS, warm_ms=150.0):
        # untimed warm-up: the host link takes a few hundred copies to reach its steady rate (the first
        # regions of a cold process are up to a third slower), so whole regions are run, every rank
        # agreeing on how many, until they have covered warm_ms
        self.region(4)
        spent, n = 0.0, 0
        while spent < warm_ms and n < 12:
            spent += self.env.reduce([self.region(steps)], "max")[0]
            n += 1
        ms = [self.region(steps) for _ in range(regions)]
        ms = self.env.reduce(ms, "max")
        med = statistics.median(ms)
        tot = self.env.reduce([float(self.h2d), float(self.d2h)], "sum")
        return {
            "value": steps / (med * 1e-3), "unit": "calls/s",
            "h2d_bytes_per_step": int(tot[0]), "d2h_bytes_per_step": int(tot[1]),
            "regions_ms": ms, "regions": regions,
            "h2d_gbs_per_rank": self.h2d * steps / (med * 1e-3) / 1e9,
            "note": "median of the regions, after untimed warm-up regions; per-step inputs (q, tree K/V, mask, lengths) of every rank's share from "
                    "pinned host memory, result copied back, copies on side streams overlapping the neighbouring "
                    "steps' calls; the KV cache is decode state resident in HBM",
        }


def stage1_roofline(env, w, name, ms_stage1, my_lens, args, head_share=1.0):
    """Roofline object of the stage-1 kernel, for the rank whose launch takes longest."""
    hbm_peak, tf_peak, tf_sust, peak_src = measured_peaks()
    kvb = 2 * 2 * w.D * w.Hkv * sum(my_lens) * head_share
    fl = (4 * w.H * w.Q * w.D * sum(my_lens) + 4 * len(my_lens) * w.H * w.Q * w.Q * w.D) * head_share
    rows = env.gather([ms_stage1, float(kvb), float(fl)])
    slow = max(range(len(rows)), key=lambda r: rows[r][0])
    ms, kvb, fl = rows[slow]
    achieved = kvb / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
    roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
            "traffic": None, "peak_source": peak_src, "kernel": "stage1", "rank": slow,
            "launch_ms": ms, "algorithmic_bytes_per_launch": int(kvb),
            "frac_of_nominal_8tbs": achieved / 8000.0}
    # G*Q query rows share every KV row: flops per KV byte = G*Q.  Above the ridge of the measured
    # peaks the tensor pipe bounds the kernel, not HBM (cfg4: 512 flop/B).
    if kvb > 0 and fl / kvb > tf_peak * 1e12 / (hbm_peak * 1e9):
        ach_tf = fl / (ms * 1e-3) / 1e12
        roof.update({"bound": "tensor", "achieved": ach_tf, "peak": tf_peak, "unit": "TFLOP/s", "frac": ach_tf / tf_peak,
                     "algorithmic_flops_per_launch": int(fl), "hbm_achieved_gbs": achieved,
                     "peak_note": "burst figure; inside a long loop under the power cap the sustained figure applies",
                     "peak_sustained": tf_sust, "frac_of_sustained": ach_tf / tf_sust})
    ratio = NCU_TRAFFIC_RATIO.get(name)
    if ratio is not None and args.batch == 0 and not args.paged:
        roof["traffic"] = ratio[0] * kvb
        roof["traffic_source"] = ratio[1]
    return roof


# ---------------------------------------------------------------------------------------------
# one workload on the GPUs of this job
# ---------------------------------------------------------------------------------------------

def measure_batched(env, args, name, w, sample_clocks=False):
    """A job whose sequences are independent: each rank holds the sequences dist.shard_batch deals
    it (all of them at N = 1) and runs the operator on them; no collective."""
    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200 import _lib
    from flash_tree_attn_b200.dist import shard_batch_and_heads, take_heads
    from flash_tree_attn_b200.workloads import draw_lengths, make_inputs

    lens = draw_lengths(w)
    shards = shard_batch_and_heads(lens, w.Hkv, env.world)
    mine, kv_lo, kv_hi = shards[env.rank]
    head_share = (kv_hi - kv_lo) / w.Hkv  # 1 unless there are fewer sequences than ranks
    my_lens = [lens[i] for i in mine]
    res = {"scaling": "strong"}
    prep = inp = None
    if mine:
        inp = make_inputs(w, env.dev, lens=lens, seqs=mine)
        if head_share < 1:  # this rank's KV heads of its sequences, and the query heads that read them
            for n, mul in (("q", w.G), ("k_cache", 1), ("v_cache", 1), ("current_k", 1), ("current_v", 1)):
                inp[n] = take_heads(inp[n], kv_lo, kv_hi, mul)
            if inp["mask"].dim() == 4 and inp["mask"].size(1) > 1:
                inp["mask"] = take_heads(inp["mask"], kv_lo, kv_hi, w.G)
        if args.paged:
            from flash_tree_attn_b200.workloads import to_paged
            kp, vp, table = to_paged(inp["k_cache"], inp["v_cache"], my_lens, page_size=args.paged, seed=w.seed)
            inp["k_cache"] = inp["v_cache"] = None  # the dense copy is not needed any more
            prep = fta.prepare(inp["q"], kp, vp, inp["current_k"], inp["current_v"], inp["mask"], inp["kv_seq_len"],
                               w.block_size, w.ctx, kv_group_num=w.G, block_table=table, want_lse=True)
        else:
            prep = fta.prepare(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
                               inp["kv_seq_len"], w.block_size, w.ctx, kv_group_num=w.G, want_lse=True)
    run = prep.run if prep else (lambda: None)

    # ---- device-timed regions: inputs resident in HBM -----------------------------------------
    for _ in range(args.warmup):
        run()
    sampler = ClockSampler(env.local) if (sample_clocks and env.rank == 0) else None
    if sampler:
        sampler.start()
    ms, regions_ms = timed_regions(env, run, args.steps)
    res.update({"value": args.steps / (ms * 1e-3), "unit": "calls/s", "ms_per_step": ms / args.steps,
                "regions_ms": regions_ms})

    # ---- the stages alone, for the roofline ---------------------------------------------------
    ms1 = local_loop_ms(prep.run_stage1, args.steps) if prep else 0.0
    ms2 = local_loop_ms(prep.run_stage2, args.steps) if prep else 0.0
    s = env.reduce([ms1, ms2], "max")
    res["stage_ms"] = {"stage1": s[0], "stage2": s[1]}
    res["roofline"] = stage1_roofline(env, w, name, ms1, my_lens, args, head_share)
    if sampler:
        # The timed regions last milliseconds, nvidia-smi samples every 50 ms: keep the same call
        # running (untimed) for half a second so that the clock record is one of this load.
        t_load = time.perf_counter()
        while time.perf_counter() - t_load < 0.5:
            for _ in range(50):
                run()
            torch.cuda.synchronize()
        res["clocks"] = sampler.stop()
    hbm_peak = measured_peaks()[0]
    all_kvb = 2 * 2 * w.D * w.Hkv * sum(lens)
    res["kv_read_gbs"] = all_kvb * res["value"] / 1e9
    res["kv_read_frac_of_measured_peak"] = res["kv_read_gbs"] / (hbm_peak * env.world)
    res["kv_read_frac_of_nominal_8tbs"] = res["kv_read_gbs"] / (8000.0 * env.world)
    res["tflops"] = (4 * w.H * w.Q * w.D * sum(lens) + 4 * w.B * w.H * w.Q * w.Q * w.D) * res["value"] / 1e12
    res["gpu_launches_per_step"] = 2 * env.world
    res["sequences_per_rank"] = [len(x.seqs) for x in shards]
    if head_share < 1:
        res["kv_heads_per_rank"] = kv_hi - kv_lo

    # ---- parity of what was timed -------------------------------------------------------------
    if not args.no_check and not args.paged:
        out, lse = prep.run() if prep else (None, None)
        torch.cuda.synchronize()
        eo, el, ex = oracle_errors(env, out, lse, inp, w.G)
        res["max_abs_out"], res["max_abs_lse"] = eo, el
        # the parity tests' rule: 2e-3 on the output beyond its own rounding, 1e-3 on the LSE
        res["within_tolerance"] = bool(ex <= 2e-3 and el <= 1e-3)
    st = _lib.load().fta_umma_status()
    res["kernel_status"] = int(env.reduce([float(st)], "max")[0])

    # ---- end to end through the public call ---------------------------------------------------
    if not args.skip_e2e and not args.paged:
        if mine:
            def call(st):
                return fta.flash_decoding_attention(st["q"], inp["k_cache"], inp["v_cache"], st["current_k"],
                                                    st["current_v"], st["mask"], st["kv_seq_len"], w.block_size, w.ctx,
                                                    kv_group_num=w.G)
            e2e = E2E(env, inp, (len(mine), (kv_hi - kv_lo) * w.G, w.Q, w.D), w.dtype, call)
            res["e2e"] = e2e.measure(args.steps)
        else:  # a rank without sequences only keeps the barriers in step
            for _ in range(REGIONS + 1):
                env.barrier(); env.barrier()
            env.reduce([0.0] * REGIONS, "max"); env.reduce([0.0, 0.0], "sum")
    res["config"] = workload_config(w, lens, env.world, {"kv_cache": f"paged, {args.paged} rows per page, shuffled"} if args.paged else None)
    res["dtype"] = {"float16": "fp16", "bfloat16": "bf16"}.get(str(w.dtype).split(".")[-1], str(w.dtype))
    res["_lens"] = lens
    return res


def measure_seq_split(env, args, name, w):
    """One long sequence on N GPUs (cfg4): every rank owns a contiguous KV range and computes an fp32
    partial (O, LSE); one exchange-merge kernel per rank over peer-mapped memory (or one all-gather +
    merge kernel) gives every rank the result.  Strong scaling: the job is the same call at every N."""
    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200 import _lib
    from flash_tree_attn_b200 import dist as fdist
    from flash_tree_attn_b200.workloads import draw_lengths, flops, kv_bytes, make_inputs

    rank, world, dev = env.rank, env.world, env.dev
    lens = draw_lengths(w)
    inp = make_inputs(w, dev, lens=lens)
    lo, hi = fdist.kv_ranges(w.ctx, world)[rank]
    k_sh, v_sh = inp["k_cache"][:, :, lo:hi], inp["v_cache"][:, :, lo:hi]
    my_rows = max(0, min(lens[0], hi) - lo)
    shard_len = torch.tensor([my_rows], dtype=torch.int32, device=dev)

    xch = None
    if args.exchange != "nccl":
        form = {"peer": "auto", "peer-gather": "gather", "peer-scatter": "scatter"}[args.exchange]
        xch = fdist.PeerExchange(w.B * w.H * w.Q * w.D, w.B * w.H * w.Q, dev, form=form)

    def step(q, ck, cv, mask):
        return fdist.kv_range_decode(q, k_sh, v_sh, ck, cv, mask, shard_len, w.block_size, w.G, exchange=xch)

    a = (inp["q"], inp["current_k"], inp["current_v"], inp["mask"])
    run = lambda: step(*a)
    pk = None
    if xch is not None:
        # device-timed region: the call validated once, as in the one-GPU arm; the end-to-end region
        # below goes through the public call every step
        pk = fdist.PreparedKvRange(inp["q"], k_sh, v_sh, inp["current_k"], inp["current_v"], inp["mask"], shard_len,
                                   w.block_size, w.G, exchange=xch)
        run = pk.run
    for _ in range(args.warmup):
        run()
    ms, regions_ms = timed_regions(env, run, args.steps)
    res = {"scaling": "strong", "value": args.steps / (ms * 1e-3), "unit": "calls/s", "ms_per_step": ms / args.steps,
           "regions_ms": regions_ms}

    # the operator's two kernels on this rank's shard alone (no exchange), and stage 1 alone
    part = fta.prepare(inp["q"], k_sh, v_sh, inp["current_k"], inp["current_v"], inp["mask"], shard_len, w.block_size,
                       None, kv_group_num=w.G, want_lse=True, out_dtype=torch.float32, with_tree=rank == world - 1)
    ms_k = local_loop_ms(part.run, args.steps)
    ms1 = local_loop_ms(part.run_stage1, args.steps)
    ms2 = local_loop_ms(part.run_stage2, args.steps)
    s = env.reduce([ms_k, ms1, ms2], "max")
    res["stage_ms"] = {"stage1": s[1], "stage2": s[2], "kernels_per_rank": s[0],
                       "exchange_and_merge": max(0.0, ms / args.steps - s[0])}
    res["roofline"] = stage1_roofline(env, w, name, ms1, [my_rows], args)
    kvb = kv_bytes(w, lens)
    res["kv_read_gbs"] = kvb * res["value"] / 1e9
    res["tflops"] = flops(w, lens) * res["value"] / 1e12
    res["whole_call_frac_of_tensor_peak"] = res["tflops"] / (measured_peaks()[1] * world)
    res["gpu_launches_per_step"] = 3 * world
    res["exchange"] = ("one exchange-merge kernel per rank over peer-mapped memory "
                       f"({'scatter' if xch.scatter else 'gather'} form)") if xch is not None else "one NCCL all-gather + merge kernel"

    if not args.no_check:
        out, lse = run()
        torch.cuda.synchronize()
        eo, el, ex = oracle_errors(env, out, lse, inp, w.G)
        res["max_abs_out"], res["max_abs_lse"] = eo, el
        # the parity tests' rule: 2e-3 on the output beyond its own rounding, 1e-3 on the LSE
        res["within_tolerance"] = bool(ex <= 2e-3 and el <= 1e-3)
    st = _lib.load().fta_umma_status()
    res["kernel_status"] = int(env.reduce([float(st)], "max")[0])

    if not args.skip_e2e:
        def call(st):
            o, _ = step(st["q"], st["current_k"], st["current_v"], st["mask"])
            return o
        e2e = E2E(env, inp, (w.B, w.H, w.Q, w.D), w.dtype, call)
        res["e2e"] = e2e.measure(args.steps)
    if xch is not None:
        xch.check()  # raises if a wait for a peer ever ran out
        torch.cuda.synchronize()
        xch.close()
    res["config"] = workload_config(w, lens, world)
    res["dtype"] = "bf16" if w.dtype == torch.bfloat16 else "fp16"
    res["_lens"] = lens
    return res


def measure(env, args, name, sample_clocks=False):
    from flash_tree_attn_b200.workloads import WORKLOADS, small

    w = WORKLOADS[name]
    if args.batch > 0:
        w = small(w, B=args.batch, name=f"{w.name}[B={args.batch}]")
    if w.lens == "full" and w.B == 1 and env.world > 1:
        r = measure_seq_split(env, args, name, w)
    else:
        r = measure_batched(env, args, name, w, sample_clocks)
    torch.cuda.synchronize()
    import flash_tree_attn_b200.op as op

    op._scratch.clear()
    torch.cuda.empty_cache()
    return r, w


def triton_arm(args):
    """The reference's Triton kernels on this GPU and the reference under the Triton interpreter on
    the host cores, each in a child process (baseline/triton_reference.py), when baseline/_ref/ holds
    the reference; otherwise says why not."""
    script = os.path.join(ROOT, "baseline", "triton_reference.py")
    if not os.path.exists(os.path.join(ROOT, "baseline", "_ref", "flash_tree_attn_head.py")):
        why = {"unavailable": "baseline/_ref/ is absent on this machine (the reference's file is not part of this repository)"}
        return why, why
    def child(extra, env_extra, limit):
        try:
            r = subprocess.run([sys.executable, script, *extra], capture_output=True, text=True, timeout=limit,
                               env=dict(os.environ, **env_extra))
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
            if r.returncode != 0 or not lines:
                return {"unavailable": ("child failed: " + (r.stderr or r.stdout)[-600:]).replace("\n", " ")}
            return json.loads(lines[-1])
        except subprocess.TimeoutExpired:
            return {"unavailable": f"child exceeded {limit} s"}
    gpu = {}
    for name in PERF_CONFIGS:  # one child per workload: a failure in one cannot take the others with it
        r = child(["--workloads", name, "--reps", "20", "--warmup", "5"], {}, 400)
        gpu[name] = r.get("workloads", {}).get(name, r)
    cpu = child(["--interpret", "cfg1"], {"TRITON_INTERPRET": "1", "CUDA_VISIBLE_DEVICES": ""}, 300)
    return {"workloads": gpu}, cpu


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg3")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", action="store_true", help="the headline workload only (no per_config, no Triton arm)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison with the fp32 oracle")
    ap.add_argument("--no-triton", action="store_true", help="skip the reference's Triton kernels")
    ap.add_argument("--kernel", default=None, choices=[None, "auto", "mma", "umma"])
    ap.add_argument("--skip-e2e", action="store_true", help="device-timed regions only (profiling runs)")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size (profiling runs)")
    ap.add_argument("--paged", type=int, default=0, metavar="PAGE_SIZE",
                    help="house the KV cache in shuffled pages of this many rows (multiple of 64) and "
                         "run the device-timed region through the block table (implies --skip-e2e)")
    ap.add_argument("--exchange", choices=["peer", "peer-gather", "peer-scatter", "nccl"], default="peer",
                    help="sequence-split arm (one long sequence on several GPUs): 'peer' = one exchange-merge "
                         "kernel per rank over peer-mapped memory (-gather: every rank reads all partials; "
                         "-scatter: every rank merges a slice of the rows and stores it to all; plain 'peer' "
                         "takes the library's choice), 'nccl' = all-gather + merge kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from flash_tree_attn_b200.workloads import WORKLOADS, small

    if args.impl == "reference":
        w = WORKLOADS[args.workload]
        if args.batch > 0:
            w = small(w, B=args.batch, name=f"{w.name}[B={args.batch}]")
        reference_arm(args, w)
        return

    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200 import _lib

    _lib.load()  # fail loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    if args.kernel:
        fta.set_kernel(args.kernel)
    if args.paged:
        args.skip_e2e = True
    env = Env()

    head, w = measure(env, args, args.workload, sample_clocks=True)
    lens = head.pop("_lens")
    per = {}
    if not args.only:
        for name in PERF_CONFIGS:
            if name == args.workload:
                continue
            try:
                r, _ = measure(env, args, name)
                r.pop("_lens")
            except Exception as e:  # one configuration's failure must not cost the line its other numbers
                r = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.synchronize()
            per[name] = r

    if env.rank == 0:
        line = {
            "metric": "tree_attn_calls_per_s", "value": head["value"], "unit": "calls/s", "n_gpus": env.world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": head["scaling"], "vs_baseline": None,
            "dtype": head["dtype"], "data": "synthetic", "config": head["config"],
            "timing": f"median of {REGIONS} regions of exactly {args.steps} steps, each between barrier + synchronise, "
                      "CUDA events, max over ranks per region",
        }
        for k in ("regions_ms", "kv_read_gbs", "kv_read_frac_of_measured_peak", "kv_read_frac_of_nominal_8tbs", "tflops",
                  "stage_ms", "roofline", "e2e", "max_abs_out", "max_abs_lse", "within_tolerance", "kernel_status",
                  "sequences_per_rank", "exchange", "whole_call_frac_of_tensor_peak", "clocks"):
            if k in head:
                line[k] = head[k]
        line["gpu_launches"] = head["gpu_launches_per_step"] * args.steps * REGIONS
        if per:
            line["per_config"] = per
        if env.world == 1 and not args.only and not args.no_triton:
            gpu, cpu = triton_arm(args)
            line["triton_gpu"] = gpu.get("workloads", gpu)
            line["reference_interpreter"] = cpu.get("interpreter", cpu)
        if not args.no_cpu_baseline and env.world == 1:
            line["cpu_baseline"] = cpu_baseline(w, lens)
        print(json.dumps(line))
    if env.dist is not None:
        env.dist.barrier()
        env.dist.destroy_process_group()


if __name__ == "__main__":
    main()
