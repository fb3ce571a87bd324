#!/usr/bin/env python
"""Benchmark of the tree-attention decode operator.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

A step is one call of flash_decoding_attention on one synthetic batch.  At N GPUs every rank
holds its own batch of the workload's shape (the job's sequences sharded by batch, no
data-path collective): weak scaling, value = calls all ranks completed per second of the
slowest rank.  Prints ONE JSON line (rank 0).

Keys beyond the basic contract:
  roofline      dominant kernel (stage 1): algorithmic KV bytes per launch / its CUDA-event
                duration, against the measured HBM copy peak
  cpu_baseline  the fp32 CPU oracle timed on this box's host cores (reported baseline only)
  e2e           same metric through the public Python call with the step's inputs (q, tree
                K/V, mask, lengths) copied from pinned host memory and the result copied back
                inside the timed region; the KV cache, which is decode state that lives in HBM
                across steps, is resident
  e2e_cold      as e2e, but the KV cache is shipped from pinned host memory every step too
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


# dram__bytes_read.sum + dram__bytes_write.sum of one stage-1 launch divided by its algorithmic KV
# bytes, from the ncu captures summarised under profiles/ (smaller batches for cfg3 / cfg5: traffic
# grows in proportion to the KV rows a launch streams)
NCU_TRAFFIC_RATIO = {
    "cfg2": (1.089, "profiles/stage1_umma_cfg2.md (one full-size launch)"),
    "cfg3": (1.043, "profiles/stage1_umma_cfg2.md (cfg3 at batch 8, scaled by KV bytes)"),
    "cfg4": (1.016, "profiles/stage1_umma_cfg2.md (one full-size launch)"),
    "cfg5": (1.011, "profiles/stage1_mma_cfg5.md (cfg5 at batch 16, scaled by KV bytes)"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def sustained_tensor_peak():
    """cuBLAS bf16 TFLOP/s of a seconds-long loop under the power cap (the figure to hold a kernel
    against when it is timed inside a long loop, as the stage-1 loop below is)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        if "bf16_tflops_sustained" in d:
            return float(d["bf16_tflops_sustained"])
    return 1400.0


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


def cpu_oracle_calls_per_s(w, min_seconds: float, max_calls: int):
    """Times the fp32 CPU oracle (oracle/tree_attention_oracle.py) on whole calls of the
    workload, on the host cores torch uses.  Returns (calls/s, calls timed, threads)."""
    from flash_tree_attn_b200.workloads import make_inputs
    from oracle.tree_attention_oracle import tree_attention_oracle  # timed CPU baseline

    inp = make_inputs(w, "cpu")
    args = (inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
            inp["kv_seq_len"], None, w.G)
    tree_attention_oracle(*args)  # warm-up (thread pool, allocator)
    n, t0 = 0, time.perf_counter()
    while True:
        tree_attention_oracle(*args)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or n >= max_calls:
            break
    return n / dt, n, torch.get_num_threads()


def reference_arm(args, w):
    """--impl reference: the CPU oracle (a port of the reference's dense checker,
    flash_tree_attn.py:388-397, ragged- and GQA-aware) on the host cores; the reference's own
    Python/Triton source is not available on the benchmark machine."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from flash_tree_attn_b200.workloads import make_inputs
    from oracle.tree_attention_oracle import tree_attention_oracle

    inp = make_inputs(w, "cpu")
    a = (inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
         inp["kv_seq_len"], None, w.G)
    for _ in range(max(1, min(args.warmup, 3))):
        tree_attention_oracle(*a)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tree_attention_oracle(*a)
    dt = time.perf_counter() - t0
    val = args.steps / dt
    print(json.dumps({
        "impl": "reference", "metric": "tree_attn_calls_per_s", "value": val, "unit": "calls/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, inp["lens"]),
        "cpu_baseline": {"value": val, "unit": "calls/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{args.steps} whole calls of {w.name} (all {w.B} sequences) on the host cores"},
        "e2e": {"value": val, "unit": "calls/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def seq_split_arm(args, w, fta, dev, rank, world, dist):
    """One long sequence on N GPUs (cfg4): every rank owns a contiguous KV range, computes an fp32
    partial (O, LSE), ONE all-gather moves the packed partials, the merge kernel runs on every
    rank.  Strong scaling: the job is the same call at every N."""
    from flash_tree_attn_b200 import dist as fdist
    from flash_tree_attn_b200.workloads import draw_lengths, flops, kv_bytes, make_inputs

    lens = draw_lengths(w)
    inp = make_inputs(w, dev, lens=lens)
    lo, hi = fdist.kv_ranges(w.ctx, world)[rank]
    k_sh, v_sh = inp["k_cache"][:, :, lo:hi], inp["v_cache"][:, :, lo:hi]
    shard_len = torch.tensor([max(0, min(lens[0], hi) - lo)], dtype=torch.int32, device=dev)

    xch = None
    if args.exchange != "nccl":
        form = {"peer": "auto", "peer-gather": "gather", "peer-scatter": "scatter"}[args.exchange]
        xch = fdist.PeerExchange(w.B * w.H * w.Q * w.D, w.B * w.H * w.Q, dev, form=form)

    def step(q, ck, cv, mask):
        return fdist.kv_range_decode(q, k_sh, v_sh, ck, cv, mask, shard_len, w.block_size, w.G, exchange=xch)

    def sync():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    a = (inp["q"], inp["current_k"], inp["current_v"], inp["mask"])
    run = lambda: step(*a)
    if xch is not None:
        # device-timed region: the call validated once, as in the one-GPU arm; the end-to-end region
        # below goes through the public call every step
        run = fdist.PreparedKvRange(inp["q"], k_sh, v_sh, inp["current_k"], inp["current_v"], inp["mask"], shard_len,
                                    w.block_size, w.G, exchange=xch).run
    for _ in range(args.warmup):
        run()
    sync()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    # end to end: the step's inputs come from pinned host memory, the result goes back
    names = ["q", "current_k", "current_v", "mask"]
    host = {n: inp[n].cpu().pin_memory() for n in names}
    stage = {n: torch.empty_like(inp[n]) for n in names}
    out_host = torch.empty((w.B, w.H, w.Q, w.D), dtype=w.dtype).pin_memory()
    x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    x0.record()
    for _ in range(args.steps):
        for n in names:
            stage[n].copy_(host[n], non_blocking=True)
        o, _ = step(stage["q"], stage["current_k"], stage["current_v"], stage["mask"])
        out_host.copy_(o, non_blocking=True)
    x1.record()
    sync()
    ms_e2e = x0.elapsed_time(x1)
    if xch is not None:
        xch.check()  # raises if a wait for a peer ever ran out
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        hbm_peak, tf_peak, peak_src = measured_peaks()
        kvb = kv_bytes(w, lens)
        calls_s = args.steps / (ms * 1e-3)
        tfl = flops(w, lens) * calls_s / 1e12
        print(json.dumps({
            "metric": "tree_attn_calls_per_s", "value": calls_s, "unit": "calls/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload_config(w, lens), parallelism=f"kv-range x{world}, " + (
                f"one exchange-merge kernel per call over peer-mapped memory ({'scatter' if xch.scatter else 'gather'} form)"
                if xch is not None
                else "one all-gather + merge per call")),
            "kv_read_gbs": kvb * calls_s / 1e9, "tflops": tfl,
            "roofline": {"bound": "tensor", "achieved": tfl, "peak": tf_peak * world, "unit": "TFLOP/s",
                         "frac": tfl / (tf_peak * world), "traffic": None, "peak_source": peak_src,
                         "kernel": "whole call (stage 1 + stage 2 + " + ("exchange-merge)" if xch is not None else "all-gather + merge)")},
            "e2e": {"value": args.steps / (ms_e2e * 1e-3), "unit": "calls/s",
                    "h2d_bytes_per_step": sum(host[n].numel() * host[n].element_size() for n in names),
                    "d2h_bytes_per_step": out_host.numel() * out_host.element_size(),
                    "note": "per-rank copies of q / tree K,V / mask from pinned host memory, result copied back; "
                            "KV cache shards resident in HBM"},
            "gpu_launches": 3 * args.steps, "clocks": clocks,
        }))
    if xch is not None:
        xch.close()
    dist.barrier()
    dist.destroy_process_group()


def workload_config(w, lens):
    return {
        "workload": f"{w.name}: B={w.B} H={w.H} kv_group_num={w.G} D={w.D} q_len={w.Q} "
                    f"{str(w.dtype).split('.')[-1]} ctx={w.ctx} lens={w.lens} tree={w.tree} block_size={w.block_size}",
        "sum_kv_len": int(sum(lens)),
        "l2": ("inputs larger than L2: the KV rows one call streams exceed the 126 MB L2, no flush needed"
               if 2 * 2 * w.D * (w.H // w.G) * sum(lens) > (126 << 20) else
               "inputs smaller than L2 and not flushed between iterations: a launch-latency figure, not a bandwidth one"),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel", default=None, choices=[None, "auto", "mma", "umma"])
    ap.add_argument("--skip-e2e", action="store_true", help="device-timed region only (profiling runs)")
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

    from flash_tree_attn_b200.workloads import WORKLOADS, draw_lengths, flops, kv_bytes, make_inputs, small

    w = WORKLOADS[args.workload]
    if args.batch > 0:
        w = small(w, B=args.batch, name=f"{w.name}[B={args.batch}]")
    if args.impl == "reference":
        reference_arm(args, w)
        return

    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200 import _lib

    _lib.load()  # fail loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    if args.kernel:
        fta.set_kernel(args.kernel)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    if w.lens == "full" and w.B == 1 and world > 1:
        seq_split_arm(args, w, fta, dev, rank, world, dist)
        return

    # each rank holds its own batch of the workload's shape (the job's batch, sharded): its own
    # values, but the sequence lengths of rank 0's draw, so that the work per GPU really is the same
    # at every N (with a draw per rank the slowest rank of 8 streams 27 % more rows than rank 0 and
    # the max-over-ranks time measures that, not the scaling)
    wr = small(w, seed=w.seed + 1000 * rank)
    lens = draw_lengths(w)
    inp = make_inputs(wr, dev, lens=lens)
    call_args = (inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
                 inp["kv_seq_len"], w.block_size, w.ctx)
    if args.paged:
        from flash_tree_attn_b200.workloads import to_paged
        args.skip_e2e = True
        kp, vp, table = to_paged(inp["k_cache"], inp["v_cache"], lens, page_size=args.paged, seed=wr.seed)
        inp["k_cache"] = inp["v_cache"] = None  # the dense copy is not needed any more
        prep = fta.prepare(inp["q"], kp, vp, inp["current_k"], inp["current_v"], inp["mask"], inp["kv_seq_len"],
                           w.block_size, w.ctx, kv_group_num=w.G, block_table=table)
    else:
        prep = fta.prepare(*call_args, kv_group_num=w.G)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-timed region: inputs resident in HBM -------------------------------------
    for _ in range(args.warmup):
        prep.run()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        prep.run()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)

    # ---- dominant kernel alone (stage 1), for the roofline -------------------------------
    for _ in range(3):
        prep.run_stage1()
    torch.cuda.synchronize()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.steps):
        prep.run_stage1()
    s1.record()
    torch.cuda.synchronize()
    ms_stage1 = s0.elapsed_time(s1) / args.steps
    m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m0.record()
    for _ in range(args.steps):
        prep.run_stage2()
    m1.record()
    torch.cuda.synchronize()
    ms_stage2 = m0.elapsed_time(m1) / args.steps
    # The timed regions last milliseconds, nvidia-smi samples every 50 ms: keep the same call running
    # (untimed) for half a second so that the clock record is one of this load, not of an idle GPU.
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 0.5:
        for _ in range(50):
            prep.run()
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the public call, per-step inputs from pinned host memory ------
    # A serving loop: step i's inputs are copied host->device on one stream while step i-1
    # computes on another and step i-2's result goes device->host on a third (two staging sets).
    # Every step's copies and its call are inside the timed region.
    names = ["q", "current_k", "current_v", "mask", "kv_seq_len"]
    NBUF = 2
    # one pinned blob per step holds all of the step's inputs (256-byte aligned sections), so a
    # step costs one host->device copy; the device-side tensors are views into the staging blob
    offs, total = {}, 0
    for n in names:
        offs[n] = total
        total += -(-(inp[n].numel() * inp[n].element_size()) // 256) * 256
    host_blob = torch.empty(total, dtype=torch.uint8).pin_memory()
    dev_blob = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(NBUF)]

    def views(blob):
        out = {}
        for n in names:
            nb = inp[n].numel() * inp[n].element_size()
            out[n] = blob[offs[n]:offs[n] + nb].view(inp[n].dtype).view(inp[n].shape)
        return out

    for n, v in views(host_blob).items():
        v.copy_(inp[n].cpu())
    stage = [views(b) for b in dev_blob]
    out_host = [torch.empty((w.B, w.H, w.Q, w.D), dtype=w.dtype).pin_memory() for _ in range(NBUF)]
    h2d = total
    d2h = out_host[0].numel() * out_host[0].element_size()
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_cmp = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(NBUF)]
    ev_cmp = [torch.cuda.Event() for _ in range(NBUF)]
    ev_out = [torch.cuda.Event() for _ in range(NBUF)]

    def e2e_step(i, cold_cache=None):
        b = i % NBUF
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[b])  # the call that last read this staging set has finished
            dev_blob[b].copy_(host_blob, non_blocking=True)
            if cold_cache is not None:
                s_in.wait_event(ev_cmp[(b + 1) % NBUF])  # the single cache copy is still being read
                inp["k_cache"].copy_(cold_cache[0], non_blocking=True)
                inp["v_cache"].copy_(cold_cache[1], non_blocking=True)
            ev_in[b].record(s_in)
        s_cmp.wait_event(ev_in[b])
        st = stage[b]
        o = fta.flash_decoding_attention(st["q"], inp["k_cache"], inp["v_cache"], st["current_k"], st["current_v"],
                                         st["mask"], st["kv_seq_len"], w.block_size, w.ctx, kv_group_num=w.G)
        ev_cmp[b].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[b])
            s_out.wait_event(ev_out[b])
            out_host[b].copy_(o, non_blocking=True)
            o.record_stream(s_out)
            ev_out[b].record(s_out)

    def e2e_region(n_steps, cold_cache=None):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(s_cmp)
        for i in range(n_steps):
            e2e_step(i, cold_cache)
        for b in range(NBUF):  # the region ends when the last results are in host memory
            s_cmp.wait_event(ev_out[b])
        t1.record(s_cmp)
        barrier()
        return t0.elapsed_time(t1)

    ms_e2e = float("nan")
    if not args.skip_e2e:
        e2e_region(4)
        ms_e2e = e2e_region(args.steps)

    cold = None
    cache_bytes = 0 if args.skip_e2e else 2 * inp["k_cache"].numel() * inp["k_cache"].element_size()
    if cache_bytes <= 8 << 30 and not args.skip_e2e:
        cold_host = (inp["k_cache"].cpu().pin_memory(), inp["v_cache"].cpu().pin_memory())
        n_cold = max(2, min(args.steps, 10))
        e2e_region(2, cold_host)
        cold = (e2e_region(n_cold, cold_host), n_cold)

    # ---- max over ranks ---------------------------------------------------------------------
    vals = torch.tensor([ms, ms_stage1, ms_stage2, ms_e2e, cold[0] if cold else 0.0, float(sum(lens))],
                        dtype=torch.float64, device=dev)
    if dist is not None:
        mx = vals.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = vals.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, ms_stage1, ms_stage2, ms_e2e = (float(x) for x in mx[:4])
        if cold:
            cold = (float(mx[4]), cold[1])
        total_len = float(sm[5])
    else:
        total_len = float(sum(lens))

    if rank == 0:
        hbm_peak, tf_peak, peak_src = measured_peaks()
        kvb = kv_bytes(w, lens)  # this rank's launch
        all_kvb = 2 * 2 * w.D * w.Hkv * total_len
        calls_s = world * args.steps / (ms * 1e-3)
        achieved = kvb / (ms_stage1 * 1e-3) / 1e9
        line = {
            "metric": "tree_attn_calls_per_s", "value": calls_s, "unit": "calls/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"float16": "fp16", "bfloat16": "bf16"}.get(str(w.dtype).split(".")[-1], str(w.dtype)),
            "data": "synthetic",
            "config": dict(workload_config(w, lens), **({"kv_cache": f"paged, {args.paged} rows per page, shuffled"} if args.paged else {})),
            "kv_read_gbs": all_kvb * args.steps / (ms * 1e-3) / 1e9,
            "kv_read_frac_of_measured_peak": all_kvb * args.steps / (ms * 1e-3) / 1e9 / (hbm_peak * world),
            "kv_read_frac_of_nominal_8tbs": all_kvb * args.steps / (ms * 1e-3) / 1e9 / (8000.0 * world),
            "tflops": world * flops(w, lens) * args.steps / (ms * 1e-3) / 1e12,
            "stage_ms": {"stage1": ms_stage1, "stage2": ms_stage2},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "traffic": None, "peak_source": peak_src,
                         "kernel": "stage1", "algorithmic_bytes_per_launch": kvb},
            "e2e": {"value": world * args.steps / (ms_e2e * 1e-3), "unit": "calls/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h,
                    "note": "per-step inputs (q, tree K/V, mask, lengths) from pinned host memory, result "
                            "copied back, copies on side streams overlapping the neighbouring steps' calls; "
                            "the KV cache is decode state resident in HBM"},
            "gpu_launches": prep.launches * args.steps,
            "clocks": clocks,
        }
        if cold:
            line["e2e_cold"] = {"value": world * cold[1] / (cold[0] * 1e-3), "unit": "calls/s",
                                "h2d_bytes_per_step": h2d + cache_bytes, "d2h_bytes_per_step": d2h,
                                "note": "KV cache also copied from pinned host memory every step (PCIe-bound)"}
        # G*Q query rows share every KV row: flops per KV byte = G*Q.  Above the ridge of the
        # measured peaks the tensor pipe bounds the kernel, not HBM (cfg4: 512 flop/B).
        fl = flops(w, lens)
        if fl / kvb > tf_peak * 1e12 / (hbm_peak * 1e9):
            ach_tf = fl / (ms_stage1 * 1e-3) / 1e12
            line["roofline"].update({"bound": "tensor", "achieved": ach_tf, "peak": tf_peak, "unit": "TFLOP/s",
                                     "frac": ach_tf / tf_peak, "algorithmic_flops_per_launch": fl,
                                     "hbm_achieved_gbs": achieved,
                                     "peak_note": "burst figure; the stage-1 loop runs long enough to sit under the power "
                                                  "cap, where the sustained figure applies",
                                     "peak_sustained": sustained_tensor_peak(),
                                     "frac_of_sustained": ach_tf / sustained_tensor_peak()})
        ratio = NCU_TRAFFIC_RATIO.get(args.workload)
        if ratio is not None and args.batch == 0:
            line["roofline"]["traffic"] = ratio[0] * kvb
            line["roofline"]["traffic_source"] = ratio[1]
        if not args.no_cpu_baseline:
            v, n, cores = cpu_oracle_calls_per_s(w, 10.0, 200)
            line["cpu_baseline"] = {"value": v, "unit": "calls/s", "cores": cores, "kind": "port",
                                    "sample": f"{n} whole calls of {w.name} by the fp32 CPU oracle (>=10 s of CPU work)"}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
