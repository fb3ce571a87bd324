#!/usr/bin/env python
"""Times the REFERENCE's own flash_decoding_attention (its Triton kernels and torch tail, loaded
from baseline/_ref/, see make_ref.py) beside this repository's operator: same process, same
seeded tensors, same stream, CUDA events.

    python baseline/triton_reference.py --workloads cfg2,cfg3,cfg4,cfg5 [--grid] [--json out.json]
    TRITON_INTERPRET=1 python baseline/triton_reference.py --interpret cfg1      # host cores

Rows per workload:
  full   the reference's whole call (flash_tree_attn.py:216-376), buffers pre-allocated and
         max_seq_len_in_batch passed, so that it neither allocates nor synchronises
  stages its two Triton launches only (:301-365), through its own host code: the call is given a
         current_k whose .transpose() raises, which is the first thing the torch tail does (:367)
  asis   the whole call with default arguments (allocates the mid buffers, reads the lengths back
         with .item(), :272-285), timed by the host clock around a synchronise
  ours   flash_tree_attn_b200.flash_decoding_attention on the same tensors

Where the reference cannot run a workload as written, the harness adapts the INPUTS, never a
Triton line: bf16 (the tail's hard-coded .half(), :370) -> the _anydtype copy; GQA (the tail's
matmul needs num_heads heads on current_k/v, :367) -> repeat_interleave; q_len 26 (block shapes
must be powers of two) -> the tree is padded to 32 nodes with zero rows that see only themselves,
and the first 26 rows are compared.  Each adaptation is named in the output.

This file is measurement tooling; nothing in the product imports it.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REF_DIR = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "flash_tree_attn_head.py"))


def load_ref(any_dtype: bool):
    name = "flash_tree_attn_head_anydtype" if any_dtype else "flash_tree_attn_head"
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF_DIR, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _StagesDone(Exception):
    pass


class _StopAfterStages:
    """Stands in for current_k: the reference touches it first at flash_tree_attn.py:367, after
    both Triton launches have been issued."""

    def transpose(self, *a):
        raise _StagesDone


def adapt_inputs(w, inp):
    """The reference's view of one call's tensors, plus the list of adaptations made."""
    import torch

    notes = []
    q, ck, cv, mask = inp["q"], inp["current_k"], inp["current_v"], inp["mask"]
    Q = w.Q
    Qp = 1 << (Q - 1).bit_length()
    if Qp != Q:
        notes.append(f"q_len {Q} padded to {Qp} (zero rows, each visible to itself only)")
        pad = lambda t: torch.cat([t, t.new_zeros(*t.shape[:2], Qp - Q, t.size(3))], dim=2)
        q, ck, cv = pad(q), pad(ck), pad(cv)
        m = torch.full((Qp, Qp), float("-inf"), dtype=torch.float32, device=mask.device)
        m[:Q, :Q] = mask if mask.dim() == 2 else mask.reshape(-1, Q, Q)[0]
        m[range(Q, Qp), range(Q, Qp)] = 0.0
        mask = m
    if w.G > 1:
        notes.append(f"current_k/v expanded to num_heads heads (repeat_interleave {w.G})")
        ck, cv = ck.repeat_interleave(w.G, dim=1), cv.repeat_interleave(w.G, dim=1)
    if mask.dim() == 3:
        mask = mask[:, None]
    if q.dtype != torch.float16:
        notes.append("bf16: tail cast `.half()` (:370) replaced by `.to(q.dtype)`")
    return dict(q=q.contiguous(), current_k=ck.contiguous(), current_v=cv.contiguous(), mask=mask, Qp=Qp), notes


def _events(fn, warmup, reps, flush=None):
    """Per-call CUDA-event times in ms (median, p20, p80) and the back-to-back average."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    ts.sort()
    q = lambda f: ts[min(len(ts) - 1, int(f * len(ts)))]
    return {"median_ms": statistics.median(ts), "p20_ms": q(0.2), "p80_ms": q(0.8),
            "back_to_back_ms": a.elapsed_time(b) / reps}


# The reference computes a block's cache offset as program_id * stride in 32-bit integers
# (flash_tree_attn.py:71-72: cur_token_idx * stride_kb + ...).  A cache of 2^31 elements or more makes
# that product wrap and the kernel read far outside the tensor: cfg5 whole (128 x 32 x 16384 x 128 =
# 8.6 G elements per cache) ended the process with a CUDA fault.  Such a workload is timed on its
# first power-of-two many sequences whose cache stays below 2^31 elements, ours on the same slice.
INT32_ELEMS = 1 << 31


def reference_sized(w):
    """(workload the reference can address, note or None)."""
    from flash_tree_attn_b200.workloads import draw_lengths, small

    per_seq = w.Hkv * w.ctx * w.D
    if w.B * per_seq < INT32_ELEMS:
        return w, None
    B = 1
    while 2 * B * per_seq < INT32_ELEMS and 2 * B <= w.B:
        B *= 2
    lens = draw_lengths(w)[:B]
    sub = small(w, B=B, lens="fixed:" + ",".join(map(str, lens)), name=f"{w.name}[first {B} sequences]")
    return sub, (f"first {B} of {w.B} sequences: the reference's 32-bit offset arithmetic (flash_tree_attn.py:71-72) "
                 f"cannot address a cache of {w.B * per_seq / 2**30:.1f} Gi elements")


def time_workload(w, warmup=5, reps=20, flush_l2=False, ours=True):
    import torch

    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200.workloads import draw_lengths, kv_bytes, make_inputs

    dev = torch.device("cuda")
    w, size_note = reference_sized(w)
    lens = draw_lengths(w)
    inp = make_inputs(w, dev, lens=lens)
    ad, notes = adapt_inputs(w, inp)
    if size_note:
        notes.append(size_note)
    ref = load_ref(any_dtype=w.dtype != torch.float16)
    B, H, D, Qp = w.B, w.H, w.D, ad["Qp"]
    S = (w.ctx + w.block_size - 1) // w.block_size
    mid_o = torch.empty((B, H, S, Qp, D), dtype=torch.float32, device=dev)
    mid_l = torch.empty((B, H, S, Qp), dtype=torch.float32, device=dev)
    output = torch.empty((B, H, Qp, D), dtype=w.dtype, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush_l2 else None

    def full():
        return ref.flash_decoding_attention(ad["q"], inp["k_cache"], inp["v_cache"], ad["current_k"], ad["current_v"],
                                            ad["mask"], inp["kv_seq_len"], w.block_size, w.ctx, output, mid_o, mid_l,
                                            None, w.G)

    stop = _StopAfterStages()

    def stages():
        try:
            ref.flash_decoding_attention(ad["q"], inp["k_cache"], inp["v_cache"], stop, None, None, inp["kv_seq_len"],
                                         w.block_size, w.ctx, output, mid_o, mid_l, None, w.G)
        except _StagesDone:
            pass

    def asis():
        return ref.flash_decoding_attention(ad["q"], inp["k_cache"], inp["v_cache"], ad["current_k"], ad["current_v"],
                                            ad["mask"], inp["kv_seq_len"], w.block_size, kv_group_num=w.G)

    res = {"workload": w.name, "sum_kv_len": int(sum(lens)), "kv_bytes": kv_bytes(w, lens), "adaptations": notes,
           "l2": "flushed between timed calls (256 MB write)" if flush_l2 else "inputs larger than L2"}
    ref_out = full()[:, :, :w.Q].float()
    torch.cuda.synchronize()
    res["full"] = _events(full, warmup, reps, flush)
    res["stages"] = _events(stages, warmup, reps, flush)
    for _ in range(2):
        asis()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_asis = max(3, reps // 4)
    for _ in range(n_asis):
        asis()
    torch.cuda.synchronize()
    res["asis"] = {"host_clock_ms": 1e3 * (time.perf_counter() - t0) / n_asis}
    del mid_o, mid_l
    if ours:
        prep = fta.prepare(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
                           inp["kv_seq_len"], w.block_size, w.ctx, kv_group_num=w.G)

        def mine():
            return fta.flash_decoding_attention(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"],
                                                inp["current_v"], inp["mask"], inp["kv_seq_len"], w.block_size, w.ctx,
                                                kv_group_num=w.G)

        my_out = mine().float()
        torch.cuda.synchronize()
        res["ours"] = _events(mine, warmup, reps, flush)                  # public call, validated every time
        res["ours_prepared"] = _events(prep.run, warmup, reps, flush)     # validated once
        res["max_abs_reference_vs_ours"] = (ref_out - my_out).abs().max().item()
        for k in ("full", "stages"):
            res[f"speedup_vs_{k}"] = res[k]["back_to_back_ms"] / res["ours"]["back_to_back_ms"]
    return res


def reference_grid(warmup=5, reps=20):
    """The reference's own benchmark grid (flash_tree_attn.py:442-483): B=2, H=32, D=128, q_len in
    {16,32,64,128}, N_CTX in {64,128,256}, fp16 N(0, 0.5), block 64, L2 flushed as its do_bench does."""
    import torch

    from flash_tree_attn_b200.workloads import Workload

    rows = []
    for q_len in (16, 32, 64, 128):
        for n_ctx in (64, 128, 256):
            w = Workload(f"grid_q{q_len}_ctx{n_ctx}", 2, 32, 1, 128, q_len, torch.float16, n_ctx, "full", "random",
                         scale=0.5, seed=4420 + q_len + n_ctx)
            r = time_workload(w, warmup, reps, flush_l2=True)
            rows.append({"q_len": q_len, "n_ctx": n_ctx,
                         "reference_full_ms": r["full"]["median_ms"], "reference_stages_ms": r["stages"]["median_ms"],
                         "ours_ms": r["ours"]["median_ms"], "max_abs_reference_vs_ours": r["max_abs_reference_vs_ours"]})
    return rows


def interpret(name: str, reps: int = 3):
    """The reference on the host cores under the Triton interpreter (TRITON_INTERPRET=1 must be in
    the environment before triton is imported).  The interpreter walks the launch grid serially in
    Python; numpy may use more cores inside a dot."""
    import torch

    from flash_tree_attn_b200.workloads import WORKLOADS, draw_lengths, make_inputs

    assert os.environ.get("TRITON_INTERPRET") == "1", "set TRITON_INTERPRET=1"
    w = WORKLOADS[name]
    assert w.dtype == torch.float16, "the interpreter cannot multiply bf16"
    lens = draw_lengths(w)
    inp = make_inputs(w, "cpu", lens=lens)
    ad, notes = adapt_inputs(w, inp)
    ref = load_ref(False)
    call = lambda: ref.flash_decoding_attention(ad["q"], inp["k_cache"], inp["v_cache"], ad["current_k"], ad["current_v"],
                                                ad["mask"], inp["kv_seq_len"], w.block_size, w.ctx, None, None, None,
                                                None, w.G)
    call()
    t0 = time.perf_counter()
    for _ in range(reps):
        call()
    dt = (time.perf_counter() - t0) / reps
    return {"workload": name, "calls_per_s": 1.0 / dt, "s_per_call": dt, "reps": reps, "cores": os.cpu_count(),
            "note": "reference under TRITON_INTERPRET=1, whole call; the interpreter runs the grid serially",
            "adaptations": notes}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workloads", default="cfg2,cfg3,cfg4,cfg5")
    ap.add_argument("--grid", action="store_true", help="also the reference's own benchmark grid")
    ap.add_argument("--interpret", default=None, metavar="WORKLOAD", help="host-core run under the Triton interpreter")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    if not available():
        print(json.dumps({"unavailable": "baseline/_ref/ is absent: run baseline/make_ref.py on a machine with the reference"}))
        return
    out = {}
    if args.interpret:
        out["interpreter"] = interpret(args.interpret)
    else:
        from flash_tree_attn_b200.workloads import WORKLOADS

        out["workloads"] = {}
        for name in [n for n in args.workloads.split(",") if n]:
            try:
                out["workloads"][name] = time_workload(WORKLOADS[name], args.warmup, args.reps)
            except Exception as e:  # a reference failure on one workload must not hide the others
                out["workloads"][name] = {"error": f"{type(e).__name__}: {e}"[:400]}
            import torch

            torch.cuda.empty_cache()
        if args.grid:
            out["reference_grid"] = reference_grid(args.warmup, args.reps)
    text = json.dumps(out)
    if args.json:
        with open(args.json, "w") as f:
            f.write(text)
    print(text)


if __name__ == "__main__":
    main()
