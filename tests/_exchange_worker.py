"""Child process of the two-GPU exchange-merge test (one per GPU, started by torch.distributed.run).

Every rank owns a contiguous KV range of one long sequence.  The same call goes through the NCCL
path (all-gather of the packed partials, then fta_merge_parts) and through fta_exchange_merge over
peer-mapped memory; both fold the ranks' partials in rank order with the same arithmetic, so the
results must be identical bit for bit, many calls in a row (two alternating buffers, growing
epochs).  Both forms of the exchange are run, and the
result is also held against the fp32 oracle of the whole sequence.  Prints one line "EXCHANGE_OK <form> ..." per rank and form
on success.
"""
import os
import sys

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads only

import torch
import torch.distributed as dist


def main():
    ctx = int(sys.argv[1]) if len(sys.argv) > 1 else 8192
    iters = int(sys.argv[2]) if len(sys.argv) > 2 else 8
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from flash_tree_attn_b200 import dist as fdist
    from flash_tree_attn_b200.workloads import Workload, make_inputs

    w = Workload("xchg", 1, 64, 8, 128, 64, torch.bfloat16, ctx, "full", "random", seed=77)
    inp = make_inputs(w, dev)  # same seed: every rank draws the same tensors
    lo, hi = fdist.kv_ranges(ctx, world)[rank]
    k_sh, v_sh = inp["k_cache"][:, :, lo:hi], inp["v_cache"][:, :, lo:hi]
    shard_len = torch.tensor([hi - lo], dtype=torch.int32, device=dev)
    B, H, Q, D = inp["q"].shape
    for form in ("gather", "scatter"):
        one_form(form, fdist, dist, inp, w, k_sh, v_sh, shard_len, dev, rank, world, ctx, iters)
    dist.barrier()
    dist.destroy_process_group()


def one_form(form, fdist, dist, inp, w, k_sh, v_sh, shard_len, dev, rank, world, ctx, iters):
    B, H, Q, D = inp["q"].shape
    xch = fdist.PeerExchange(B * H * Q * D, B * H * Q, dev, timeout_s=2.0, form=form)

    def call(q, exchange):
        return fdist.kv_range_decode(q, k_sh, v_sh, inp["current_k"], inp["current_v"], inp["mask"], shard_len,
                                     w.block_size, w.G, exchange=exchange)

    gen = torch.Generator(device=dev).manual_seed(5)
    worst = 0.0
    for _ in range(iters):
        q = torch.randn(inp["q"].shape, generator=gen, device=dev, dtype=torch.float32).to(inp["q"].dtype)
        o_ref, l_ref = call(q, None)
        o_x, l_x = call(q, xch)
        xch.check()
        assert torch.equal(o_ref, o_x), f"rank {rank}: outputs differ, max {float((o_ref.float() - o_x.float()).abs().max())}"
        assert torch.equal(l_ref, l_x), f"rank {rank}: LSEs differ"
        worst = max(worst, float(o_x.float().abs().max()))
    assert worst > 0.0 and torch.isfinite(o_x.float()).all()

    # and against the fp32 oracle of the WHOLE sequence (every rank holds all of it here)
    from oracle.tree_attention_oracle import tree_attention_oracle

    ora = tree_attention_oracle(q, inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
                                inp["kv_seq_len"], None, w.G)
    eo = float((o_x.float() - ora["out"]).abs().max())
    el = float((l_x - ora["lse"]).abs().max())
    assert eo <= 2e-3 + 2.0 ** -8 * float(ora["out"].abs().max()) and el <= 1e-3, f"rank {rank}: {form}: out {eo} lse {el} off the oracle"

    # the prepared form gives the same bits, run after run, interleaved with plain calls
    prep = fdist.PreparedKvRange(inp["q"], k_sh, v_sh, inp["current_k"], inp["current_v"], inp["mask"], shard_len,
                                 w.block_size, w.G, exchange=xch)
    o_ref, l_ref = call(inp["q"], None)
    for i in range(5):
        o_p, l_p = prep.run()
        assert torch.equal(o_ref, o_p) and torch.equal(l_ref, l_p), f"rank {rank}: prepared run {i} differs"
        if i == 2:
            o_x, _ = call(inp["q"], xch)
            assert torch.equal(o_ref, o_x)
            o_p, l_p = None, None  # (scatter form: the views were overwritten by that call)
    xch.check()

    def timed(exchange, n=30):
        for _ in range(5):
            call(inp["q"], exchange)
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            call(inp["q"], exchange)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) * 1e3

    def timed_prepared(n=30):
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            prep.run()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) * 1e3

    us_nccl, us_x, us_p = timed(None), timed(xch), timed_prepared()
    xch.check()
    print(f"EXCHANGE_OK {form} rank {rank}/{world} ctx {ctx}: all-gather+merge {us_nccl:.1f} us/call, "
          f"exchange-merge {us_x:.1f} us/call, prepared {us_p:.1f} us/call", flush=True)
    xch.close()


if __name__ == "__main__":
    main()
