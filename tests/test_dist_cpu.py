"""CPU: the multi-rank host logic (sharding, packing, one all-gather, merge) on two gloo ranks,
with the oracle standing in for the CUDA operator and merge kernel."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_golden


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_decode(q, k, v, ck, cv, mask, lens, block_size, G, with_tree):
    from oracle.tree_attention_oracle import tree_attention_oracle

    o = tree_attention_oracle(q, k, v, ck, cv, mask, lens, None, G, with_tree=with_tree)
    return o["out"], o["lse"]


def _oracle_merge(po, pl, out_dtype):
    from oracle.tree_attention_oracle import merge_partials_oracle

    o, l = merge_partials_oracle(po, pl)
    return o.to(out_dtype), l


def _oracle_decode_into(q, k, v, ck, cv, mask, lens, block_size, G, with_tree, out_buf=None, lse_buf=None):
    o, l = _oracle_decode(q, k, v, ck, cv, mask, lens, block_size, G, with_tree)
    out_buf.copy_(o)
    lse_buf.copy_(l)


class _GlooExchange:
    """Stand-in that follows PeerExchange's host protocol (epoch count, two alternating partial
    buffers, mine() before merge()); the peers' buffers are reached by a gloo all-gather instead of
    mapped memory.  A buffer is poisoned once merged, so a call that read a stale one would show."""

    scatter = False

    def __init__(self, no, nl):
        self.no, self.nl, self.epoch = no, nl, 0
        self.buf = torch.full((2, no + nl), float("nan"))

    def mine(self):
        b = self.buf[(self.epoch + 1) & 1]
        return b[:self.no], b[self.no:]

    def merge(self, o_shape, lse_shape, out_dtype, out=None, lse=None):
        from oracle.tree_attention_oracle import merge_partials_oracle

        self.epoch += 1
        mine = self.buf[self.epoch & 1]
        every = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(every, mine.clone())
        mine.fill_(float("nan"))
        po = torch.stack([e[:self.no].view(tuple(o_shape)) for e in every])
        pl = torch.stack([e[self.no:].view(tuple(lse_shape)) for e in every])
        o, l = merge_partials_oracle(po, pl)
        return o.to(out_dtype), l


def _exchange_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from flash_tree_attn_b200.dist import kv_range_decode, kv_ranges
        from oracle.tree_attention_oracle import tree_attention_oracle

        g = load_golden("cfg1")
        lens = g["kv_seq_len"]
        lo, hi = kv_ranges(g["k_cache"].size(2), world, align=16)[rank]
        shard_len = torch.clamp(lens - lo, min=0, max=hi - lo).to(torch.int32)
        B, H, Q, D = g["q"].shape
        xch = _GlooExchange(B * H * Q * D, B * H * Q)
        worst = 0.0
        for call in range(3):  # consecutive calls alternate between the two buffers
            q = g["q"].float() * (1.0 + 0.25 * call)
            out, lse = kv_range_decode(q, g["k_cache"][:, :, lo:hi], g["v_cache"][:, :, lo:hi], g["current_k"],
                                       g["current_v"], g["mask"], shard_len, 64, 1, out_dtype=torch.float32,
                                       decode_fn=_oracle_decode_into, exchange=xch)
            whole = tree_attention_oracle(q, g["k_cache"], g["v_cache"], g["current_k"], g["current_v"], g["mask"],
                                          lens, None, 1)
            worst = max(worst, (out - whole["out"]).abs().max().item(), (lse - whole["lse"]).abs().max().item())
        ret[rank] = (worst, xch.epoch)
    except Exception as e:
        ret[rank] = repr(e)
    finally:
        dist.destroy_process_group()


def test_kv_range_decode_through_an_exchange_object_two_ranks():
    """The exchange branch of kv_range_decode: the operator writes into the exchange's current
    buffer, merge() finishes the call, three calls in a row."""
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_exchange_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], tuple), ret[r]
        assert ret[r][0] < 1e-5 and ret[r][1] == 3


def _worker(rank, world, port, fail_rank, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from flash_tree_attn_b200.dist import kv_range_decode, kv_ranges
        from oracle.tree_attention_oracle import tree_attention_oracle

        g = load_golden("cfg1")
        lens = g["kv_seq_len"]
        ctx = g["k_cache"].size(2)
        lo, hi = kv_ranges(ctx, world, align=16)[rank]
        shard_len = torch.clamp(lens - lo, min=0, max=hi - lo).to(torch.int32)
        if rank == fail_rank:
            raise RuntimeError("injected failure before the collective")
        out, lse = kv_range_decode(g["q"], g["k_cache"][:, :, lo:hi], g["v_cache"][:, :, lo:hi], g["current_k"],
                                   g["current_v"], g["mask"], shard_len, 64, 1, out_dtype=torch.float32,
                                   decode_fn=_oracle_decode, merge_fn=_oracle_merge)
        whole = tree_attention_oracle(g["q"], g["k_cache"], g["v_cache"], g["current_k"], g["current_v"], g["mask"],
                                      lens, None, 1)
        ret[rank] = ((out - whole["out"]).abs().max().item(), (lse - whole["lse"]).abs().max().item())
    except Exception as e:  # the test inspects what each rank saw
        ret[rank] = repr(e)
    finally:
        dist.destroy_process_group()


def _run(world, fail_rank=-1):
    port = _free_port()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, port, fail_rank, ret), nprocs=world, join=True)
    return dict(ret)


def test_kv_range_decode_two_ranks_matches_whole_sequence():
    ret = _run(2)
    for r in range(2):
        assert isinstance(ret[r], tuple), ret[r]
        assert ret[r][0] < 1e-5 and ret[r][1] < 1e-5


def test_rank_failing_before_the_collective_is_reported_not_hung():
    """A rank that raises before the all-gather: the survivor's collective ends with an error
    (peer gone / process-group timeout) instead of hanging."""
    ret = _run(2, fail_rank=1)
    assert "injected failure" in ret[1]
    assert isinstance(ret[0], str), "the surviving rank must see an error, not a result"


def test_shard_batch_balances_ragged_lengths():
    from flash_tree_attn_b200.dist import shard_batch
    from flash_tree_attn_b200.workloads import WORKLOADS, draw_lengths

    lens = draw_lengths(WORKLOADS["cfg5"])
    for world in (2, 4, 8):
        parts = shard_batch(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(len(lens)))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= 1.1 * sum(lens) / world


def test_kv_ranges_cover_the_sequence():
    from flash_tree_attn_b200.dist import kv_ranges

    for L in (1, 63, 64, 100, 131072):
        for world in (1, 2, 4, 8):
            r = kv_ranges(L, world)
            assert r[0][0] == 0 and r[-1][1] == L
            assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
            assert all(lo % 64 == 0 for lo, _ in r if lo < L)


def test_exchange_layout_is_aligned_and_disjoint():
    """Two partial buffers, the result, its LSE and two flags per rank: every region on a 16-byte
    boundary, nothing overlapping."""
    from flash_tree_attn_b200 import dist as fdist

    for no, nl, world in [(8 * 64 * 128, 8 * 64, 2), (130, 13, 8), (4, 1, 3)]:
        L = fdist.exchange_layout(no, nl, world)
        assert all(x % 4 == 0 for x in L)
        assert L.stride >= no + nl and L.out == 2 * L.stride
        assert L.lse >= L.out + no and L.flags >= L.lse + nl and L.total >= L.flags + 2 * world


def test_batch_then_kv_head_shards_cover_the_job_once_and_reassemble():
    """Sharding by batch, then by KV head when sequences run out: every (sequence, KV head) pair
    lands on exactly one rank, and the ranks' results put side by side are the whole job's (the
    oracle stands in for the operator)."""
    import torch

    from flash_tree_attn_b200.dist import shard_batch_and_heads, take_heads
    from flash_tree_attn_b200.workloads import Workload, make_inputs
    from oracle.tree_attention_oracle import tree_attention_oracle

    for B, Hkv, G, world in ((8, 4, 2, 4), (2, 8, 1, 8), (3, 2, 4, 8), (1, 4, 2, 2), (5, 3, 1, 4)):
        lens = [17 + 31 * b for b in range(B)]
        shards = shard_batch_and_heads(lens, Hkv, world)
        assert len(shards) == world
        seen = {}
        for sh in shards:
            for b in sh.seqs:
                for h in range(sh.kv_lo, sh.kv_hi):
                    seen[(b, h)] = seen.get((b, h), 0) + 1
        assert seen == {(b, h): 1 for b in range(B) for h in range(Hkv)}, (B, Hkv, world)

    w = Workload("shard", 2, 8, 2, 32, 4, torch.float16, 128, "fixed:100,37", "random", seed=5)
    inp = make_inputs(w, "cpu")
    whole = tree_attention_oracle(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"],
                                  inp["mask"], inp["kv_seq_len"], None, w.G)["out"]
    got = torch.full_like(whole, float("nan"))
    for sh in shard_batch_and_heads(draw := [100, 37], w.Hkv, 8):
        if not sh.seqs:
            continue
        part = make_inputs(w, "cpu", lens=draw, seqs=sh.seqs)
        for n, mul in (("q", w.G), ("k_cache", 1), ("v_cache", 1), ("current_k", 1), ("current_v", 1)):
            part[n] = take_heads(part[n], sh.kv_lo, sh.kv_hi, mul)
        o = tree_attention_oracle(part["q"], part["k_cache"], part["v_cache"], part["current_k"], part["current_v"],
                                  part["mask"], part["kv_seq_len"], None, w.G)["out"]
        for i, b in enumerate(sh.seqs):
            got[b, sh.kv_lo * w.G:sh.kv_hi * w.G] = o[i]
    assert torch.equal(got, whole)
