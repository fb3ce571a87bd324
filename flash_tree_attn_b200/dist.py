"""Multi-GPU use of the operator on one box: one process per GPU over torch.distributed.

Two partitionings, following how the work decomposes (every (sequence, KV head) pair is
independent, flash_tree_attn.py:49-51,71-73; the LSE merge is associative, :195-208):

* batched workloads: each rank takes a slice of the batch, no collective (`shard_batch`);
* one long sequence: each rank takes a contiguous KV range and produces an fp32 partial
  (O, LSE); the tree tokens are attached to the last rank's range; ONE all-gather of the
  packed partials, then the merge kernel on every rank (`kv_range_decode`).

The packing, gather and merge are written against an injectable `decode_fn` / `merge_fn` so
that the host logic runs on CPU ranks (gloo) in the tests; on GPUs the defaults are the CUDA
operator and `fta_merge_parts`.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_batch(lengths: Sequence[int], world_size: int) -> List[List[int]]:
    """Assign sequences to ranks so that sum(kv_seq_len) per rank is balanced (greedy longest-
    first); returns the sequence indices of every rank, each list sorted."""
    order = sorted(range(len(lengths)), key=lambda i: -int(lengths[i]))
    load = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], len(out[k])))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(x) for x in out]


def kv_ranges(kv_len: int, world_size: int, align: int = 64) -> List[Tuple[int, int]]:
    """Contiguous KV row ranges [lo, hi) per rank, boundaries rounded to `align` rows."""
    per = -(-kv_len // world_size)
    per = -(-per // align) * align
    return [(min(kv_len, r * per), min(kv_len, (r + 1) * per)) for r in range(world_size)]


def pack_partial(o: torch.Tensor, lse: torch.Tensor) -> torch.Tensor:
    """(O [..,D] fp32, LSE [..] fp32) -> one flat fp32 buffer [numel(O) + numel(LSE)]."""
    return torch.cat([o.reshape(-1).float(), lse.reshape(-1).float()])


def unpack_partials(buf: torch.Tensor, n: int, o_shape, lse_shape):
    """[n * (|O|+|LSE|)] -> (O [n, *o_shape], LSE [n, *lse_shape]) views."""
    no = 1
    for d in o_shape:
        no *= d
    nl = 1
    for d in lse_shape:
        nl *= d
    buf = buf.view(n, no + nl)
    return buf[:, :no].reshape(n, *o_shape), buf[:, no:].reshape(n, *lse_shape)


def _default_decode(q, k, v, ck, cv, mask, lens, block_size, kv_group_num, with_tree, out_buf=None, lse_buf=None):
    from .op import flash_decoding_attention_with_lse

    return flash_decoding_attention_with_lse(q, k, v, ck, cv, mask, lens, block_size, None, kv_group_num=kv_group_num,
                                             out_dtype=torch.float32, with_tree=with_tree, out_buf=out_buf,
                                             lse_buf=lse_buf)


_gather_bufs = {}  # (device, world, numel) -> (mine, gathered), reused across calls


def _default_merge(po, pl, out_dtype):
    from .op import merge_partials

    return merge_partials(po, pl, out_dtype)


def kv_range_decode(
    q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, current_k: torch.Tensor, current_v: torch.Tensor,
    mask: torch.Tensor, shard_len: torch.Tensor, block_size: int = 64, kv_group_num: int = 1,
    group: Optional[dist.ProcessGroup] = None, out_dtype: Optional[torch.dtype] = None,
    decode_fn: Callable = _default_decode, merge_fn: Callable = _default_merge,
):
    """Sequence-split decode.  Every rank passes the same q / current_k / current_v / mask and
    ITS OWN KV rows (`k_shard`, `v_shard`: [B, Hkv, rows_of_this_rank, D]; `shard_len` [B]: how
    many of them are real).  Returns (out, lse) on every rank.

    The tree tokens are counted once: only the last rank's partial includes them.
    """
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    B, H, Q, D = q.shape
    if decode_fn is _default_decode:
        # the operator writes its partial straight into this rank's slot of the packed buffer
        no, nl = B * H * Q * D, B * H * Q
        key = (q.device, world, no + nl)
        if key not in _gather_bufs:
            _gather_bufs[key] = (torch.empty(no + nl, dtype=torch.float32, device=q.device),
                                 torch.empty(world * (no + nl), dtype=torch.float32, device=q.device))
        mine, gathered = _gather_bufs[key]
        o, lse = decode_fn(q, k_shard, v_shard, current_k, current_v, mask, shard_len, block_size, kv_group_num,
                           rank == world - 1, out_buf=mine[:no].view(B, H, Q, D), lse_buf=mine[no:].view(B, H, Q))
    else:
        o, lse = decode_fn(q, k_shard, v_shard, current_k, current_v, mask, shard_len, block_size, kv_group_num,
                           rank == world - 1)
        mine = pack_partial(o, lse)
        gathered = torch.empty(world * mine.numel(), dtype=torch.float32, device=mine.device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    po, pl = unpack_partials(gathered, world, tuple(o.shape), tuple(lse.shape))
    return merge_fn(po, pl, out_dtype or q.dtype)
