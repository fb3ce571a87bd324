"""Multi-GPU use of the operator on one box: one process per GPU over torch.distributed.

Two partitionings, following how the work decomposes (every (sequence, KV head) pair is
independent, flash_tree_attn.py:49-51,71-73; the LSE merge is associative, :195-208):

* batched workloads: each rank takes a slice of the batch, no collective (`shard_batch`);
* one long sequence: each rank takes a contiguous KV range and produces an fp32 partial
  (O, LSE); the tree tokens are attached to the last rank's range; ONE all-gather of the
  packed partials, then the merge kernel on every rank (`kv_range_decode`).

  `kv_range_decode(..., exchange=PeerExchange(...))` replaces the all-gather and the merge by ONE
  kernel per rank that signals, waits (bounded) and reads the peers' partials over NVLink from
  memory the ranks mapped into each other once (`fta_exchange_merge`).

The packing, gather and merge are written against an injectable `decode_fn` / `merge_fn` so
that the host logic runs on CPU ranks (gloo) in the tests; on GPUs the defaults are the CUDA
operator and `fta_merge_parts`.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, NamedTuple, Optional, Sequence, Tuple

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


class Shard(NamedTuple):
    """What one rank of a batched job computes: these sequences, KV heads [kv_lo, kv_hi) of each
    (query heads [kv_lo * kv_group_num, kv_hi * kv_group_num))."""
    seqs: List[int]
    kv_lo: int
    kv_hi: int


def shard_batch_and_heads(lengths: Sequence[int], num_kv_heads: int, world_size: int) -> List[Shard]:
    """Batch first, then KV heads: with at least as many sequences as ranks every rank takes whole
    sequences (`shard_batch`); with fewer, the KV heads are cut into d parts, d the smallest power
    of two with len(lengths) * d >= world_size that divides both num_kv_heads and world_size, and the
    sequences are dealt to world_size / d groups of d ranks.  Every (sequence, KV head) pair is
    independent (flash_tree_attn.py:49-51,71-73), so no rank needs another's result."""
    B = len(lengths)
    d = 1
    while B * d < world_size and num_kv_heads % (2 * d) == 0 and world_size % (2 * d) == 0:
        d *= 2
    groups = shard_batch(lengths, world_size // d)
    per = num_kv_heads // d
    return [Shard(groups[r // d], (r % d) * per, (r % d + 1) * per) for r in range(world_size)]


def take_heads(t: torch.Tensor, lo: int, hi: int, mul: int = 1) -> torch.Tensor:
    """Heads [lo * mul, hi * mul) of a [bsz, heads, ...] tensor (a view)."""
    return t[:, lo * mul:hi * mul]


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


class ExchangeLayout(NamedTuple):
    """Offsets, in 4-byte words, inside one rank's peer-mapped allocation."""
    stride: int   # distance between the two packed partial buffers (each [numel_o + numel_lse] fp32)
    out: int      # merged result, numel_o elements of up to 4 bytes
    lse: int      # merged LSE, numel_lse fp32
    flags: int    # 2 * world uint32: first-round flags, then second-round flags
    total: int


def exchange_layout(numel_o: int, numel_lse: int, world: int) -> ExchangeLayout:
    """Every region starts on a 16-byte boundary."""
    up = lambda n: -(-n // 4) * 4
    stride = up(numel_o + numel_lse)
    out = 2 * stride
    lse = out + up(numel_o)
    flags = lse + up(numel_lse)
    return ExchangeLayout(stride, out, lse, flags, flags + up(2 * world))


class PeerExchange:
    """Peer-mapped partial buffers, result buffer and flags of the ranks of one box, for
    `fta_exchange_merge`.

    Construction is collective (every rank of `group`, same arguments).  The memory comes from
    torch.distributed._symmetric_memory: one allocation per rank, mapped into every peer by its
    rendezvous; only plain peer loads and stores are used on it.
    `form`: "gather" (every rank reads all partials and merges all rows; the results are new
    tensors), "scatter" (every rank merges its slice of the rows and stores it into every rank's
    result buffer; the results are views of that buffer, overwritten by the next call), or
    "auto": the gather form on 2 GPUs, the scatter form on 4 or more (the faster one where both were
    measured).
    The calls `mine()` ... `merge()` must come in the same order on every rank; the object counts
    the epoch and alternates between the two partial buffers itself.
    """

    def __init__(self, numel_o: int, numel_lse: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 timeout_s: float = 1.0, form: str = "auto"):
        import os

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > _lib.FTA_MAX_RANKS:
            raise ValueError(f"at most {_lib.FTA_MAX_RANKS} ranks")
        if form not in ("auto", "gather", "scatter"):
            raise ValueError(form)
        # measured on one box (one 131072-row sequence, µs per call, gather / scatter): 2 GPUs 177 / 183,
        # 4 GPUs 118 / 115, 8 GPUs 111 / 83: the gather form pulls (world - 1) whole partials per GPU
        self.scatter = form == "scatter" or (form == "auto" and self.world >= 4)
        self.no, self.nl = int(numel_o), int(numel_lse)
        self.layout = exchange_layout(self.no, self.nl, self.world)
        self.stride = self.layout.stride
        self.device = torch.device(device)
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        self._words = torch.zeros(3, dtype=torch.int32, device=self.device)  # status; finished blocks, waits lost in the launch
        self.status = self._words[:1]
        self._keep = []
        self._params = None
        # plain peer mappings only: no NVLink multicast object is bound to this memory
        if os.environ.get("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1") != "1":
            raise RuntimeError("PeerExchange needs TORCH_SYMM_MEM_DISABLE_MULTICAST=1: its buffers must be plain peer "
                               "mappings, never bound to an NVLink multicast object")
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
        self.local = symm_mem.empty(self.layout.total, dtype=torch.float32, device=self.device)
        self.local.zero_()
        hdl = symm_mem.rendezvous(self.local, self.group)
        self.base = [int(x) for x in hdl.buffer_ptrs]
        self._keep.append(hdl)
        assert self.base[self.rank] == self.local.data_ptr()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anyone signals

    def mine(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(O, LSE) flat fp32 views of the buffer this rank fills for the NEXT merge()."""
        off = ((self.epoch + 1) & 1) * self.stride
        return self.local[off:off + self.no], self.local[off + self.no:off + self.no + self.nl]

    def merge(self, o_shape, lse_shape, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
              lse: Optional[torch.Tensor] = None):
        """Signal, wait for the peers, merge all ranks' partials: (out, lse) on this rank.
        Gather form: written into `out` / `lse` (contiguous, of `out_dtype` / fp32) when given, else
        into new tensors.  Scatter form: views of this rank's peer-mapped result buffer, valid until
        the next merge(); `out` / `lse` are not used."""
        from . import _lib
        from .op import _DT

        self.epoch += 1
        D = int(o_shape[-1])
        assert self.nl * D == self.no
        L = self.layout
        if self.scatter:
            out = self.local[L.out:L.out + self.no].view(out_dtype)[:self.no].view(tuple(o_shape))
            lse = self.local[L.lse:L.lse + self.nl].view(tuple(lse_shape))
        else:
            if out is None:
                out = torch.empty(tuple(o_shape), dtype=out_dtype, device=self.device)
            if lse is None:
                lse = torch.empty(tuple(lse_shape), dtype=torch.float32, device=self.device)
            assert out.is_contiguous() and lse.is_contiguous() and out.dtype == out_dtype and lse.dtype == torch.float32
        p = self._params
        if p is None:
            p = self._params = _lib.FtaExchangeParams()
            for s in range(self.world):
                p.flag_peer[s] = self.base[s] + (L.flags + self.rank) * 4
                if self.scatter:
                    p.out_peer[s] = self.base[s] + L.out * 4
                    p.lse_peer[s] = self.base[s] + L.lse * 4
            p.flag_local = self.base[self.rank] + L.flags * 4
            p.status = self._words.data_ptr()
            p.done = self._words.data_ptr() + 4 if self.scatter else None
            p.timeout_ns = self.timeout_ns
            p.world, p.rank, p.rows = self.world, self.rank, self.nl
        off = (self.epoch & 1) * self.stride * 4
        for s in range(self.world):
            p.part[s] = self.base[s] + off
        p.epoch = self.epoch & 0xFFFFFFFF
        p.D, p.out_dtype = D, _DT[out_dtype]
        if not self.scatter:
            p.out, p.lse = out.data_ptr(), lse.data_ptr()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.load().fta_exchange_merge(C.byref(p), stream), "fta_exchange_merge")
        return out, lse

    def check(self) -> None:
        """Synchronise and raise if a wait for a peer ran out since the last check."""
        st = int(self.status.item())
        if st:
            self.status.zero_()
            late = sorted({s for s in range(self.world) if (st >> s & 1) or (st >> (8 + s) & 1)})
            raise TimeoutError(f"rank {self.rank}: no signal from rank(s) {late} within {self.timeout_ns / 1e9:.1f} s")

    def close(self) -> None:
        """Collective: nobody unmaps while a peer may still read."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._keep.clear()


class PreparedKvRange:
    """`kv_range_decode` through a PeerExchange, validated once: the operator call is prepared
    for each of the exchange's two buffers, the result tensors are allocated here, and `run()` is
    three launches (stage 1, stage 2, exchange-merge) with no other host work.  The input tensors
    may be overwritten in place between runs; every rank calls `run()` the same number of times.
    """

    def __init__(self, q, k_shard, v_shard, current_k, current_v, mask, shard_len, block_size: int = 64,
                 kv_group_num: int = 1, *, exchange: "PeerExchange", out_dtype: Optional[torch.dtype] = None):
        from .op import prepare

        B, H, Q, D = q.shape
        x = self.exchange = exchange
        assert x.no == B * H * Q * D and x.nl == B * H * Q
        self.calls = []
        for parity in (0, 1):
            off = parity * x.stride
            self.calls.append(prepare(
                q, k_shard, v_shard, current_k, current_v, mask, shard_len, block_size, None, kv_group_num=kv_group_num,
                want_lse=True, out_dtype=torch.float32, with_tree=x.rank == x.world - 1,
                out_buf=x.local[off:off + x.no].view(B, H, Q, D), lse_buf=x.local[off + x.no:off + x.no + x.nl].view(B, H, Q)))
        self.out_dtype = out_dtype or q.dtype
        self.o_shape, self.lse_shape = (B, H, Q, D), (B, H, Q)
        self.out = self.lse = None
        if not x.scatter:
            self.out = torch.empty(self.o_shape, dtype=self.out_dtype, device=q.device)
            self.lse = torch.empty(self.lse_shape, dtype=torch.float32, device=q.device)
        self.launches = 3

    def run(self):
        """(out, lse); the same tensors every time, overwritten by the next run."""
        x = self.exchange
        self.calls[(x.epoch + 1) & 1].run()
        return x.merge(self.o_shape, self.lse_shape, self.out_dtype, out=self.out, lse=self.lse)


def kv_range_decode(
    q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, current_k: torch.Tensor, current_v: torch.Tensor,
    mask: torch.Tensor, shard_len: torch.Tensor, block_size: int = 64, kv_group_num: int = 1,
    group: Optional[dist.ProcessGroup] = None, out_dtype: Optional[torch.dtype] = None,
    decode_fn: Callable = _default_decode, merge_fn: Callable = _default_merge,
    exchange: Optional["PeerExchange"] = None,
):
    """Sequence-split decode.  Every rank passes the same q / current_k / current_v / mask and
    ITS OWN KV rows (`k_shard`, `v_shard`: [B, Hkv, rows_of_this_rank, D]; `shard_len` [B]: how
    many of them are real).  Returns (out, lse) on every rank.

    The tree tokens are counted once: only the last rank's partial includes them.
    """
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    B, H, Q, D = q.shape
    if exchange is not None:
        # the operator writes its partial into this rank's peer-mapped buffer; one kernel then
        # signals, waits for the peers and merges what it reads from them
        mo, ml = exchange.mine()
        decode_fn(q, k_shard, v_shard, current_k, current_v, mask, shard_len, block_size, kv_group_num,
                  rank == world - 1, out_buf=mo.view(B, H, Q, D), lse_buf=ml.view(B, H, Q))
        out, lse = exchange.merge((B, H, Q, D), (B, H, Q), out_dtype or q.dtype)
        # scatter form: the result sits in the exchange's buffer and the next call overwrites it
        return (out.clone(), lse.clone()) if exchange.scatter else (out, lse)
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
