"""Caller-side pieces of a tree speculative-decoding loop around the operator: an attention layer
that owns its KV cache and runs verify -> accept -> commit, step after step.

The reference stops at the operator and lists "integration into transformers, medusa, glide" and
"kv cache management" as to do (README.md:60-64); its tree tokens stay outside the cache
(README.md:41-43).  This module is what a decoder's attention layer needs on top of
`flash_decoding_attention` to close that loop, written against plain torch interfaces only:

    layer = TreeVerifyAttention(num_heads, num_kv_heads, head_dim, max_batch, max_seq_len)
    layer.load_prefix(k_prompt, v_prompt, prompt_lens)          # after prefill
    for every decoding step:
        out = layer(q, k_new, v_new, mask)                      # verify: the tree's nodes attend to the
                                                                #   cache and, under the mask, to each other
        idx, n = accept_longest_path(tree, node_ok)             # caller's acceptance rule -> a root path
        layer.commit(idx, n)                                    # accepted nodes' K/V join the cache

Nothing here synchronises with the host: the lengths live on the device, the operator plans from
them on the device, and `commit` updates them in place, so a whole step can sit in a CUDA graph.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .op import commit_accepted, flash_decoding_attention, flash_decoding_attention_paged


class DraftTree:
    """A fixed draft-tree topology: parents[i] < i, parents[0] = -1 (node 0 is the root).

    Precomputes what a step needs on the device: the additive ancestor-or-self mask the operator
    takes (flash_tree_attn.py:368 adds it to the scores), the ancestor matrix, node depths and, per
    node, the root-to-node path."""

    def __init__(self, parents: Sequence[int], device="cuda", allowed: float = 0.0):
        parents = [int(p) for p in parents]
        assert parents and parents[0] == -1 and all(0 <= p < i for i, p in enumerate(parents) if i > 0)
        self.parents = parents
        Q = self.Q = len(parents)
        depth = [0] * Q
        for i in range(1, Q):
            depth[i] = depth[parents[i]] + 1
        self.max_depth = max(depth) + 1
        anc = torch.zeros((Q, Q), dtype=torch.bool)
        paths = torch.zeros((Q, self.max_depth), dtype=torch.int32)
        for i in range(Q):
            j, chain = i, []
            while j >= 0:
                anc[i, j] = True
                chain.append(j)
                j = parents[j]
            chain.reverse()
            paths[i, :len(chain)] = torch.tensor(chain, dtype=torch.int32)
        dev = torch.device(device)
        self.ancestors = anc.to(dev)                                   # [Q, Q] j is i or an ancestor of i
        self.paths = paths.to(dev)                                     # [Q, max_depth] root ... node, zero padded
        self.depth = torch.tensor(depth, dtype=torch.int32, device=dev)
        self.mask = torch.where(self.ancestors, float(allowed), float("-inf")).to(torch.float32)


def accept_longest_path(tree: DraftTree, node_ok: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """From per-node verdicts to the path to commit, on the device and without a host sync.

    node_ok [bsz, q_len] bool: whether the caller's rule accepts node i given its parent (for greedy
    verification: the token drafted at node i equals the model's choice at its parent).  A node can be
    committed only if it and all its ancestors are accepted; the deepest such node wins (lowest index
    among equals).  Returns (accept_idx [bsz, max_depth] int32: the path from the root in order,
    accept_len [bsz] int32: its length, 0 if even the root is rejected) as `commit` takes them."""
    ok = node_ok.to(torch.bool)
    Q = tree.Q
    assert ok.dim() == 2 and ok.size(1) == Q
    # rejected[b, i] = number of rejected nodes on the path to i
    rejected = (~ok).to(torch.float32) @ tree.ancestors.to(torch.float32).t()
    reach = rejected == 0
    score = torch.where(reach, tree.depth.to(torch.int64)[None] + 1, torch.zeros((), dtype=torch.int64, device=ok.device))
    best = torch.argmax(score * Q + (Q - 1 - torch.arange(Q, device=ok.device))[None], dim=1)
    n = score.gather(1, best[:, None])[:, 0].to(torch.int32)
    return tree.paths[best].contiguous(), n


class TreeVerifyAttention(torch.nn.Module):
    """The attention of one decoder layer during tree verification, with its KV cache.

    Dense cache: k_cache / v_cache [max_batch, num_kv_heads, max_seq_len, head_dim] right-padded per
    sequence, the layout the reference's operator reads (flash_tree_attn.py:238-239).  With
    `page_size` (a multiple of 64) the cache is a pool of pages and a block table, the layout the
    reference's docstring announces (:233); sequence b owns the pages block_table[b], handed out in a
    shuffled order at construction.

    forward() is the verify step and leaves the cache untouched; commit() appends the accepted
    nodes' keys and values (as given to the last forward) and grows kv_seq_len in place."""

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, max_batch: int, max_seq_len: int,
                 dtype: torch.dtype = torch.float16, device="cuda", page_size: Optional[int] = None,
                 sm_scale: Optional[float] = None, seed: int = 0):
        super().__init__()
        assert num_heads % num_kv_heads == 0
        self.H, self.Hkv, self.D = num_heads, num_kv_heads, head_dim
        self.G = num_heads // num_kv_heads
        self.max_seq_len = int(max_seq_len)
        self.sm_scale = sm_scale
        dev = torch.device(device)
        self.page_size = page_size
        if page_size is None:
            k = torch.zeros((max_batch, num_kv_heads, max_seq_len, head_dim), dtype=dtype, device=dev)
            table = None
        else:
            assert page_size % 64 == 0
            per_seq = -(-max_seq_len // page_size)
            g = torch.Generator().manual_seed(seed)
            order = torch.randperm(max_batch * per_seq, generator=g).to(torch.int32)
            table = order.view(max_batch, per_seq).to(dev)
            k = torch.zeros((max_batch * per_seq, num_kv_heads, page_size, head_dim), dtype=dtype, device=dev)
        self.register_buffer("k_cache", k, persistent=False)
        self.register_buffer("v_cache", torch.zeros_like(k), persistent=False)
        self.register_buffer("kv_seq_len", torch.zeros(max_batch, dtype=torch.int32, device=dev), persistent=False)
        self.register_buffer("block_table", table, persistent=False)
        self._last_kv = None

    @torch.no_grad()
    def load_prefix(self, k: torch.Tensor, v: torch.Tensor, lens: Sequence[int]) -> None:
        """Fill the cache after prefill: k, v [bsz, num_kv_heads, L, head_dim], lens[b] <= L rows count."""
        B = k.size(0)
        for b in range(B):
            n = int(lens[b])
            if self.block_table is None:
                self.k_cache[b, :, :n] = k[b, :, :n]
                self.v_cache[b, :, :n] = v[b, :, :n]
            else:
                ps = self.page_size
                for s in range(-(-n // ps)):
                    pg = int(self.block_table[b, s])
                    r0, r1 = s * ps, min((s + 1) * ps, n)
                    self.k_cache[pg, :, : r1 - r0] = k[b, :, r0:r1]
                    self.v_cache[pg, :, : r1 - r0] = v[b, :, r0:r1]
        self.kv_seq_len[:B] = torch.as_tensor(list(lens), dtype=torch.int32)

    @torch.no_grad()
    def forward(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """Verify: q [bsz, num_heads, q_len, head_dim], k_new / v_new [bsz, num_kv_heads, q_len, head_dim]
        of the draft tree's nodes, additive mask over the nodes.  Returns [bsz, num_heads, q_len, head_dim]."""
        B = q.size(0)
        lens = self.kv_seq_len[:B]
        self._last_kv = (k_new, v_new)
        if self.block_table is None:
            return flash_decoding_attention(q, self.k_cache[:B], self.v_cache[:B], k_new, v_new, mask, lens, 64,
                                            self.max_seq_len, sm_scale=self.sm_scale, kv_group_num=self.G)
        return flash_decoding_attention_paged(q, self.k_cache, self.v_cache, self.block_table[:B], k_new, v_new, mask, lens,
                                              self.max_seq_len, sm_scale=self.sm_scale, kv_group_num=self.G)

    @torch.no_grad()
    def commit(self, accept_idx: torch.Tensor, accept_len: torch.Tensor) -> None:
        """Append nodes accept_idx[b, :accept_len[b]] of the last forward's k_new / v_new to sequence
        b's cache rows kv_seq_len[b]..., and add accept_len to kv_seq_len, in place."""
        assert self._last_kv is not None, "commit() follows forward()"
        k_new, v_new = self._last_kv
        B = k_new.size(0)
        if self.block_table is None:
            commit_accepted(self.k_cache[:B], self.v_cache[:B], k_new, v_new, self.kv_seq_len[:B], accept_idx, accept_len,
                            kv_group_num=self.G)
        else:
            commit_accepted(self.k_cache, self.v_cache, k_new, v_new, self.kv_seq_len[:B], accept_idx, accept_len,
                            kv_group_num=self.G, block_table=self.block_table[:B])


def reference_path_walk(parents: Sequence[int], ok_row: Sequence[bool]) -> List[int]:
    """Plain-Python statement of accept_longest_path for one sequence (used by the tests)."""
    best: List[int] = []
    for i in range(len(parents)):
        chain, j, good = [], i, True
        while j >= 0:
            good = good and bool(ok_row[j])
            chain.append(j)
            j = parents[j]
        if good and len(chain) > len(best):
            best = chain[::-1]
    return best
