"""CPU restatement of the accept/commit step (test infrastructure only: imported by tests/, never by
the product path).

The reference has no code for this step (its README only says that the tree tokens are "not yet in
the cache" and lists cache management as to do), so there is nothing of it to follow or to pin
against: parity unpinned.  The rule restated here is the one include/fta.h states for
fta_commit_accepted: node accept_idx[b, i] (i < accept_len[b]) of the tree tokens becomes cache row
kv_seq_len[b] + i of every KV head; rows at or past ctx are dropped; lengths grow by the number
accepted and saturate at ctx.
"""
from __future__ import annotations

import torch


def commit_accepted_oracle(k_cache, v_cache, current_k, current_v, kv_seq_len, accept_idx, accept_len,
                           kv_group_num=1, block_table=None):
    """Returns (k_cache', v_cache', kv_seq_len') as new CPU tensors; plain loops."""
    k = k_cache.detach().cpu().clone()
    v = v_cache.detach().cpu().clone()
    ck = current_k.detach().cpu()
    cv = current_v.detach().cpu()
    lens = kv_seq_len.detach().cpu().clone()
    idx = accept_idx.detach().cpu()
    n_acc = accept_len.detach().cpu()
    table = None if block_table is None else block_table.detach().cpu()
    B = lens.numel()
    Hkv = k.size(1)
    page = k.size(2)
    ctx = page * table.size(1) if table is not None else k.size(2)
    Q = ck.size(2)
    mul = kv_group_num if ck.size(1) == Hkv * kv_group_num and kv_group_num > 1 else 1
    for b in range(B):
        n = min(int(n_acc[b]), idx.size(1))
        L = min(max(int(lens[b]), 0), ctx)
        for i in range(max(n, 0)):
            row, node = L + i, int(idx[b, i])
            if row >= ctx or node < 0 or node >= Q:
                continue
            for h in range(Hkv):
                if table is None:
                    k[b, h, row] = ck[b, h * mul, node]
                    v[b, h, row] = cv[b, h * mul, node]
                else:
                    pg = int(table[b, row // page])
                    k[pg, h, row % page] = ck[b, h * mul, node]
                    v[pg, h, row % page] = cv[b, h * mul, node]
        if n > 0:
            lens[b] = min(L + n, ctx)
    return k, v, lens
