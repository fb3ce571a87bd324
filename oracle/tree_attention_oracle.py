"""TEST INFRASTRUCTURE ONLY — fp32 dense evaluation of tree-attention decode.

Parity status: PINNED.  tests/test_oracle.py checks this file against tests/golden/*.npz,
which hold outputs of the reference's own flash_decoding_attention executed in the
development container (Triton interpreter on CPU; generator: tests/golden/make_golden.py).

It follows the reference's dense checker torch_tree_attention (flash_tree_attn.py:388-397):
scores = q @ concat(cache, tree)^T * sm_scale, the additive mask is added to the last
q_len columns (:390-392), lse = logsumexp (:393), out = softmax @ concat(V) (:394-395); made
ragged-aware (rows at or past kv_seq_len[b] do not exist) and GQA-aware (query head h reads
KV head h // kv_group_num, flash_tree_attn.py:71).  Everything is computed in fp32.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch


def _mask_for(mask: torch.Tensor, b: int, H: int, Q: int) -> torch.Tensor:
    """-> [H or 1, Q, Q] fp32 mask of sequence b."""
    m = mask.float()
    if m.dim() == 2:
        return m[None]
    if m.dim() == 3:
        # torch broadcasting against [B,H,Q,Q] scores (flash_tree_attn.py:368) reads the first
        # dimension as heads; a first dimension that is not num_heads is read per sequence
        if m.size(0) == H and H > 1:
            return m
        return m[b if m.size(0) > 1 else 0][None]
    mb = m[b if m.size(0) > 1 else 0]
    return mb  # [H or 1, Q, Q]


def tree_attention_oracle(q, k_cache, v_cache, current_k, current_v, mask, kv_seq_len,
                          sm_scale: Optional[float] = None, kv_group_num: int = 1,
                          with_tree: bool = True, chunk: int = 16384) -> Dict[str, torch.Tensor]:
    """Returns fp32 tensors: out [B,H,Q,D], lse [B,H,Q] (merged softmax), cache_out,
    cache_lse (cache rows only; flash_tree_attn.py:340-365 leaves these in `output`),
    tree_out, tree_lse (tree tokens only; :367-371)."""
    B, H, Q, D = q.shape
    G = kv_group_num
    sm_scale = 1.0 / (D ** 0.5) if sm_scale is None else sm_scale
    lens = [int(x) for x in kv_seq_len.tolist()]
    dev = q.device
    out = torch.zeros((B, H, Q, D), dtype=torch.float32, device=dev)
    lse = torch.full((B, H, Q), float("-inf"), dtype=torch.float32, device=dev)
    c_out, c_lse = out.clone(), lse.clone()
    t_out, t_lse = out.clone(), lse.clone()
    for b in range(B):
        qb = q[b].float()  # [H,Q,D]
        L = min(lens[b], k_cache.size(2))
        # ---- cache part, chunked online accumulation in fp32 ----
        m = torch.full((H, Q), float("-inf"), dtype=torch.float32, device=dev)
        l = torch.zeros((H, Q), dtype=torch.float32, device=dev)
        acc = torch.zeros((H, Q, D), dtype=torch.float32, device=dev)
        for s in range(0, L, chunk):
            e = min(L, s + chunk)
            kb = k_cache[b, :, s:e].float().repeat_interleave(G, dim=0)  # [H,n,D]
            vb = v_cache[b, :, s:e].float().repeat_interleave(G, dim=0)
            sc = torch.matmul(qb, kb.transpose(1, 2)) * sm_scale  # [H,Q,n]
            mn = torch.maximum(m, sc.amax(dim=-1))
            p = torch.exp(sc - mn[..., None])
            a = torch.exp(m - mn)
            l = l * a + p.sum(-1)
            acc = acc * a[..., None] + torch.matmul(p, vb)
            m = mn
        if L > 0:
            c_out[b] = acc / l[..., None]
            c_lse[b] = m + torch.log(l)
        # ---- tree part ----
        if with_tree:
            hk = current_k.size(1)
            rep = H // hk
            ck = current_k[b].float().repeat_interleave(rep, dim=0)  # [H,Q,D]
            cv = current_v[b].float().repeat_interleave(rep, dim=0)
            sc = torch.matmul(qb, ck.transpose(1, 2)) * sm_scale + _mask_for(mask, b, H, Q).to(dev)
            t_lse[b] = torch.logsumexp(sc, dim=-1)
            t_out[b] = torch.matmul(torch.softmax(sc, dim=-1), cv)
        # ---- merge ----
        if with_tree and L > 0:
            tot = torch.logaddexp(c_lse[b], t_lse[b])
            wc = torch.exp(c_lse[b] - tot)[..., None]
            wt = torch.exp(t_lse[b] - tot)[..., None]
            out[b] = wc * c_out[b] + wt * t_out[b]
            lse[b] = tot
        elif with_tree:
            out[b], lse[b] = t_out[b], t_lse[b]
        else:
            out[b], lse[b] = c_out[b], c_lse[b]
    return {"out": out, "lse": lse, "cache_out": c_out, "cache_lse": c_lse, "tree_out": t_out, "tree_lse": t_lse}


def merge_partials_oracle(part_o: torch.Tensor, part_lse: torch.Tensor):
    """fp32 merge of n normalised partials: part_o [n, ..., D], part_lse [n, ...]; the
    closed form of the reference's stage-2 recurrence (flash_tree_attn.py:195-208)."""
    tot = torch.logsumexp(part_lse.float(), dim=0)
    w = torch.exp(part_lse.float() - tot[None])
    w = torch.nan_to_num(w, nan=0.0)
    return (w[..., None] * part_o.float()).sum(0), tot
