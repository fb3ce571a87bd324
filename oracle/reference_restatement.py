"""TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's own algorithm, step by
step and with its roundings, for buffer-level parity (mid_output, mid_output_lse, output).

Parity status: PINNED against tests/golden/*.npz (outputs of the reference executed in the
development container under the Triton interpreter; see tests/golden/make_golden.py).

Steps and where they come from:
  stage 1  one partial per block_size rows: S = q k^T, rows past kv_seq_len -> -inf, scale,
           m = rowmax, p = exp(S - m), l = rowsum, P rounded to the cache dtype, acc = P v,
           acc / l, lse = m + log l                      flash_tree_attn.py:92-144
  stage 2  serial online merge over ceil(L/block) partials; O and LSE rounded to the query
           dtype                                          flash_tree_attn.py:185-211
  tail     p = (q ck^T)*scale in the query dtype, p += mask, lse = logsumexp(p),
           p = softmax(p.float()) rounded to the query dtype, o = p cv
                                                          flash_tree_attn.py:367-371
  blend    out = O - sigmoid(lse_t - lse_c) * (O - o)     flash_tree_attn.py:373
Deviation, stated: the reference hard-codes `.half()` at :370, which makes bf16 inputs raise;
this restatement rounds to the query dtype instead so that bf16 cases have a definition.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch


def reference_restatement(q, k_cache, v_cache, current_k, current_v, mask, kv_seq_len,
                          block_size: int = 64, sm_scale: Optional[float] = None,
                          kv_group_num: int = 1) -> Dict[str, torch.Tensor]:
    B, H, Q, D = q.shape
    G = kv_group_num
    dt = q.dtype
    sm_scale = 1.0 / (D ** 0.5) if sm_scale is None else sm_scale
    lens = [int(x) for x in kv_seq_len.tolist()]
    S = (max(lens + [1]) + block_size - 1) // block_size
    mid_o = torch.full((B, H, S, Q, D), float("nan"), dtype=torch.float32)
    mid_lse = torch.full((B, H, S, Q), float("nan"), dtype=torch.float32)
    output = torch.zeros((B, H, Q, D), dtype=dt)
    output_lse = torch.zeros((B, H, Q, 1), dtype=dt)
    for b in range(B):
        nsp = (lens[b] + block_size - 1) // block_size
        qb = q[b].float()
        m_i = torch.full((H, Q), float("-inf"))
        l_i = torch.zeros((H, Q))
        acc = torch.zeros((H, Q, D))
        for s in range(nsp):
            lo = s * block_size
            n = min(block_size, lens[b] - lo)
            kb = k_cache[b, :, lo:lo + n].float().repeat_interleave(G, dim=0)
            vb = v_cache[b, :, lo:lo + n].float().repeat_interleave(G, dim=0)
            sc = torch.matmul(qb, kb.transpose(1, 2)) * sm_scale
            m = sc.amax(-1)
            p = torch.exp(sc - m[..., None])
            l = p.sum(-1)
            o = torch.matmul(p.to(dt).float(), vb) / l[..., None]
            lse = m + torch.log(l)
            mid_o[b, :, s] = o
            mid_lse[b, :, s] = lse
            # stage-2 recurrence
            m_new = torch.maximum(m_i, lse)
            scale = torch.exp(m_i - m_new)
            e = torch.exp(lse - m_new)
            acc = acc * scale[..., None] + e[..., None] * o
            l_i = scale * l_i + e
            m_i = m_new
        output[b] = (acc / l_i[..., None]).to(dt)
        output_lse[b] = (m_i + torch.log(l_i))[..., None].to(dt)
    # tail in the query dtype (emulated: fp32 math, rounded where the reference rounds)
    rep = H // current_k.size(1)
    ck = current_k.repeat_interleave(rep, dim=1)
    cv = current_v.repeat_interleave(rep, dim=1)
    p = (torch.matmul(q.float(), ck.float().transpose(2, 3)).to(dt).float() * sm_scale).to(dt)
    mk = mask.float()
    if mk.dim() == 3:
        mk = mk[:, None]
    p = (p.float() + mk).to(dt)
    cur_lse = torch.logsumexp(p.float(), dim=-1, keepdim=True).to(dt)
    pr = torch.softmax(p.float(), dim=-1).to(dt)
    cur_out = torch.matmul(pr.float(), cv.float()).to(dt)
    w = torch.sigmoid((cur_lse.float() - output_lse.float()).to(dt).float()).to(dt)
    diff = (output.float() - cur_out.float()).to(dt)
    out = (output.float() - (w.float() * diff.float()).to(dt).float()).to(dt)
    return {"out": out, "output": output, "output_lse": output_lse, "mid_o": mid_o, "mid_lse": mid_lse,
            "cur_out": cur_out, "cur_lse": cur_lse}
