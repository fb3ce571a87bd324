"""Accept/commit step (fta_commit_accepted): the CUDA kernels against the CPU restatement in
oracle/commit_oracle.py, bit for bit (it is a copy), dense and paged, plus the property that makes
it useful: attention over the grown cache equals attention over the old cache with the accepted
nodes still passed as tree tokens."""
import random

import pytest
import torch


def _case(B, Hkv, G, Q, D, ctx, dtype, seed, cur_heads="kv"):
    g = torch.Generator().manual_seed(seed)
    rng = random.Random(seed)
    lens = [rng.choice([0, 1, 63, 64, ctx - 3, ctx - 1, ctx, rng.randint(0, ctx)]) for _ in range(B)]
    k = torch.randn(B, Hkv, ctx, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, ctx, D, generator=g).to(dtype)
    hc = Hkv if cur_heads == "kv" else Hkv * G
    ck = torch.randn(B, hc, Q, D, generator=g).to(dtype)
    cv = torch.randn(B, hc, Q, D, generator=g).to(dtype)
    max_acc = min(Q, 6)
    n_acc = torch.tensor([rng.randint(0, max_acc) for _ in range(B)], dtype=torch.int32)
    idx = torch.tensor([[rng.randrange(Q) for _ in range(max_acc)] for _ in range(B)], dtype=torch.int32)
    return k, v, ck, cv, torch.tensor(lens, dtype=torch.int32), idx, n_acc


def test_commit_oracle_appends_rows_and_saturates():
    from oracle.commit_oracle import commit_accepted_oracle

    k, v, ck, cv, lens, idx, n_acc = _case(4, 2, 1, 8, 32, 128, torch.float16, 1)
    lens[0], n_acc[0] = 126, 5      # only two rows fit
    lens[1], n_acc[1] = 10, 0       # nothing accepted
    k2, v2, l2 = commit_accepted_oracle(k, v, ck, cv, lens, idx, n_acc)
    assert int(l2[0]) == 128 and int(l2[1]) == 10
    assert torch.equal(k2[0, :, 126], ck[0, :, int(idx[0, 0])]) and torch.equal(v2[0, :, 127], cv[0, :, int(idx[0, 1])])
    assert torch.equal(k2[1], k[1]) and torch.equal(k2[0, :, :126], k[0, :, :126])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 2, 1, 8, 64, 256, "kv"), (3, 2, 4, 26, 128, 320, "all"), (64, 8, 1, 4, 128, 128, "kv")])
def test_commit_matches_oracle_dense(shape, dtype):
    import flash_tree_attn_b200 as fta
    from oracle.commit_oracle import commit_accepted_oracle

    B, Hkv, G, Q, D, ctx, cur = shape
    k, v, ck, cv, lens, idx, n_acc = _case(B, Hkv, G, Q, D, ctx, dtype, B + Q, cur)
    ek, ev, el = commit_accepted_oracle(k, v, ck, cv, lens, idx, n_acc, kv_group_num=G)
    for len_dtype in (torch.int32, torch.int64):
        kd, vd, ld = k.cuda(), v.cuda(), lens.to(len_dtype).cuda()
        fta.commit_accepted(kd, vd, ck.cuda(), cv.cuda(), ld, idx.cuda(), n_acc.cuda(), kv_group_num=G)
        torch.cuda.synchronize()
        assert torch.equal(kd.cpu(), ek) and torch.equal(vd.cpu(), ev)
        assert torch.equal(ld.cpu().to(torch.int32), el.to(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("page_size", [64, 128])
def test_commit_matches_oracle_paged(page_size):
    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200.workloads import to_paged
    from oracle.commit_oracle import commit_accepted_oracle

    B, Hkv, G, Q, D, ctx = 6, 2, 2, 16, 64, 256
    k, v, ck, cv, lens, idx, n_acc = _case(B, Hkv, G, Q, D, ctx, torch.float16, 11)
    # every sequence owns all its pages here, so that the new rows have somewhere to go
    kp, vp, table = to_paged(k, v, [ctx] * B, page_size=page_size, seed=5, spare_pages=0)
    ek, ev, el = commit_accepted_oracle(kp, vp, ck, cv, lens, idx, n_acc, kv_group_num=G, block_table=table)
    kd, vd, ld = kp.cuda(), vp.cuda(), lens.cuda()
    fta.commit_accepted(kd, vd, ck.cuda(), cv.cuda(), ld, idx.cuda(), n_acc.cuda(), kv_group_num=G, block_table=table.cuda())
    torch.cuda.synchronize()
    assert torch.equal(kd.cpu(), ek) and torch.equal(vd.cpu(), ev) and torch.equal(ld.cpu(), el)


@pytest.mark.gpu
def test_attention_after_commit_equals_attention_with_accepted_nodes_as_a_chain():
    """Commit a root-to-leaf path, then ask a fresh single query about the grown cache: the answer
    must be what the oracle gives for the old cache followed by those rows."""
    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200.workloads import Workload, make_inputs
    from oracle.tree_attention_oracle import tree_attention_oracle

    w = Workload(name="t", B=3, H=4, G=2, D=128, Q=8, dtype=torch.float16, ctx=512, lens="fixed:300,64,17",
                 tree="random", seed=21)
    inp = make_inputs(w, "cuda")
    path = torch.tensor([[0, 1, 5, 0], [0, 2, 0, 0], [0, 3, 4, 7]], dtype=torch.int32, device="cuda")
    n_acc = torch.tensor([3, 2, 4], dtype=torch.int32, device="cuda")
    old = inp["kv_seq_len"].clone()
    fta.commit_accepted(inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["kv_seq_len"], path, n_acc,
                        kv_group_num=2)
    torch.cuda.synchronize()
    assert torch.equal(inp["kv_seq_len"].cpu(), (old.cpu() + n_acc.cpu()).to(old.dtype))
    # next step: one new node per sequence, attending to everything in the cache and to itself
    q1 = torch.randn(3, 4, 1, 128, device="cuda", dtype=torch.float16)
    k1 = torch.randn(3, 2, 1, 128, device="cuda", dtype=torch.float16)
    v1 = torch.randn(3, 2, 1, 128, device="cuda", dtype=torch.float16)
    m1 = torch.zeros(1, 1, device="cuda")
    out, lse = fta.flash_decoding_attention_with_lse(q1, inp["k_cache"], inp["v_cache"], k1, v1, m1, inp["kv_seq_len"], 64, 512,
                                                     kv_group_num=2)
    ora = tree_attention_oracle(q1, inp["k_cache"], inp["v_cache"], k1, v1, m1, inp["kv_seq_len"], None, 2)
    assert (out.float() - ora["out"]).abs().max().item() <= 2e-3 and (lse - ora["lse"]).abs().max().item() <= 1e-3
