"""The caller-side loop around the operator (flash_tree_attn_b200/speculative.py): verify ->
accept a root path -> commit -> next step on the grown cache.  The reference has no such code
(README.md:41-43,63 list it as to do), so the check is against the fp32 oracle evaluated, at every
step, on a cache kept by plain concatenation on the side."""
import random

import pytest
import torch


def test_accept_longest_path_matches_a_plain_walk():
    from flash_tree_attn_b200.speculative import DraftTree, accept_longest_path, reference_path_walk
    from flash_tree_attn_b200.workloads import tree_parents

    rng = random.Random(3)
    for kind, Q in (("topk", 64), ("random", 26), ("parents:-1,0,0,1", 4), ("random", 1)):
        parents = tree_parents(kind, Q, 11)
        tree = DraftTree(parents, device="cpu")
        ok = torch.tensor([[rng.random() < 0.7 for _ in range(Q)] for _ in range(50)])
        ok[0] = True
        ok[1] = False
        idx, n = accept_longest_path(tree, ok)
        for b in range(ok.size(0)):
            want = reference_path_walk(parents, ok[b].tolist())
            assert int(n[b]) == len(want)
            assert idx[b, : len(want)].tolist() == want
        assert torch.equal(tree.mask == 0, tree.ancestors)


@pytest.mark.gpu
@pytest.mark.parametrize("page_size", [None, 64, 128])
@pytest.mark.parametrize("H,Hkv,Q,dtype", [(8, 8, 16, torch.float16), (8, 2, 26, torch.bfloat16), (4, 4, 64, torch.float16)])
def test_verify_accept_commit_loop_matches_the_oracle_on_the_concatenated_cache(H, Hkv, Q, dtype, page_size):
    from flash_tree_attn_b200.speculative import DraftTree, TreeVerifyAttention, accept_longest_path
    from flash_tree_attn_b200.workloads import tree_parents
    from oracle.tree_attention_oracle import tree_attention_oracle

    B, D, ctx = 3, 128, 512
    G = H // Hkv
    g = torch.Generator(device="cuda").manual_seed(Q + H)
    rnd = lambda *shape: (torch.randn(shape, generator=g, device="cuda") * 0.7).to(dtype)
    layer = TreeVerifyAttention(H, Hkv, D, B, ctx, dtype=dtype, page_size=page_size, seed=5)
    lens = [300, 0, 61]
    k0, v0 = rnd(B, Hkv, max(lens), D), rnd(B, Hkv, max(lens), D)
    layer.load_prefix(k0, v0, lens)
    # the cache kept on the side: one [Hkv, L_b, D] tensor per sequence, grown by concatenation
    side_k = [k0[b, :, : lens[b]].clone() for b in range(B)]
    side_v = [v0[b, :, : lens[b]].clone() for b in range(B)]
    tree = DraftTree(tree_parents("random" if Q != 64 else "topk", Q, 7))
    for step in range(4):
        q, k_new, v_new = rnd(B, H, Q, D), rnd(B, Hkv, Q, D), rnd(B, Hkv, Q, D)
        out = layer(q, k_new, v_new, tree.mask)
        # oracle on the equivalent dense cache
        L = [t.size(1) for t in side_k]
        dk = torch.zeros((B, Hkv, max(max(L), 1), D), dtype=dtype, device="cuda")
        dv = torch.zeros_like(dk)
        for b in range(B):
            dk[b, :, : L[b]], dv[b, :, : L[b]] = side_k[b], side_v[b]
        ora = tree_attention_oracle(q, dk, dv, k_new, v_new, tree.mask, torch.tensor(L), None, G)
        ref = ora["out"]
        half_ulp = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}[dtype]
        excess = ((out.float() - ref).abs() - half_ulp * ref.abs()).max().item()
        # bf16 on a cache of a few dozen rows: every output is a sum of a handful of terms whose
        # weights P were rounded to 8 bits before P.V, as the reference rounds them
        # (flash_tree_attn.py:117); the randomised sweep saw up to 3.0e-3 there
        assert excess <= (2e-3 if dtype == torch.float16 else 4e-3), f"step {step}: {excess}"
        assert layer.kv_seq_len.tolist() == L
        # accept: random verdicts; sequence 1 accepts everything at step 0, sequence 2 nothing at step 1
        ok = torch.rand((B, Q), generator=g, device="cuda") < 0.8
        if step == 0:
            ok[1] = True
        if step == 1:
            ok[2, 0] = False
        idx, n = accept_longest_path(tree, ok)
        layer.commit(idx, n)
        for b in range(B):
            path = idx[b, : int(n[b])].long()
            side_k[b] = torch.cat([side_k[b], k_new[b][:, path]], dim=1)
            side_v[b] = torch.cat([side_v[b], v_new[b][:, path]], dim=1)
    assert layer.kv_seq_len.tolist() == [t.size(1) for t in side_k]
    assert max(t.size(1) for t in side_k) > max(lens)  # something was accepted
