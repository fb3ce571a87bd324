"""GPU: the CUDA path (through the C ABI) against the fp32 oracle, the reference-output
fixtures and the reference restatement.  Tolerances are the ones the operator is specified
to: max-abs 2e-3 on fp16/bf16 outputs and 1e-3 on the LSE, both against an fp32 evaluation
of the same masked attention."""
import pytest
import torch

from conftest import GOLDEN, load_golden

pytestmark = pytest.mark.gpu

OUT_TOL = 2e-3
KERNELS = ["mma", "auto"]  # "auto" takes the tcgen05 family wherever it applies
LSE_TOL = 1e-3


@pytest.fixture(scope="module")
def fta():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import flash_tree_attn_b200 as m
    from flash_tree_attn_b200 import _lib

    _lib.load()  # raises if libfta.so is absent: there is no fallback to test
    yield m
    m.set_split_mode("balanced")
    m.set_kernel("auto")
    m.set_grid_override(0)


def _oracle(inp, G, with_tree=True):
    from oracle.tree_attention_oracle import tree_attention_oracle

    return tree_attention_oracle(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"],
                                 inp["mask"], inp["kv_seq_len"], None, G, with_tree=with_tree)


def _run(fta, inp, G, block_size=64, ctx=None, **kw):
    from flash_tree_attn_b200 import _lib

    res = fta.flash_decoding_attention_with_lse(
        inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
        inp["kv_seq_len"], block_size, ctx, kv_group_num=G, **kw)
    torch.cuda.synchronize()
    # a bounded barrier wait that gave up inside the tcgen05 kernel shows here, not as a hang
    assert _lib.load().fta_umma_status() == 0, "tcgen05 stage-1 kernel reported a barrier timeout"
    return res


def _check(out, lse, ora, tag=""):
    """2e-3 on the output, plus half a unit in the last place of the output dtype where a
    value is large enough for its own rounding to exceed that (short sequences give |o| ~ 1,
    and bf16 keeps 8 bits); 1e-3 on the LSE."""
    assert out.dtype in (torch.float16, torch.bfloat16, torch.float32)
    ref = ora["out"]
    half_ulp = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8, torch.float32: 0.0}[out.dtype]
    excess = ((out.float() - ref).abs() - half_ulp * ref.abs()).max().item()
    eo = (out.float() - ref).abs().max().item()
    el = (lse - ora["lse"]).abs().max().item()
    assert torch.isfinite(out.float()).all(), tag
    assert excess <= OUT_TOL, f"{tag}: out max-abs {eo} (beyond output rounding: {excess})"
    assert el <= LSE_TOL, f"{tag}: lse max-abs {el}"
    return eo, el


def _workload(**kw):
    from flash_tree_attn_b200.workloads import Workload

    base = dict(name="t", B=2, H=8, G=1, D=128, Q=8, dtype=torch.float16, ctx=256, lens="fixed:200,37",
                tree="random", seed=99)
    base.update(kw)
    return Workload(**base)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", GOLDEN)
def test_golden_fixtures(fta, name, kernel):
    fta.set_kernel(kernel)
    g = load_golden(name)
    inp = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in g.items()}
    out, lse = _run(fta, inp, g["kv_group_num"], g["block_size"])
    ora = _oracle(inp, g["kv_group_num"])
    _check(out, lse, ora, name)
    # and against what the reference itself returned for these inputs (its own error included)
    assert (out.float() - inp["ref_out"].float()).abs().max().item() <= 3e-3
    # the drop-in entry point returns the same tensor
    out2 = fta.flash_decoding_attention(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"],
                                        inp["mask"], inp["kv_seq_len"], g["block_size"], kv_group_num=g["kv_group_num"])
    assert out2.dtype == inp["q"].dtype and out2.shape == inp["q"].shape
    assert torch.equal(out2, out)


SHAPES = [
    # (B, H, G, D, Q, ctx, lens)
    (2, 8, 1, 64, 8, 128, "fixed:100,37"),
    (3, 4, 1, 128, 4, 512, "fixed:16,500,129"),
    (2, 8, 4, 128, 26, 1024, "fixed:1000,333"),
    (2, 4, 1, 128, 64, 1024, "fixed:1024,700"),
    (1, 16, 8, 128, 64, 2048, "fixed:2048"),
    (2, 4, 2, 32, 16, 256, "fixed:255,64"),
    (1, 2, 1, 256, 16, 256, "fixed:130"),
    (2, 2, 1, 128, 128, 512, "fixed:512,65"),
    (5, 6, 3, 64, 7, 320, "fixed:1,63,64,65,320"),
    (2, 2, 1, 128, 100, 256, "fixed:256,10"),
]


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_shapes_against_oracle(fta, shape, dtype, kernel):
    from flash_tree_attn_b200.workloads import make_inputs

    fta.set_kernel(kernel)
    B, H, G, D, Q, ctx, lens = shape
    w = _workload(B=B, H=H, G=G, D=D, Q=Q, ctx=ctx, lens=lens, dtype=dtype, scale=0.5 if dtype == torch.bfloat16 else 1.0)
    inp = make_inputs(w, "cuda")
    out, lse = _run(fta, inp, G, ctx=ctx)
    _check(out, lse, _oracle(inp, G), str(shape))


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("grid", [1, 3, 37, 148, 1000])
def test_result_independent_of_split_count(fta, grid, kernel):
    from flash_tree_attn_b200.workloads import make_inputs

    fta.set_kernel(kernel)
    w = _workload(B=3, H=8, G=2, D=128, Q=32, ctx=2048, lens="fixed:2048,900,3")
    inp = make_inputs(w, "cuda")
    ora = _oracle(inp, 2)
    fta.set_grid_override(grid)
    out, lse = _run(fta, inp, 2)
    fta.set_grid_override(0)
    _check(out, lse, ora, f"grid={grid}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("B,Q,G", [(96, 64, 1), (40, 26, 4), (700, 64, 1)])
def test_many_short_sequences(fta, B, Q, G, kernel):
    """Dozens of units per block, most of them one or two tiles long: every block ends many
    units, the ring of piece descriptors wraps, and (B = 700) the prefix table of the lengths is
    large."""
    from flash_tree_attn_b200.workloads import make_inputs
    import random

    fta.set_kernel(kernel)
    rng = random.Random(B)
    lens = [rng.choice([0, 1, 5, 63, 64, 65, 100, 130, 200]) for _ in range(B)]
    w = _workload(B=B, H=2 * G, G=G, D=128, Q=Q, ctx=256, lens="fixed:" + ",".join(map(str, lens)))
    inp = make_inputs(w, "cuda")
    out, lse = _run(fta, inp, G, ctx=256)
    _check(out, lse, _oracle(inp, G), f"B={B} Q={Q} G={G}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("B,Q,G,Hkv,long_len", [(40, 26, 4, 4, 30000), (160, 64, 1, 1, 20000), (150, 4, 1, 2, 24000)])
def test_one_long_sequence_among_many_short_ones(fta, B, Q, G, Hkv, long_len, kernel):
    """As many units as stage-1 blocks or more, so the merge asks for a cut unit's first two pieces
    before it has read the cut's descriptor, while one sequence is long enough for its units to be
    cut into many pieces: pieces 2.. come after the descriptor, in the same order."""
    from flash_tree_attn_b200.workloads import make_inputs
    import random

    fta.set_kernel(kernel)
    rng = random.Random(B + Q)
    lens = [rng.choice([1, 30, 64, 65, 100, 130]) for _ in range(B)]
    lens[B // 3] = long_len
    ctx = -(-long_len // 64) * 64
    w = _workload(B=B, H=Hkv * G, G=G, D=128, Q=Q, ctx=ctx, lens="fixed:" + ",".join(map(str, lens)))
    inp = make_inputs(w, "cuda")
    out, lse = _run(fta, inp, G, ctx=ctx)
    _check(out, lse, _oracle(inp, G), f"B={B} Q={Q} G={G} long={long_len}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("page_size", [64, 128])
@pytest.mark.parametrize("shape", [(3, 4, 1, 128, 4, 512, "fixed:16,500,129"), (2, 8, 4, 128, 26, 1024, "fixed:1000,333"),
                                   (2, 4, 1, 128, 64, 1024, "fixed:1024,0"), (2, 4, 2, 64, 16, 256, "fixed:255,64")])
def test_paged_cache_matches_dense_cache(fta, shape, page_size, kernel):
    """The same rows housed in shuffled pages give the same bits as the dense cache (the page
    lookup changes addresses only), and agree with the oracle; pages nobody references and rows
    past a sequence's length inside its last page are NaN and must not matter."""
    from flash_tree_attn_b200.workloads import make_inputs, to_paged

    fta.set_kernel(kernel)
    B, H, G, D, Q, ctx, lens = shape
    w = _workload(B=B, H=H, G=G, D=D, Q=Q, ctx=ctx, lens=lens)
    inp = make_inputs(w, "cuda")
    dense, dense_lse = _run(fta, inp, G, ctx=ctx)
    L = [int(x) for x in inp["kv_seq_len"].tolist()]
    kp, vp, table = to_paged(inp["k_cache"], inp["v_cache"], L, page_size=page_size, seed=page_size + B)
    out, lse = fta.flash_decoding_attention_paged(inp["q"], kp, vp, table, inp["current_k"], inp["current_v"], inp["mask"],
                                                  inp["kv_seq_len"], kv_group_num=G, return_lse=True)
    torch.cuda.synchronize()
    assert torch.equal(out, dense) and torch.equal(lse, dense_lse)
    _check(out, lse, _oracle(inp, G), f"paged {shape} page={page_size}")


@pytest.mark.parametrize("kernel", KERNELS)
def test_padding_rows_are_never_read(fta, kernel):
    """NaN in every cache row at or past kv_seq_len must not reach the result (the reference
    needs finite padding, flash_tree_attn.py:93-94)."""
    from flash_tree_attn_b200.workloads import make_inputs

    fta.set_kernel(kernel)
    w = _workload(B=2, H=4, G=1, D=128, Q=64, ctx=512, lens="fixed:301,64")
    inp = make_inputs(w, "cuda", pad_value=float("nan"))
    out, lse = _run(fta, inp, 1)
    clean = dict(inp)
    clean["k_cache"] = torch.nan_to_num(inp["k_cache"], nan=0.0)
    clean["v_cache"] = torch.nan_to_num(inp["v_cache"], nan=0.0)
    _check(out, lse, _oracle(clean, 1), "nan padding")


def test_zero_length_sequence_is_tree_only(fta):
    from flash_tree_attn_b200.workloads import make_inputs

    w = _workload(B=2, H=4, G=1, D=64, Q=8, ctx=128, lens="fixed:0,77")
    inp = make_inputs(w, "cuda")
    out, lse = _run(fta, inp, 1)
    ora = _oracle(inp, 1)
    _check(out, lse, ora, "L=0")
    assert (out[0].float() - ora["tree_out"][0]).abs().max().item() <= OUT_TOL


def test_int64_lengths_and_strided_views(fta):
    """The reference's benchmark passes sliced cache views (flash_tree_attn.py:483) and its
    test int64 lengths (:434)."""
    from flash_tree_attn_b200.workloads import make_inputs

    w = _workload(B=2, H=4, G=1, D=128, Q=16, ctx=384, lens="fixed:256,100")
    inp = make_inputs(w, "cuda")
    big_k = torch.randn(2, 4, 384 + 16, 128, device="cuda").half()
    big_v = torch.randn(2, 4, 384 + 16, 128, device="cuda").half()
    inp["k_cache"], inp["current_k"] = big_k[:, :, :384], big_k[:, :, 384:]
    inp["v_cache"], inp["current_v"] = big_v[:, :, :384], big_v[:, :, 384:]
    inp["kv_seq_len"] = inp["kv_seq_len"].long()
    assert not inp["k_cache"].is_contiguous()
    out, lse = _run(fta, inp, 1)
    _check(out, lse, _oracle(inp, 1), "strided")


@pytest.mark.parametrize("mask_kind", ["2d", "3d", "3d_heads", "4d_b1", "4d_bh", "ones"])
def test_mask_forms(fta, mask_kind):
    """Additive mask semantics: any finite allowed value is added (the reference's test uses
    1.0, flash_tree_attn.py:409), and every broadcastable shape is accepted."""
    from flash_tree_attn_b200.workloads import ancestor_mask, make_inputs, tree_parents

    w = _workload(B=2, H=4, G=2, D=64, Q=16, ctx=128, lens="fixed:128,50")
    inp = make_inputs(w, "cuda")
    m = ancestor_mask(tree_parents("random", 16, 3), 1.0 if mask_kind == "ones" else 0.0).cuda()
    if mask_kind == "3d":
        m = torch.stack([m, ancestor_mask(tree_parents("random", 16, 4)).cuda()])
    elif mask_kind == "3d_heads":  # [num_heads, Q, Q]: torch broadcasting against [B,H,Q,Q], as in the reference
        m = torch.stack([ancestor_mask(tree_parents("random", 16, 20 + h)).cuda() for h in range(4)])
    elif mask_kind == "4d_b1":
        m = torch.stack([m, ancestor_mask(tree_parents("random", 16, 5)).cuda()])[:, None]
    elif mask_kind == "4d_bh":
        m = torch.stack([torch.stack([ancestor_mask(tree_parents("random", 16, 10 * b + h)) for h in range(4)])
                         for b in range(2)]).cuda()
        m = m + 0.25 * torch.isfinite(m) * torch.randn_like(m).nan_to_num(0.0)
        m = torch.where(torch.isnan(m), torch.full_like(m, float("-inf")), m)
    inp["mask"] = m
    out, lse = _run(fta, inp, 2)
    _check(out, lse, _oracle(inp, 2), mask_kind)


def test_current_kv_with_all_query_heads(fta):
    """current_k/v given with num_heads heads, replicated per group, as the reference's tail
    requires under GQA (flash_tree_attn.py:367)."""
    from flash_tree_attn_b200.workloads import make_inputs

    w = _workload(B=2, H=8, G=4, D=128, Q=8, ctx=128, lens="fixed:128,9")
    inp = make_inputs(w, "cuda")
    ora = _oracle(inp, 4)
    inp["current_k"] = inp["current_k"].repeat_interleave(4, dim=1)
    inp["current_v"] = inp["current_v"].repeat_interleave(4, dim=1)
    out, lse = _run(fta, inp, 4)
    _check(out, lse, ora, "expanded current kv")


@pytest.mark.parametrize("kernel", KERNELS)
def test_output_argument_receives_cache_only_attention(fta, kernel):
    """Like the reference, `output` ends up holding the cache-only attention and the
    returned tensor is a different one (flash_tree_attn.py:340-376)."""
    from flash_tree_attn_b200.workloads import make_inputs

    fta.set_kernel(kernel)
    w = _workload(B=2, H=4, G=1, D=128, Q=16, ctx=1024, lens="fixed:1000,130")
    inp = make_inputs(w, "cuda")
    output = torch.full((2, 4, 16, 128), float("nan"), dtype=torch.float16, device="cuda")
    out, lse = _run(fta, inp, 1, output=output)
    ora = _oracle(inp, 1)
    _check(out, lse, ora, "with output")
    assert out.data_ptr() != output.data_ptr()
    assert (output.float() - ora["cache_out"]).abs().max().item() <= OUT_TOL


@pytest.mark.parametrize("name", GOLDEN)
def test_block_mode_fills_mid_buffers_like_the_reference(fta, name):
    """Split mode "block": mid_output / mid_output_lse hold one partial per block_size rows
    exactly where the reference's stage 1 writes them (flash_tree_attn.py:124-144), slots
    past a sequence stay untouched, and `output` holds the stage-2 result."""
    g = load_golden(name)
    inp = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in g.items()}
    B, H, Q, D = inp["q"].shape
    bs = g["block_size"]
    S = inp["ref_mid_o"].shape[2]
    mid_o = torch.full((B, H, S, Q, D), float("nan"), device="cuda")
    mid_l = torch.full((B, H, S, Q), float("nan"), device="cuda")
    output = torch.zeros((B, H, Q, D), dtype=inp["q"].dtype, device="cuda")
    fta.set_split_mode("block")
    try:
        out, lse = _run(fta, inp, g["kv_group_num"], bs, ctx=S * bs, output=output, mid_output=mid_o,
                        mid_output_lse=mid_l)
    finally:
        fta.set_split_mode("balanced")
    _check(out, lse, _oracle(inp, g["kv_group_num"]), name + " block mode")
    for b, L in enumerate(inp["kv_seq_len"].tolist()):
        n = (L + bs - 1) // bs
        assert (mid_o[b, :, :n] - inp["ref_mid_o"][b, :, :n]).abs().max().item() <= 1e-3
        assert (mid_l[b, :, :n] - inp["ref_mid_lse"][b, :, :n]).abs().max().item() <= 1e-3
        assert torch.isnan(mid_o[b, :, n:]).all() and torch.isnan(mid_l[b, :, n:]).all()
    assert (output.float() - inp["ref_output"].float()).abs().max().item() <= OUT_TOL


def test_reference_assertions_are_kept(fta):
    from flash_tree_attn_b200.workloads import make_inputs

    w = _workload(B=2, H=4, G=1, D=64, Q=8, ctx=128, lens="fixed:128,50")
    inp = make_inputs(w, "cuda")
    a = (inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"], inp["kv_seq_len"])
    with pytest.raises(AssertionError):
        fta.flash_decoding_attention(*a, 48)  # block_size outside {16,32,64,128}
    with pytest.raises(AssertionError):
        fta.flash_decoding_attention(a[0], a[1], a[2][:, :, :64], *a[3:])  # cache length mismatch
    with pytest.raises(AssertionError):
        small = torch.empty(2, 4, 1, 8, 64, device="cuda")
        fta.flash_decoding_attention(*a, 64, 128, None, small, torch.empty(2, 4, 1, 8, device="cuda"))
    with pytest.raises(AssertionError):
        bad = inp["q"][..., :48]
        fta.flash_decoding_attention(bad, *a[1:])  # head_dim outside {32,64,128,256}


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("cfg,B", [("cfg2", 8), ("cfg3", 8), ("cfg4", 1), ("cfg5", 16)])
def test_benchmark_shapes(fta, cfg, B, kernel):
    """The benchmark configurations at full per-sequence size (batch reduced where the
    caches would not fit a quick test)."""
    from flash_tree_attn_b200.workloads import WORKLOADS, make_inputs, small

    fta.set_kernel(kernel)
    w = WORKLOADS[cfg]
    if cfg == "cfg4":
        w = small(w, ctx=32768)
    w = small(w, B=B)
    inp = make_inputs(w, "cuda")
    out, lse = _run(fta, inp, w.G, ctx=w.ctx)
    _check(out, lse, _oracle(inp, w.G), cfg)


@pytest.mark.parametrize("cfg", ["cfg3", "cfg4", "cfg5"])
def test_benchmark_shapes_at_full_size(fta, cfg):
    """The configurations the benchmark times, whole (32 sequences of cfg3, all 131072 rows of cfg4,
    the 128 ragged sequences of cfg5; cfg2 runs whole in test_benchmark_shapes): at full size the
    balanced plan has other tile ranges per block, 64-bit line positions where the line is long,
    more pieces per unit and a wrapped descriptor ring, which is what the timed launches exercise."""
    from flash_tree_attn_b200.workloads import WORKLOADS, make_inputs

    fta.set_kernel("auto")
    w = WORKLOADS[cfg]
    inp = make_inputs(w, "cuda")
    out, lse = _run(fta, inp, w.G, ctx=w.ctx)
    _check(out, lse, _oracle(inp, w.G), cfg + " full size")
    del inp
    torch.cuda.empty_cache()


@pytest.mark.parametrize("kernel", KERNELS)
def test_reference_test_case_at_its_own_size(fta, kernel):
    """The reference's only test, test_tree_op (flash_tree_attn.py:416-440), at its own size and
    conventions: Z=32, H=32, N_CTX=4096, head_dim 128, q_len 128, block_size 128 passed
    positionally, int64 lengths all equal to N_CTX, q/k/v ~ N(0, 0.5), tree tokens ~ N(0, 1), a random
    0/1 visibility pattern with the diagonal set whose allowed entries are 1.0 (added to the scores),
    fp16.  The reference accepts atol 1e-2 against its dense torch evaluation; here 2e-3 against
    the fp32 oracle, which follows that evaluation."""
    fta.set_kernel(kernel)
    Z, H, N_CTX, D, q_len = 32, 32, 4096, 128, 128
    g = torch.Generator(device="cuda").manual_seed(416)
    rnd = lambda shape, std: (torch.randn(shape, generator=g, device="cuda") * std).half()
    inp = {"q": rnd((Z, H, q_len, D), 0.5), "k_cache": rnd((Z, H, N_CTX, D), 0.5), "v_cache": rnd((Z, H, N_CTX, D), 0.5),
           "current_k": rnd((Z, H, q_len, D), 1.0), "current_v": rnd((Z, H, q_len, D), 1.0)}
    vis = torch.rand((q_len, q_len), generator=g, device="cuda") < 0.5
    vis |= torch.eye(q_len, dtype=torch.bool, device="cuda")
    inp["mask"] = torch.where(vis, 1.0, float("-inf")).float()
    inp["kv_seq_len"] = torch.tensor([N_CTX] * Z).cuda()  # int64, as the reference's test builds it
    assert inp["kv_seq_len"].dtype == torch.int64
    out = fta.flash_decoding_attention(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"],
                                       inp["mask"], inp["kv_seq_len"], 128)
    out2, lse = _run(fta, inp, 1, 128)
    assert torch.equal(out, out2)
    ora = _oracle(inp, 1)
    _check(out, lse, ora, "reference test case")
    assert torch.allclose(ora["out"], out.float(), atol=1e-2, rtol=0)  # the reference's own criterion
    del inp
    torch.cuda.empty_cache()


def test_kv_range_shards_merge_to_whole(fta):
    """One sequence cut into KV ranges (what each GPU of a sequence-split job computes),
    tree attached to the last range, merged by fta_merge_parts."""
    from flash_tree_attn_b200.workloads import make_inputs

    w = _workload(B=1, H=16, G=8, D=128, Q=64, ctx=4096, lens="fixed:4096", dtype=torch.bfloat16)
    inp = make_inputs(w, "cuda")
    ora = _oracle(inp, 8)
    n = 4
    parts_o, parts_l = [], []
    for r in range(n):
        lo, hi = r * 1024, (r + 1) * 1024
        sh = dict(inp)
        sh["k_cache"], sh["v_cache"] = inp["k_cache"][:, :, lo:hi], inp["v_cache"][:, :, lo:hi]
        sh["kv_seq_len"] = torch.tensor([1024], dtype=torch.int32, device="cuda")
        o, l = _run(fta, sh, 8, out_dtype=torch.float32, with_tree=(r == n - 1))
        parts_o.append(o)
        parts_l.append(l)
    out, lse = fta.merge_partials(torch.stack(parts_o), torch.stack(parts_l), torch.bfloat16)
    _check(out, lse, ora, "kv-range shards")


def test_call_is_capturable_in_a_cuda_graph_and_follows_the_lengths(fta):
    """A prepared call neither allocates nor synchronises, and it builds its plan on the device from
    kv_seq_len: captured once in a CUDA graph, it gives the right answer on every replay even after
    q and the lengths have been changed in place (the reference reads the lengths back with .item(),
    flash_tree_attn.py:272, which a capture cannot contain)."""
    from flash_tree_attn_b200.workloads import make_inputs

    fta.set_kernel("auto")
    w = _workload(B=3, H=8, G=2, D=128, Q=32, ctx=2048, lens="fixed:2048,900,3")
    inp = make_inputs(w, "cuda")
    args = (inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"], inp["kv_seq_len"], 64, 2048)
    fta.prepare(*args, kv_group_num=2, want_lse=True).run()  # first launch outside the capture: tensor maps, function attributes
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        # the capture runs on its own stream: prepare there so that the call is issued on it
        out, lse = fta.prepare(*args, kv_group_num=2, want_lse=True).run()
    for lens in ([2048, 900, 3], [5, 2047, 1111], [64, 0, 2048]):
        inp["kv_seq_len"].copy_(torch.tensor(lens, dtype=inp["kv_seq_len"].dtype))
        inp["q"].normal_()
        graph.replay()
        torch.cuda.synchronize()
        _check(out, lse, _oracle(inp, 2), f"graph replay lens={lens}")


def test_two_calls_in_one_cuda_graph(fta):
    """Two calls captured back to back: the second call's stage 1 is a programmatic dependent of the
    first call's stage 2 inside the graph (its set-up overlaps that kernel's drain), and the two
    calls share the library's workspace, so the second must not touch it before the first is done."""
    from flash_tree_attn_b200.workloads import make_inputs

    fta.set_kernel("auto")
    wa = _workload(B=4, H=8, G=2, D=128, Q=32, ctx=4096, lens="fixed:4096,900,3,2500", seed=5)
    wb = _workload(B=4, H=8, G=2, D=128, Q=32, ctx=4096, lens="fixed:70,4000,1234,64", seed=6)
    ia, ib = make_inputs(wa, "cuda"), make_inputs(wb, "cuda")

    def args(i):
        return (i["q"], i["k_cache"], i["v_cache"], i["current_k"], i["current_v"], i["mask"], i["kv_seq_len"], 64, 4096)

    fta.prepare(*args(ia), kv_group_num=2, want_lse=True).run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        oa, la = fta.prepare(*args(ia), kv_group_num=2, want_lse=True).run()
        ob, lb = fta.prepare(*args(ib), kv_group_num=2, want_lse=True).run()
    for rep in range(3):
        ia["q"].normal_()
        ib["q"].normal_()
        graph.replay()
        torch.cuda.synchronize()
        _check(oa, la, _oracle(ia, 2), f"first call, replay {rep}")
        _check(ob, lb, _oracle(ib, 2), f"second call, replay {rep}")


@pytest.mark.parametrize("kernel", KERNELS)
def test_alternating_calls_share_the_workspace(fta, kernel):
    """Two different jobs issued alternately, hundreds of times, without a synchronisation between
    them: a call's stage 1 is set up while the previous call's stage 2 is still reading the partial
    results that both keep in the same workspace, and must not write there before that is over."""
    from flash_tree_attn_b200.workloads import make_inputs

    fta.set_kernel(kernel)
    wa = _workload(B=6, H=8, G=2, D=128, Q=32, ctx=8192, lens="fixed:8192,900,3,2500,7000,64", seed=7)
    wb = _workload(B=6, H=8, G=2, D=128, Q=32, ctx=8192, lens="fixed:70,8000,1234,64,1,5000", seed=8)
    ia, ib = make_inputs(wa, "cuda"), make_inputs(wb, "cuda")

    def prep(i):
        return fta.prepare(i["q"], i["k_cache"], i["v_cache"], i["current_k"], i["current_v"], i["mask"],
                           i["kv_seq_len"], 64, 8192, kv_group_num=2, want_lse=True)

    pa, pb = prep(ia), prep(ib)
    ref_a, ref_b = _oracle(ia, 2), _oracle(ib, 2)
    for rep in range(3):
        for _ in range(100):
            oa, la = pa.run()
            ob, lb = pb.run()
        torch.cuda.synchronize()
        _check(oa, la, ref_a, f"job A after round {rep}")
        _check(ob, lb, ref_b, f"job B after round {rep}")
