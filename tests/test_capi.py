"""CPU: the C-ABI library loads, exports every symbol include/fta.h declares, and its host
logic (argument validation, the split plan) behaves.  No kernel is launched."""
import ctypes as C
import os
import random
import re

import pytest

from flash_tree_attn_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fta.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fta_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(fta_lib):
    names = declared_symbols()
    assert "fta_decode" in names and "fta_plan_host" in names
    for n in names:
        assert hasattr(fta_lib, n), f"{n} declared in include/fta.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype"


def test_version_and_strerror(fta_lib):
    assert fta_lib.fta_version() == 101
    assert fta_lib.fta_strerror(0) == b"ok"
    for code in range(1, 6):
        assert len(fta_lib.fta_strerror(code)) > 3


def test_struct_layout_matches_header():
    # sizes printed by a C++ compile of include/fta.h
    assert C.sizeof(_lib.FtaParams) == 496
    assert C.sizeof(_lib.FtaMergeParams) == 64
    assert C.sizeof(_lib.FtaExchangeParams) == 328
    assert _lib.FtaExchangeParams.out.offset == 312


def test_exchange_merge_arguments_are_validated(fta_lib):
    """Bad rank counts, ranks and null pointers are refused before anything is launched."""
    p = _lib.FtaExchangeParams()
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG
    p.out = p.flag_local = p.status = 4096
    p.world, p.rank, p.rows, p.D, p.out_dtype, p.timeout_ns = 9, 0, 16, 128, _lib.DTYPE_F32, 1000
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG  # more than FTA_MAX_RANKS
    p.world, p.rank = 2, 2
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG  # rank outside the group
    p.rank = 0
    p.part[0] = 4096
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG  # rank 1's partial missing
    p.part[1] = 4096
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG  # no flag address for rank 1
    p.flag_peer[1] = 4096
    p.timeout_ns = 0
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG  # the wait must be bounded
    p.timeout_ns = 1000
    p.done = 4096  # scatter form: every rank's result buffers must be given
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG
    p.out_peer[0] = p.out_peer[1] = p.lse_peer[0] = 4096
    assert fta_lib.fta_exchange_merge(C.byref(p), None) == _lib.FTA_E_BADARG  # rank 1's LSE buffer missing


def _params(B, H, Hkv, Q, D, ctx, grid, with_tree=1, kernel=_lib.KERNEL_MMA):
    p = _lib.FtaParams()
    p.B, p.H, p.Hkv, p.Q, p.D, p.ctx = B, H, Hkv, Q, D, ctx
    p.dtype = p.out_dtype = _lib.DTYPE_F16
    p.with_tree = with_tree
    p.kernel = kernel
    p.grid_override = grid
    return p


def test_decode_rejects_bad_arguments(fta_lib):
    p = _params(2, 8, 8, 8, 48, 128, 4)  # head_dim outside {32,64,128,256}
    assert fta_lib.fta_decode(C.byref(p), None) == _lib.FTA_E_BADARG
    p = _params(2, 8, 3, 8, 64, 128, 4)  # H not a multiple of Hkv
    assert fta_lib.fta_decode(C.byref(p), None) == _lib.FTA_E_BADARG
    p = _params(2, 8, 8, 8, 64, 128, 4)  # null pointers
    assert fta_lib.fta_decode(C.byref(p), None) == _lib.FTA_E_BADARG
    assert fta_lib.fta_decode(None, None) == _lib.FTA_E_BADARG


def test_sizing_entry_points_validate_sizes_and_dtype(fta_lib):
    """fta_workspace_bytes / fta_plan_grid / fta_plan_host read sizes only, but they index tables by
    dtype and head_dim: bad values must come back as an error code, not as an out-of-range read."""
    good = _params(2, 8, 8, 8, 64, 128, 4)
    assert fta_lib.fta_workspace_bytes(C.byref(good)) > 0 and fta_lib.fta_plan_grid(C.byref(good)) == 4
    lens = (C.c_int64 * 2)(100, 37)
    for field, value in (("dtype", 7), ("dtype", -1), ("D", 48), ("Hkv", 3), ("B", 0), ("Q", 0)):
        p = _params(2, 8, 8, 8, 64, 128, 4)
        setattr(p, field, value)
        assert fta_lib.fta_workspace_bytes(C.byref(p)) == -_lib.FTA_E_BADARG, field
        assert fta_lib.fta_plan_grid(C.byref(p)) == -_lib.FTA_E_BADARG, field
        assert fta_lib.fta_plan_host(C.byref(p), lens, None, 0, None, None) == -_lib.FTA_E_BADARG, field
    assert fta_lib.fta_workspace_bytes(None) == -_lib.FTA_E_BADARG


def test_paged_cache_arguments_are_validated(fta_lib):
    """Pointers here are fake but aligned: validation ends before anything is dereferenced or
    launched.  A page must hold whole 64-row tiles and the table must cover ctx."""
    def base():
        p = _params(2, 8, 8, 8, 64, 256, 4, with_tree=0)
        p.split_mode = _lib.SPLIT_BALANCED
        for name in ("q", "k_cache", "v_cache", "kv_seq_len", "out", "workspace"):
            setattr(p, name, 4096)
        for name in ("q_sb", "q_sh", "q_sq", "k_sb", "k_sh", "k_st", "v_sb", "v_sh", "v_st", "o_sb", "o_sh", "o_sq"):
            setattr(p, name, 64)
        p.block_table = 4096
        p.n_pages = 16
        return p

    p = base(); p.page_size = 32; p.bt_sb = 8   # smaller than a tile
    assert fta_lib.fta_decode(C.byref(p), None) == _lib.FTA_E_BADARG
    p = base(); p.page_size = 96; p.bt_sb = 8   # not a multiple of 64
    assert fta_lib.fta_decode(C.byref(p), None) == _lib.FTA_E_BADARG
    p = base(); p.page_size = 64; p.bt_sb = 3   # 3 pages of 64 rows cannot hold ctx = 256
    assert fta_lib.fta_decode(C.byref(p), None) == _lib.FTA_E_BADARG
    p = base(); p.page_size = 64; p.bt_sb = 4; p.n_pages = 0
    assert fta_lib.fta_decode(C.byref(p), None) == _lib.FTA_E_BADARG


def test_pages_hold_the_dense_rows():
    """workloads.to_paged (used by the GPU tests and bench.py --paged): reading the pages back
    through the table gives the dense rows below each length; everything else in the pool is NaN."""
    import torch
    from flash_tree_attn_b200.workloads import to_paged

    torch.manual_seed(3)
    lens = [130, 0, 64, 1]
    k = torch.randn(4, 2, 192, 32).half()
    v = torch.randn(4, 2, 192, 32).half()
    for page in (64, 128):
        kp, vp, table = to_paged(k, v, lens, page_size=page, seed=7)
        used = set()
        for b, L in enumerate(lens):
            for r in range(L):
                pg = int(table[b, r // page])
                used.add(pg)
                assert torch.equal(kp[pg, :, r % page], k[b, :, r]) and torch.equal(vp[pg, :, r % page], v[b, :, r])
        assert len(used) == sum(-(-L // page) for L in lens)
        finite = torch.isfinite(kp.float()).all(dim=-1).all(dim=1)  # [n_pages, page]
        assert int(finite.sum()) == sum(lens)


def plan(fta_lib, lens, H, Hkv, Q, D, grid, with_tree=1):
    B = len(lens)
    p = _params(B, H, Hkv, Q, D, max(lens + [1]), grid, with_tree)
    arr = (C.c_int64 * B)(*lens)
    cap = 1 << 16
    segs = (C.c_int64 * (cap * 8))()
    g, per = C.c_int32(), C.c_int32()
    n = fta_lib.fta_plan_host(C.byref(p), arr, segs, cap, C.byref(g), C.byref(per))
    assert 0 <= n <= cap
    rows = [tuple(segs[i * 8:(i + 1) * 8]) for i in range(n)]
    return rows, g.value, per.value


@pytest.mark.parametrize("seed", range(6))
def test_balanced_plan_covers_every_tile_once(fta_lib, seed):
    rng = random.Random(seed)
    B = rng.choice([1, 2, 5, 32, 128])
    G = rng.choice([1, 4, 8])
    Hkv = rng.choice([1, 2, 8])
    Q = rng.choice([1, 4, 26, 64, 100])
    lens = [rng.choice([0, 1, 63, 64, 65, rng.randint(1, 5000)]) for _ in range(B)]
    grid = rng.choice([1, 7, 148, 296])
    rows, g, per = plan(fta_lib, lens, Hkv * G, Hkv, Q, 128, grid)
    assert g == grid and per >= 2
    M = G * Q
    R = 16 if M <= 16 else 32 if M <= 32 else 64
    qpt = min(Q, R)
    hpt = min(G, R // qpt)
    U = Hkv * (-(-Q // qpt)) * (-(-G // hpt))
    n_tree = -(-Q // 64)
    seen_cache, seen_tree, pieces, slots = {}, {}, {}, set()
    per_block = {}
    for (c, b, j, c0, c1, t0, t1, packed) in rows:
        split, nsplit = packed >> 16, packed & 0xFFFF
        assert 0 <= b < B and 0 <= j < U and 0 <= split < nsplit
        assert c0 % 64 == 0 and c0 <= max(c0, c1) and c1 <= lens[b]
        for r in range(c0, c1):
            seen_cache[(b, j, r)] = seen_cache.get((b, j, r), 0) + 1
        for t in range(t0, t1):
            seen_tree[(b, j, t)] = seen_tree.get((b, j, t), 0) + 1
        pieces.setdefault((b, j), []).append((split, nsplit))
        per_block[c] = per_block.get(c, 0) + (-(-max(c1 - c0, 0) // 64)) + (t1 - t0)
    for b in range(B):
        for j in range(U):
            for r in range(lens[b]):
                assert seen_cache.get((b, j, r)) == 1
            for t in range(n_tree):
                assert seen_tree.get((b, j, t)) == 1
            ps = sorted(pieces[(b, j)])
            assert [s for s, _ in ps] == list(range(ps[0][1])), "split indices of a unit are 0..n-1"
    assert len(seen_cache) == sum(lens) * U
    # balance: no block gets more than `per` tiles
    assert max(per_block.values()) <= per
    mtiles = U // Hkv  # M tiles of one KV head walk the same range in neighbouring blocks ("lanes")
    _check_slot_rule(rows, lanes=mtiles if (mtiles > 1 and grid >= mtiles) else 1)


def test_plan_is_balanced_for_ragged_batch(fta_lib):
    rng = random.Random(5)
    lens = [rng.randint(16, 16384) for _ in range(128)]
    rows, g, per = plan(fta_lib, lens, 32, 32, 4, 128, 296)
    # every unit is charged 4 tiles on top of its own (cache tiles + 1 tree tile) for ending: blocks
    # that finish many short units get fewer tiles to stream
    pad = 4
    total = sum(-(-L // 64) + 1 + pad for L in lens) * 32
    assert per == -(-total // 296)
    cost = {}
    ends = {}
    for (c, b, j, c0, c1, t0, t1, packed) in rows:
        cost[c] = cost.get(c, 0) + (-(-max(c1 - c0, 0) // 64)) + (t1 - t0)
        if t1 == 1:  # the piece that ends its unit
            ends[c] = ends.get(c, 0) + 1
    # a block's tiles plus the charge of the units that end well inside it never exceed its share
    assert max(cost[c] + pad * max(ends.get(c, 0) - 1, 0) for c in cost) <= per
    # at most two cut pieces per block, so partial slots 2*block + {0,1} never collide
    cut = {}
    for (c, b, j, c0, c1, t0, t1, packed) in rows:
        if (packed & 0xFFFF) > 1:
            cut[c] = cut.get(c, 0) + 1
    assert max(cut.values()) <= 2
    _check_slot_rule(rows)


def _check_slot_rule(rows, lanes=1):
    """A cut unit's first piece goes to slot 1 of its block and every later piece to slot 0 (stage 2
    finds all of them from the index of the block that holds the second piece), so a block must
    never hold two first pieces or two later pieces, a unit's pieces must sit in consecutive groups
    of blocks, and the second piece must open its block."""
    first, later, where = {}, {}, {}
    seen_in_block = {}
    for (c, b, j, c0, c1, t0, t1, packed) in rows:
        split, nsplit = packed >> 16, packed & 0xFFFF
        seen_in_block.setdefault(c, []).append((b, j, split, nsplit))
        if nsplit < 2:
            continue
        if split == 0:
            first[c] = first.get(c, 0) + 1
        else:
            later[c] = later.get(c, 0) + 1
        where[(b, j, split)] = c
    assert all(v == 1 for v in first.values()) and all(v == 1 for v in later.values())
    for (b, j, split), c in where.items():
        if split > 0:
            assert where[(b, j, split - 1)] == c - lanes, "pieces of a unit sit in consecutive blocks"
            assert seen_in_block[c][0][:3] == (b, j, split), "a later piece opens its block"
        else:
            assert seen_in_block[c][-1][:3] == (b, j, 0), "a first piece closes its block"
