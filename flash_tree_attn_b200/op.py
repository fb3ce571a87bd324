"""Host side of the operator: the reference's Python interface over the C-ABI library.

`flash_decoding_attention` keeps the reference's signature, argument meaning, return value
and assertion behaviour (flash_tree_attn.py:216-376) so that it can be imported in its
place.  All arithmetic happens in libfta.so; torch is used for device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import FtaParams

_DT = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}

# "balanced": planner-chosen splits (default).  "block": one partial per `block_size` rows
# written to mid_output / mid_output_lse exactly where the reference writes them
# (flash_tree_attn.py:124-144), for callers or tests that read those buffers.
_split_mode = os.environ.get("FTA_SPLIT_MODE", "balanced")
_kernel = {"auto": _lib.KERNEL_AUTO, "mma": _lib.KERNEL_MMA, "umma": _lib.KERNEL_UMMA}[
    os.environ.get("FTA_KERNEL", "auto")
]
_grid_override = int(os.environ.get("FTA_GRID", "0"))

_scratch = {}  # (device index, stream, tag) -> tensor, grown on demand


def set_split_mode(mode: str) -> None:
    """"balanced" or "block" (see module docstring)."""
    global _split_mode
    if mode not in ("balanced", "block"):
        raise ValueError(mode)
    _split_mode = mode


def set_kernel(name: str) -> None:
    """Force a stage-1 kernel family: "auto", "mma" (warp MMA) or "umma" (tcgen05)."""
    global _kernel
    _kernel = {"auto": _lib.KERNEL_AUTO, "mma": _lib.KERNEL_MMA, "umma": _lib.KERNEL_UMMA}[name]


def set_grid_override(n: int) -> None:
    """Number of stage-1 thread blocks (0 = planner's choice); results must not depend on it."""
    global _grid_override
    _grid_override = int(n)


def _scratch_buf(dev: torch.device, stream: int, tag: str, nbytes: int) -> torch.Tensor:
    key = (dev.index, stream, tag)
    t = _scratch.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        _scratch[key] = t
    return t


_warned_cache_copy = False


def _warn_cache_copy(t: torch.Tensor) -> None:
    global _warned_cache_copy
    if not _warned_cache_copy:
        import warnings

        _warned_cache_copy = True
        warnings.warn(
            f"flash_decoding_attention: KV cache with strides {tuple(t.stride())} / data pointer alignment "
            f"{t.data_ptr() % 16} is copied to a contiguous layout on every call "
            f"({2 * t.numel() * t.element_size() / 2**20:.0f} MiB per call); give the caches unit stride in head_dim, "
            "other strides that are multiples of 8 elements and a 16-byte aligned base to avoid it", RuntimeWarning,
            stacklevel=4)


def _rows_ok(t: torch.Tensor) -> bool:
    if t.stride(-1) != 1 or t.data_ptr() % 16:
        return False
    return all(s % 8 == 0 for s in t.stride()[:-1])


def _mask_strides(mask: torch.Tensor, B: int, H: int, Q: int):
    """fp32 additive mask -> (tensor, stride_b, stride_h, stride_q); 0 broadcasts.

    Accepted shapes: [Q,Q], [H,Q,Q], [B,1,Q,Q], [B,H,Q,Q] (and size-1 broadcast dims), the
    set that broadcasts against the reference's [B,H,Q,Q] scores (flash_tree_attn.py:368),
    plus [B,Q,Q] read per sequence when B != H.
    """
    if mask.dtype != torch.float32 or mask.stride(-1) != 1:
        mask = mask.float().contiguous()
    if mask.dim() == 2:
        sb = sh = 0
    elif mask.dim() == 3:
        # The reference adds the mask to [B,H,Q,Q] scores, so torch broadcasting reads a 3-D mask's
        # first dimension as HEADS (flash_tree_attn.py:368).  That reading is kept whenever the size
        # fits it (also when bsz == num_heads); a first dimension of bsz != num_heads, which the
        # reference rejects, is read per sequence.  Pass [bsz,1,Q,Q] to be explicit.
        if mask.size(0) == H and H > 1:
            sb, sh = 0, mask.stride(0)
        else:
            sb, sh = (mask.stride(0) if mask.size(0) > 1 else 0), 0
            assert mask.size(0) in (1, B), "mask's first dimension matches neither num_heads nor bsz"
    elif mask.dim() == 4:
        sb = mask.stride(0) if mask.size(0) > 1 else 0
        sh = mask.stride(1) if mask.size(1) > 1 else 0
        assert mask.size(0) in (1, B) and mask.size(1) in (1, H), "mask does not broadcast against [B,H,Q,Q]"
    else:
        raise AssertionError("mask must have 2, 3 or 4 dimensions")
    assert mask.size(-1) == Q and mask.size(-2) == Q, "mask must be [.., q_len, q_len]"
    return mask, sb, sh, mask.stride(-2)


class PreparedCall:
    """One validated call: the filled C-ABI parameter block, its output tensors and the
    stream it was prepared for.  `run()` launches it (again); the tensors it points at may
    be overwritten in place between runs.  Used by the benchmark to time the stages apart
    and by callers that want to pay validation once per shape."""

    __slots__ = ("p", "out", "lse", "stream", "_keep", "launches")

    def __init__(self, p, out, lse, stream, keep):
        self.p, self.out, self.lse, self.stream, self._keep = p, out, lse, stream, keep
        self.launches = 2  # stage 1 + stage 2

    def run(self):
        _lib.check(_lib.load().fta_decode(C.byref(self.p), self.stream), "fta_decode")
        return self.out, self.lse

    def run_stage1(self):
        _lib.check(_lib.load().fta_stage1(C.byref(self.p), self.stream), "fta_stage1")

    def run_stage2(self):
        _lib.check(_lib.load().fta_stage2(C.byref(self.p), self.stream), "fta_stage2")


def prepare(
    q, k_cache, v_cache, current_k, current_v, mask, kv_seq_len, block_size=64, max_seq_len_in_batch=None,
    output=None, mid_output=None, mid_output_lse=None, sm_scale=None, kv_group_num=1, *,
    want_lse=False, out_dtype=None, with_tree=True, out_buf=None, lse_buf=None, block_table=None,
) -> PreparedCall:
    """Validate the arguments of flash_decoding_attention and build the C-ABI call without
    launching it.  With `block_table` [bsz, max_pages] int32 the caches are pools of pages
    [n_pages, num_kv_heads, page_size, head_dim] (see flash_decoding_attention_paged)."""
    lib = _lib.load()
    if not q.is_cuda:
        raise RuntimeError("flash_decoding_attention runs on CUDA tensors only (no CPU path exists)")
    B, H, Q, D = q.shape
    Q = int(Q)

    # the reference's own asserts (flash_tree_attn.py:263-268)
    assert D in {32, 64, 128, 256}
    assert k_cache.size(-2) == v_cache.size(-2), "Got incompatible block size on kv caches:\n"
    assert block_size in {16, 32, 64, 128}
    assert q.dtype in (torch.float16, torch.bfloat16), "q must be fp16 or bf16"
    assert k_cache.dtype == q.dtype and v_cache.dtype == q.dtype, "kv cache dtype must equal q dtype"
    G = int(kv_group_num)
    assert G >= 1 and H % G == 0, "num_heads must be a multiple of kv_group_num"
    Hkv = H // G
    paged = block_table is not None
    if paged:
        assert k_cache.size(1) == Hkv and tuple(k_cache.shape) == tuple(v_cache.shape), \
            "paged caches must be [n_pages, num_kv_heads, page_size, head_dim]"
        page_size = int(k_cache.size(-2))
        assert page_size % 64 == 0, "page_size must be a multiple of 64"
        assert block_table.dim() == 2 and block_table.size(0) == B, "block_table must be [bsz, max_pages]"
    else:
        assert k_cache.size(0) >= B and k_cache.size(1) == Hkv, "k_cache must be [bsz, num_kv_heads, ctx, head_dim]"

    sm_scale = 1.0 / (D ** 0.5) if sm_scale is None else float(sm_scale)
    ctx = int(block_table.size(1)) * page_size if paged else int(k_cache.size(-2))
    if max_seq_len_in_batch is not None:
        ctx = min(ctx, int(max_seq_len_in_batch))
    # For compatibility with the reference's buffer contract (flash_tree_attn.py:274)
    max_len = ctx if max_seq_len_in_batch is None else int(max_seq_len_in_batch)
    kv_max_split_num = (max_len + block_size - 1) // block_size

    if mid_output is not None or mid_output_lse is not None:
        assert mid_output is not None and mid_output_lse is not None
        assert (
            mid_output.size(2) == mid_output_lse.size(2) >= kv_max_split_num
        ), "Incompatible kv split number of intermediate output tensors"
        assert (
            mid_output.size(0) == mid_output_lse.size(0) >= B
        ), "Incompatible first dimension of output tensors"
    if output is not None:
        assert output.size(0) == B, "Incompatible first dimension of output tensors"

    dev = q.device
    stream = torch.cuda.current_stream(dev).cuda_stream

    if not _rows_ok(q):
        q = q.contiguous()
    if not (_rows_ok(k_cache) and _rows_ok(v_cache)):
        # every copy engine here moves 16-byte row chunks; a cache laid out otherwise has to be
        # re-packed, which costs a full read and write of it on every call: say so, once
        _warn_cache_copy(k_cache)
        k_cache, v_cache = k_cache.contiguous(), v_cache.contiguous()
    if kv_seq_len.dtype not in (torch.int32, torch.int64) or not kv_seq_len.is_contiguous():
        kv_seq_len = kv_seq_len.to(torch.int64).contiguous()
    if kv_seq_len.device != dev:
        kv_seq_len = kv_seq_len.to(dev)

    p = FtaParams()
    p.q = q.data_ptr(); p.q_sb, p.q_sh, p.q_sq = q.stride(0), q.stride(1), q.stride(2)
    p.k_cache = k_cache.data_ptr(); p.k_sb, p.k_sh, p.k_st = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    p.v_cache = v_cache.data_ptr(); p.v_sb, p.v_sh, p.v_st = v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
    p.kv_seq_len = kv_seq_len.data_ptr()
    p.len_is_i64 = 1 if kv_seq_len.dtype == torch.int64 else 0
    p.cur_head_mul = 1
    keep = [q, k_cache, v_cache, kv_seq_len]
    if paged:
        if block_table.dtype != torch.int32 or not block_table.is_contiguous() or block_table.device != dev:
            block_table = block_table.to(device=dev, dtype=torch.int32).contiguous()
        p.block_table = block_table.data_ptr(); p.bt_sb = block_table.stride(0)
        p.page_size = page_size; p.n_pages = int(k_cache.size(0))
        keep.append(block_table)

    if with_tree:
        assert current_k.dtype == q.dtype and current_v.dtype == q.dtype
        assert current_k.size(2) == Q and current_v.size(2) == Q, "current_k/current_v must hold q_len rows"
        hk = current_k.size(1)
        assert hk in (Hkv, H) and current_v.size(1) == hk, "current_k/current_v must have num_kv_heads or num_heads heads"
        if not _rows_ok(current_k):
            current_k = current_k.contiguous()
        if not _rows_ok(current_v):
            current_v = current_v.contiguous()
        # [B,H,Q,D] inputs under GQA: head kvh*G of the group is read (the reference's own
        # tail needs the heads replicated per group, flash_tree_attn.py:367,371)
        p.cur_head_mul = G if (hk == H and G > 1) else 1
        p.cur_k = current_k.data_ptr(); p.ck_sb, p.ck_sh, p.ck_st = current_k.stride(0), current_k.stride(1), current_k.stride(2)
        p.cur_v = current_v.data_ptr(); p.cv_sb, p.cv_sh, p.cv_st = current_v.stride(0), current_v.stride(1), current_v.stride(2)
        mask, msb, msh, msq = _mask_strides(mask.to(dev) if mask.device != dev else mask, B, H, Q)
        p.mask = mask.data_ptr(); p.m_sb, p.m_sh, p.m_sq = msb, msh, msq
        keep += [current_k, current_v, mask]

    out_dtype = q.dtype if out_dtype is None else out_dtype
    if out_buf is not None:  # caller-owned result storage (e.g. a slice of a gather buffer)
        assert out_buf.dtype == out_dtype and tuple(out_buf.shape) == (B, H, Q, D) and out_buf.is_contiguous()
        out = out_buf
    else:
        out = torch.empty((B, H, Q, D), dtype=out_dtype, device=dev)
    p.out = out.data_ptr(); p.o_sb, p.o_sh, p.o_sq = out.stride(0), out.stride(1), out.stride(2)
    lse = None
    if want_lse and lse_buf is not None:
        assert lse_buf.dtype == torch.float32 and tuple(lse_buf.shape) == (B, H, Q) and lse_buf.is_contiguous()
        lse = lse_buf
        p.lse = lse.data_ptr(); p.l_sb, p.l_sh = lse.stride(0), lse.stride(1)
    elif want_lse:
        lse = torch.empty((B, H, Q), dtype=torch.float32, device=dev)
        p.lse = lse.data_ptr(); p.l_sb, p.l_sh = lse.stride(0), lse.stride(1)

    p.B, p.H, p.Hkv, p.Q, p.D, p.ctx = B, H, Hkv, Q, D, ctx
    p.dtype = _DT[q.dtype]
    p.out_dtype = _DT[out_dtype]
    p.sm_scale = sm_scale
    p.with_tree = 1 if with_tree else 0
    p.kernel = _kernel
    p.grid_override = _grid_override

    block_mode = _split_mode == "block"
    if output is None and not block_mode:
        # planner-balanced splits, fixed-size workspace
        p.split_mode = _lib.SPLIT_BALANCED
        # asked every time: the size depends on the kernel family the library picks for THESE
        # strides and options, and the query is a few hundred nanoseconds of host arithmetic
        nbytes = lib.fta_workspace_bytes(C.byref(p))
        if nbytes < 0:
            raise _lib.FtaError(-nbytes, "fta_workspace_bytes")
        ws = _scratch_buf(dev, stream, "ws", nbytes)
        p.workspace = ws.data_ptr(); p.workspace_bytes = ws.numel()
        keep.append(ws)
    else:
        # one partial per split: the reference's buffer layout (flash_tree_attn.py:276-281)
        if block_mode:
            split = block_size
        else:
            p.split_mode = _lib.SPLIT_BALANCED  # only sizes are read by fta_plan_grid
            grid = max(lib.fta_plan_grid(C.byref(p)), 1)
            units = B * Hkv * max(1, (G * Q + 127) // 128)
            split = max(256, -(-(units * max(ctx, 1)) // (grid * 4)))
            split = min(-(-split // 64) * 64, max(64, -(-ctx // 64) * 64))
        p.split_mode = _lib.SPLIT_FIXED
        p.split_tokens = split
        S = max(1, -(-ctx // split))
        use_caller_mid = (
            block_mode and mid_output is not None and mid_output.dtype == torch.float32
            and mid_output_lse.dtype == torch.float32 and mid_output.stride(-1) == 1
            and mid_output_lse.stride(-1) == 1 and mid_output.data_ptr() % 16 == 0
            and all(s % 4 == 0 for s in mid_output.stride()[:-1])
            and tuple(mid_output.shape[1:]) == (H, mid_output.size(2), Q, D)
        )
        if use_caller_mid:
            mo, ml = mid_output, mid_output_lse
        else:
            mo = _scratch_buf(dev, stream, "mid_o", B * H * S * Q * D * 4).view(torch.float32)[: B * H * S * Q * D].view(B, H, S, Q, D)
            ml = _scratch_buf(dev, stream, "mid_l", B * H * S * Q * 4).view(torch.float32)[: B * H * S * Q].view(B, H, S, Q)
        p.mid_o = mo.data_ptr(); p.mo_sb, p.mo_sh, p.mo_ss, p.mo_sq = mo.stride(0), mo.stride(1), mo.stride(2), mo.stride(3)
        p.mid_lse = ml.data_ptr(); p.ml_sb, p.ml_sh, p.ml_ss = ml.stride(0), ml.stride(1), ml.stride(2)
        p.mid_splits = int(mo.size(2))
        keep += [mo, ml]
        if with_tree:
            to = _scratch_buf(dev, stream, "tree_o", B * H * Q * D * 4)
            tl = _scratch_buf(dev, stream, "tree_l", B * H * Q * 4)
            p.tree_o = to.data_ptr(); p.tree_lse = tl.data_ptr()
            keep += [to, tl]
        if output is not None:
            assert output.dtype == q.dtype and tuple(output.shape) == (B, H, Q, D) and output.stride(-1) == 1
            p.out_cache = output.data_ptr()
            p.oc_sb, p.oc_sh, p.oc_sq = output.stride(0), output.stride(1), output.stride(2)
            keep.append(output)

    return PreparedCall(p, out, lse, stream, keep)


def _decode(*args, **kw) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    return prepare(*args, **kw).run()


def flash_decoding_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    current_k: torch.Tensor,
    current_v: torch.Tensor,
    mask: torch.Tensor,
    kv_seq_len: torch.Tensor,
    block_size: int = 64,
    max_seq_len_in_batch: int = None,
    output: torch.Tensor = None,
    mid_output: torch.Tensor = None,
    mid_output_lse: torch.Tensor = None,
    sm_scale: int = None,
    kv_group_num: int = 1,
):
    """Tree-attention verification step of speculative decoding (drop-in for the
    reference's flash_decoding_attention, flash_tree_attn.py:216-376).

    Args:
        q: [bsz, num_heads, q_len, head_dim] fp16/bf16, the tree nodes' queries.
        k_cache, v_cache: [bsz, num_kv_heads, ctx, head_dim] dense right-padded caches; rows at
            or past kv_seq_len[b] are never read.
        current_k, current_v: [bsz, num_kv_heads, q_len, head_dim] (or num_heads heads,
            replicated per group) keys/values of the tree nodes, not yet in the cache.
        mask: additive float mask over the tree nodes, [q_len,q_len], [bsz,q_len,q_len],
            [bsz,1,q_len,q_len] or [bsz,num_heads,q_len,q_len]; it is ADDED to the scaled
            scores (flash_tree_attn.py:368), so allowed entries may be any finite value.
        kv_seq_len: [bsz] int32/int64 cache lengths (tree tokens not included).
        block_size: reference's split size; here it only sizes the mid buffers' contract,
            unless split mode "block" is selected (`set_split_mode`).
        max_seq_len_in_batch: upper bound of kv_seq_len; never read from the device here,
            so the call does not synchronise (the reference does `.max().item()`, :272).
        output: optional [bsz, num_heads, q_len, head_dim] buffer; as in the reference it
            receives the CACHE-ONLY attention (:340-365), not the returned tensor.
        mid_output, mid_output_lse: optional fp32 scratch in the reference's shapes
            (:276-281); validated as the reference does (:286-291), written only in split
            mode "block".
        sm_scale: defaults to 1/sqrt(head_dim) (:271).
        kv_group_num: query heads per KV head; head h reads KV head h // kv_group_num (:71).

    Returns:
        A new tensor [bsz, num_heads, q_len, head_dim] of q's dtype (:373-376).
    """
    out, _ = _decode(
        q, k_cache, v_cache, current_k, current_v, mask, kv_seq_len, block_size, max_seq_len_in_batch,
        output, mid_output, mid_output_lse, sm_scale, kv_group_num,
        want_lse=False, out_dtype=None, with_tree=True,
    )
    return out


def flash_decoding_attention_paged(
    q, k_pages, v_pages, block_table, current_k, current_v, mask, kv_seq_len, max_seq_len_in_batch=None,
    sm_scale=None, kv_group_num=1, *, return_lse: bool = False,
):
    """The same operator over a paged KV cache, the layout the reference's docstring announces
    (flash_tree_attn.py:233) and its README lists as to do, while its kernels index a dense padded
    cache (:72-73).

    Args:
        k_pages, v_pages: [n_pages, num_kv_heads, page_size, head_dim] pools of pages shared by all
            sequences; page_size a multiple of 64.
        block_table: [bsz, max_pages] int32; row r of sequence b is row r % page_size of page
            block_table[b, r // page_size].  Entries past ceil(kv_seq_len[b] / page_size) are
            never read.
        others: as flash_decoding_attention.

    Returns the attention [bsz, num_heads, q_len, head_dim] (and the fp32 LSE if `return_lse`).
    Nothing is gathered or copied: the stage-1 kernels look the page of every 64-row tile up.
    """
    out, lse = _decode(
        q, k_pages, v_pages, current_k, current_v, mask, kv_seq_len, 64, max_seq_len_in_batch,
        None, None, None, sm_scale, kv_group_num,
        want_lse=return_lse, out_dtype=None, with_tree=True, block_table=block_table,
    )
    return (out, lse) if return_lse else out


def flash_decoding_attention_with_lse(
    q, k_cache, v_cache, current_k, current_v, mask, kv_seq_len, block_size=64, max_seq_len_in_batch=None,
    output=None, mid_output=None, mid_output_lse=None, sm_scale=None, kv_group_num=1,
    *, out_dtype: Optional[torch.dtype] = None, with_tree: bool = True,
    out_buf: Optional[torch.Tensor] = None, lse_buf: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same operator, also returning the fp32 natural-log LSE [bsz, num_heads, q_len] of the
    merged softmax.  `out_dtype=torch.float32` keeps the result unrounded and
    `with_tree=False` leaves the tree tokens out: together they give the (O, LSE) partial of
    one KV-range shard, to be merged across shards (see dist.py).  `out_buf` / `lse_buf` make
    the call write into caller-owned contiguous tensors instead of new ones.  The reference
    keeps its LSE internal and in 16 bits (flash_tree_attn.py:285,:373).
    """
    return _decode(
        q, k_cache, v_cache, current_k, current_v, mask, kv_seq_len, block_size, max_seq_len_in_batch,
        output, mid_output, mid_output_lse, sm_scale, kv_group_num,
        want_lse=True, out_dtype=out_dtype, with_tree=with_tree, out_buf=out_buf, lse_buf=lse_buf,
    )


def commit_accepted(k_cache, v_cache, current_k, current_v, kv_seq_len, accept_idx, accept_len, *,
                    kv_group_num: int = 1, block_table: Optional[torch.Tensor] = None) -> None:
    """The step after the operator in a speculative-decoding loop: append the accepted tree nodes'
    keys and values to the cache, in place, and grow `kv_seq_len`, in place.

    Args:
        k_cache, v_cache: the caches the operator read (dense [bsz, num_kv_heads, ctx, head_dim],
            or pools of pages with `block_table`), updated in place.
        current_k, current_v: the tree nodes' keys/values as given to the operator.
        kv_seq_len: [bsz] int32/int64 on the device, updated in place (+= accept_len, at most ctx).
        accept_idx: [bsz, max_accept] int32 tree-node indices in path order.
        accept_len: [bsz] int32 number of accepted nodes per sequence.

    Node accept_idx[b, i] becomes cache row kv_seq_len[b] + i.  Asynchronous on the current stream,
    no host synchronisation.  The reference has no such step (its tree tokens stay outside the
    cache, README), so this follows the rule stated in include/fta.h only.
    """
    lib = _lib.load()
    assert k_cache.is_cuda and kv_seq_len.is_cuda, "commit_accepted runs on CUDA tensors only"
    assert k_cache.dtype == v_cache.dtype == current_k.dtype == current_v.dtype
    assert k_cache.dtype in (torch.float16, torch.bfloat16)
    assert _rows_ok(k_cache) and _rows_ok(v_cache), "caches are updated in place and must have 16-byte rows"
    assert kv_seq_len.dtype in (torch.int32, torch.int64) and kv_seq_len.is_contiguous()
    dev = k_cache.device
    B = kv_seq_len.numel()
    Hkv, D = int(k_cache.size(1)), int(k_cache.size(3))
    hk, Q = int(current_k.size(1)), int(current_k.size(2))
    G = int(kv_group_num)
    assert hk in (Hkv, Hkv * G) and current_v.size(1) == hk
    if not _rows_ok(current_k):
        current_k = current_k.contiguous()
    if not _rows_ok(current_v):
        current_v = current_v.contiguous()
    accept_idx = accept_idx.to(device=dev, dtype=torch.int32)
    if accept_idx.stride(-1) != 1:
        accept_idx = accept_idx.contiguous()
    accept_len = accept_len.to(device=dev, dtype=torch.int32).contiguous()
    assert accept_idx.dim() == 2 and accept_idx.size(0) == B and accept_len.numel() == B

    p = _lib.FtaCommitParams()
    p.cur_k = current_k.data_ptr(); p.ck_sb, p.ck_sh, p.ck_st = current_k.stride(0), current_k.stride(1), current_k.stride(2)
    p.cur_v = current_v.data_ptr(); p.cv_sb, p.cv_sh, p.cv_st = current_v.stride(0), current_v.stride(1), current_v.stride(2)
    p.k_cache = k_cache.data_ptr(); p.k_sb, p.k_sh, p.k_st = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    p.v_cache = v_cache.data_ptr(); p.v_sb, p.v_sh, p.v_st = v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
    p.accept_idx = accept_idx.data_ptr(); p.ai_sb = accept_idx.stride(0)
    p.accept_len = accept_len.data_ptr()
    p.kv_seq_len = kv_seq_len.data_ptr()
    p.len_is_i64 = 1 if kv_seq_len.dtype == torch.int64 else 0
    p.cur_head_mul = G if (hk == Hkv * G and G > 1) else 1
    keep = [accept_idx, accept_len, current_k, current_v]
    if block_table is not None:
        if block_table.dtype != torch.int32 or not block_table.is_contiguous() or block_table.device != dev:
            block_table = block_table.to(device=dev, dtype=torch.int32).contiguous()
        p.block_table = block_table.data_ptr(); p.bt_sb = block_table.stride(0)
        p.page_size = int(k_cache.size(2)); p.n_pages = int(k_cache.size(0))
        p.ctx = int(block_table.size(1)) * p.page_size
        keep.append(block_table)
    else:
        assert k_cache.size(0) >= B
        p.ctx = int(k_cache.size(2))
    p.B, p.Hkv, p.Q, p.D, p.max_accept = B, Hkv, Q, D, int(accept_idx.size(1))
    _lib.check(lib.fta_commit_accepted(C.byref(p), torch.cuda.current_stream(dev).cuda_stream), "fta_commit_accepted")
    # the temporaries above are read by the kernels after this returns: tie them to the stream
    for t in keep:
        t.record_stream(torch.cuda.current_stream(dev))


def check_status() -> None:
    """Synchronise the current device and raise if a kernel of the tcgen05 stage-1 family gave up on
    one of its bounded barrier waits since the last check (a protocol error: the block then leaves
    early and the call's output is not a result).  The status is sticky until read here.  The
    operator itself never synchronises, so a caller that wants this certainty calls it at a point
    where a synchronisation is acceptable, e.g. once per decoded token batch or at shutdown."""
    st = _lib.load().fta_umma_status()
    if st < 0:
        raise RuntimeError("fta_umma_status: the status word could not be read")
    if st:
        raise RuntimeError(f"tcgen05 stage-1 kernel: a bounded barrier wait ran out (site code {st:#x}); "
                           "outputs of calls since the last check are not results")


def merge_partials(part_o: torch.Tensor, part_lse: torch.Tensor, out_dtype: torch.dtype = torch.float32):
    """LSE-merge n normalised partial attentions: part_o [n, rows.., D] fp32, part_lse
    [n, rows..] fp32 -> (out [rows.., D], lse [rows..]).  Used after the all-gather of
    KV-range shards; restates the reference's stage-2 recurrence (flash_tree_attn.py:195-208).
    """
    lib = _lib.load()
    assert part_o.is_cuda and part_o.dtype == torch.float32 and part_lse.dtype == torch.float32
    n, D = part_o.size(0), part_o.size(-1)
    # parts may be slices of one gather buffer: each part contiguous, any 16-byte-aligned stride
    # between parts
    if not (part_o[0].is_contiguous() and part_o.stride(0) % 4 == 0 and part_o.data_ptr() % 16 == 0):
        part_o = part_o.contiguous()
    if not part_lse[0].is_contiguous():
        part_lse = part_lse.contiguous()
    rows = part_lse[0].numel()
    assert part_o[0].numel() == rows * D
    out = torch.empty(part_o.shape[1:], dtype=out_dtype, device=part_o.device)
    lse = torch.empty(part_lse.shape[1:], dtype=torch.float32, device=part_o.device)
    mp = _lib.FtaMergeParams()
    mp.part_o = part_o.data_ptr(); mp.po_ss = part_o.stride(0)
    mp.part_lse = part_lse.data_ptr(); mp.pl_ss = part_lse.stride(0)
    mp.n_parts, mp.rows, mp.D, mp.out_dtype = n, rows, D, _DT[out_dtype]
    mp.out = out.data_ptr(); mp.lse = lse.data_ptr()
    stream = torch.cuda.current_stream(part_o.device).cuda_stream
    _lib.check(lib.fta_merge_parts(C.byref(mp), stream), "fta_merge_parts")
    return out, lse
