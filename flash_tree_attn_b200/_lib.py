"""ctypes binding of libfta.so, the C-ABI library declared in include/fta.h.

The library is the product: there is no fallback.  If it cannot be loaded, importing any
operator of this package raises, and on a machine with a GPU nothing else will compute the
attention in its place.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FTA_LIB_PATH points at a library built elsewhere (same ABI); the default is the in-tree build.
LIB_PATH = os.environ.get("FTA_LIB_PATH") or os.path.join(_HERE, "libfta.so")

ABI_VERSION = 101  # FTA_VERSION of include/fta.h this binding was written against

FTA_OK = 0
FTA_E_BADARG = 1
FTA_E_UNSUPPORTED = 2
FTA_E_WORKSPACE = 3
FTA_E_CUDA = 4
FTA_E_TOO_LARGE = 5

DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
SPLIT_BALANCED, SPLIT_FIXED = 0, 1
KERNEL_AUTO, KERNEL_MMA, KERNEL_UMMA = 0, 1, 2

_i64, _i32, _vp, _f32 = C.c_int64, C.c_int32, C.c_void_p, C.c_float


class FtaParams(C.Structure):
    """Mirror of `struct FtaParams` (include/fta.h); field order and types must match."""

    _fields_ = [
        ("q", _vp), ("q_sb", _i64), ("q_sh", _i64), ("q_sq", _i64),
        ("k_cache", _vp), ("k_sb", _i64), ("k_sh", _i64), ("k_st", _i64),
        ("v_cache", _vp), ("v_sb", _i64), ("v_sh", _i64), ("v_st", _i64),
        ("cur_k", _vp), ("ck_sb", _i64), ("ck_sh", _i64), ("ck_st", _i64),
        ("cur_v", _vp), ("cv_sb", _i64), ("cv_sh", _i64), ("cv_st", _i64),
        ("mask", _vp), ("m_sb", _i64), ("m_sh", _i64), ("m_sq", _i64),
        ("kv_seq_len", _vp), ("len_is_i64", _i32), ("cur_head_mul", _i32),
        ("out", _vp), ("o_sb", _i64), ("o_sh", _i64), ("o_sq", _i64),
        ("out_cache", _vp), ("oc_sb", _i64), ("oc_sh", _i64), ("oc_sq", _i64),
        ("lse", _vp), ("l_sb", _i64), ("l_sh", _i64),
        ("workspace", _vp), ("workspace_bytes", _i64),
        ("mid_o", _vp), ("mo_sb", _i64), ("mo_sh", _i64), ("mo_ss", _i64), ("mo_sq", _i64),
        ("mid_lse", _vp), ("ml_sb", _i64), ("ml_sh", _i64), ("ml_ss", _i64),
        ("mid_splits", _i32),
        ("tree_o", _vp), ("tree_lse", _vp),
        ("B", _i32), ("H", _i32), ("Hkv", _i32), ("Q", _i32), ("D", _i32), ("ctx", _i32),
        ("dtype", _i32), ("out_dtype", _i32), ("sm_scale", _f32),
        ("split_mode", _i32), ("split_tokens", _i32), ("with_tree", _i32), ("kernel", _i32),
        ("grid_override", _i32), ("reserved_", _i32),
        ("block_table", _vp), ("bt_sb", _i64), ("page_size", _i32), ("n_pages", _i32),
    ]


class FtaMergeParams(C.Structure):
    """Mirror of `struct FtaMergeParams` (include/fta.h)."""

    _fields_ = [
        ("part_o", _vp), ("po_ss", _i64),
        ("part_lse", _vp), ("pl_ss", _i64),
        ("n_parts", _i32), ("rows", _i32), ("D", _i32), ("out_dtype", _i32),
        ("out", _vp), ("lse", _vp),
    ]


class FtaCommitParams(C.Structure):
    """Mirror of `struct FtaCommitParams` (include/fta.h)."""

    _fields_ = [
        ("cur_k", _vp), ("ck_sb", _i64), ("ck_sh", _i64), ("ck_st", _i64),
        ("cur_v", _vp), ("cv_sb", _i64), ("cv_sh", _i64), ("cv_st", _i64),
        ("k_cache", _vp), ("k_sb", _i64), ("k_sh", _i64), ("k_st", _i64),
        ("v_cache", _vp), ("v_sb", _i64), ("v_sh", _i64), ("v_st", _i64),
        ("accept_idx", _vp), ("ai_sb", _i64),
        ("accept_len", _vp), ("kv_seq_len", _vp),
        ("block_table", _vp), ("bt_sb", _i64),
        ("len_is_i64", _i32), ("cur_head_mul", _i32), ("page_size", _i32), ("n_pages", _i32),
        ("B", _i32), ("Hkv", _i32), ("Q", _i32), ("D", _i32), ("ctx", _i32), ("max_accept", _i32),
    ]


FTA_MAX_RANKS = 8


class FtaExchangeParams(C.Structure):
    """Mirror of `struct FtaExchangeParams` (include/fta.h)."""

    _fields_ = [
        ("part", _vp * FTA_MAX_RANKS), ("flag_peer", _vp * FTA_MAX_RANKS),
        ("out_peer", _vp * FTA_MAX_RANKS), ("lse_peer", _vp * FTA_MAX_RANKS),
        ("flag_local", _vp), ("status", _vp), ("done", _vp), ("timeout_ns", _i64),
        ("world", _i32), ("rank", _i32), ("epoch", C.c_uint32), ("rows", _i32), ("D", _i32), ("out_dtype", _i32),
        ("out", _vp), ("lse", _vp),
    ]


# every symbol include/fta.h declares: (restype, argtypes)
SYMBOLS = {
    "fta_version": (C.c_int, []),
    "fta_strerror": (C.c_char_p, [C.c_int]),
    "fta_last_cuda_error": (C.c_char_p, []),
    "fta_workspace_bytes": (_i64, [C.POINTER(FtaParams)]),
    "fta_decode": (C.c_int, [C.POINTER(FtaParams), _vp]),
    "fta_decode_static": (C.c_int, [C.POINTER(FtaParams), _vp]),
    "fta_static_scratch_bytes": (_i64, []),
    "fta_stage1": (C.c_int, [C.POINTER(FtaParams), _vp]),
    "fta_stage2": (C.c_int, [C.POINTER(FtaParams), _vp]),
    "fta_merge_parts": (C.c_int, [C.POINTER(FtaMergeParams), _vp]),
    "fta_commit_accepted": (C.c_int, [C.POINTER(FtaCommitParams), _vp]),
    "fta_exchange_merge": (C.c_int, [C.POINTER(FtaExchangeParams), _vp]),
    "fta_plan_host": (_i64, [C.POINTER(FtaParams), C.POINTER(_i64), C.POINTER(_i64), _i64,
                             C.POINTER(_i32), C.POINTER(_i32)]),
    "fta_plan_grid": (C.c_int, [C.POINTER(FtaParams)]),
    "fta_umma_status": (C.c_int, []),
}

_lib = None


class FtaLibraryMissing(RuntimeError):
    pass


def load():
    """Load libfta.so once; raise FtaLibraryMissing (never fall back) if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FtaLibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m flash_tree_attn_b200.build` "
            "(there is no non-CUDA fallback for this operator)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.fta_version() != ABI_VERSION:
        raise FtaLibraryMissing(f"{LIB_PATH} has ABI version {lib.fta_version()}, this package binds version {ABI_VERSION}: "
                                "rebuild it with `python -m flash_tree_attn_b200.build`")
    _lib = lib
    return lib


class FtaError(RuntimeError):
    def __init__(self, code: int, where: str):
        lib = load()
        msg = lib.fta_strerror(code).decode()
        if code == FTA_E_CUDA:
            msg += ": " + lib.fta_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} (code {code})")
        self.code = code


def check(code: int, where: str) -> None:
    if code != FTA_OK:
        raise FtaError(code, where)
