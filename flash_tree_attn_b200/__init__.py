"""B200-native tree-attention decode: a drop-in for `flash_tree_attn.flash_decoding_attention`.

    from flash_tree_attn_b200 import flash_decoding_attention

The arithmetic lives in libfta.so (hand-written sm_100a CUDA behind the C ABI of
include/fta.h); build it with `python -m flash_tree_attn_b200.build`.
"""
from .op import (  # noqa: F401
    check_status,
    commit_accepted,
    flash_decoding_attention,
    flash_decoding_attention_paged,
    flash_decoding_attention_with_lse,
    merge_partials,
    prepare,
    set_grid_override,
    set_kernel,
    set_split_mode,
)

from .speculative import DraftTree, TreeVerifyAttention, accept_longest_path  # noqa: F401,E402

__all__ = [
    "check_status",
    "DraftTree",
    "TreeVerifyAttention",
    "accept_longest_path",
    "commit_accepted",
    "flash_decoding_attention",
    "flash_decoding_attention_paged",
    "flash_decoding_attention_with_lse",
    "merge_partials",
    "prepare",
    "set_split_mode",
    "set_kernel",
    "set_grid_override",
]
