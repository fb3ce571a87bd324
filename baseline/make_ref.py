"""Places the reference's operator under baseline/_ref/ (git-ignored) so that it can be timed on
a GPU machine that has no reference checkout.

    python baseline/make_ref.py /path/to/reference

The reference module cannot be imported whole: it runs its CUDA benchmark at import
(flash_tree_attn.py:487).  Two files are written, both the reference's own lines 1-376 (the two
Triton kernels and flash_decoding_attention) followed by its late
`import torch.nn.functional as F` (:401, needed by :373):

  _ref/flash_tree_attn_head.py          unmodified
  _ref/flash_tree_attn_head_anydtype.py the one token `.half()` at :370 replaced by
                                        `.to(q.dtype)`: without it a bf16 call raises at :371
                                        (Half x BFloat16 matmul); no Triton line is touched

Nothing under baseline/_ref/ is committed or imported by the product.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEAD_LINES = 376


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    src = open(os.path.join(sys.argv[1], "flash_tree_attn.py")).read().split("\n")
    head = src[:HEAD_LINES]
    tail = "\nimport torch.nn.functional as F\n"
    out = os.path.join(HERE, "_ref")
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "flash_tree_attn_head.py"), "w") as f:
        f.write("\n".join(head) + tail)
    line = head[369]
    assert line.count(".half()") == 1, "unexpected reference text at line 370: " + line
    shim = list(head)
    shim[369] = line.replace(".half()", ".to(q.dtype)")
    with open(os.path.join(out, "flash_tree_attn_head_anydtype.py"), "w") as f:
        f.write("\n".join(shim) + tail)
    print("wrote", out)


if __name__ == "__main__":
    main()
