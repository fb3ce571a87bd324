"""Generates tests/golden/*.npz by executing the REFERENCE's own flash_decoding_attention
(flash_tree_attn.py:216-376) on seeded inputs, on CPU, under the Triton interpreter.

Run in the development container only (it needs the reference checkout):
    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference
The reference module cannot be imported as is: it runs a CUDA benchmark at import
(flash_tree_attn.py:487).  Lines 1-376 plus its late `import torch.nn.functional as F`
(:401) are loaded from a temporary copy outside this repository (triton.jit needs a real
file for inspect.getsource); no reference source is written into the repository.
Each fixture stores the inputs and the reference's out / output / mid_output /
mid_output_lse so that the tests need neither the reference nor Triton.
"""
import importlib.util
import os
import sys
import tempfile

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from flash_tree_attn_b200.workloads import WORKLOADS, Workload, make_inputs  # noqa: E402


def load_reference(ref_dir):
    src = open(os.path.join(ref_dir, "flash_tree_attn.py")).read().split("\n")
    head = "\n".join(src[:376]) + "\nimport torch.nn.functional as F\n"
    tmp = tempfile.mkdtemp(prefix="fta_ref_")
    path = os.path.join(tmp, "_ref_head.py")
    with open(path, "w") as f:
        f.write(head)
    spec = importlib.util.spec_from_file_location("_ref_head", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


CASES = {
    # the plumbing configuration, exactly as specified
    "cfg1": (WORKLOADS["cfg1"], 0.0),
    # GQA with ragged lengths, one of them shorter than a block
    "gqa_ragged": (Workload("gqa_ragged", 2, 8, 4, 64, 16, torch.float16, 256, "fixed:200,37", "random",
                            seed=777, mask_batch=False), 0.0),
    # the reference test's mask convention: allowed entries are 1.0, not 0 (flash_tree_attn.py:409)
    "mask_one": (Workload("mask_one", 1, 4, 1, 128, 16, torch.float16, 128, "fixed:128", "random",
                          seed=778, scale=0.5), 1.0),
}


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <directory holding the reference's flash_tree_attn.py>")
    ref = load_reference(sys.argv[1])
    torch.manual_seed(0)
    for name, (w, allowed) in CASES.items():
        inp = make_inputs(w, "cpu", allowed=allowed)
        q, k, v = inp["q"], inp["k_cache"], inp["v_cache"]
        ck, cv, mask, lens = inp["current_k"], inp["current_v"], inp["mask"], inp["kv_seq_len"]
        # the reference's tail needs num_heads heads on current_k/v (flash_tree_attn.py:367)
        ck_ref = ck.repeat_interleave(w.G, dim=1)
        cv_ref = cv.repeat_interleave(w.G, dim=1)
        S = (w.ctx + w.block_size - 1) // w.block_size
        mid_o = torch.full((w.B, w.H, S, w.Q, w.D), float("nan"), dtype=torch.float32)
        mid_l = torch.full((w.B, w.H, S, w.Q), float("nan"), dtype=torch.float32)
        output = torch.zeros((w.B, w.H, w.Q, w.D), dtype=w.dtype)
        out = ref.flash_decoding_attention(q, k, v, ck_ref, cv_ref, mask, lens, w.block_size, w.ctx,
                                           output, mid_o, mid_l, None, w.G)
        np.savez(
            os.path.join(HERE, name + ".npz"),
            q=q.numpy(), k_cache=k.numpy(), v_cache=v.numpy(), current_k=ck.numpy(), current_v=cv.numpy(),
            mask=mask.numpy(), kv_seq_len=lens.numpy(), kv_group_num=np.int32(w.G), block_size=np.int32(w.block_size),
            ref_out=out.numpy(), ref_output=output.numpy(), ref_mid_o=mid_o.numpy(), ref_mid_lse=mid_l.numpy(),
        )
        print(name, "ok", tuple(out.shape), float(out.float().abs().max()))


if __name__ == "__main__":
    main()
