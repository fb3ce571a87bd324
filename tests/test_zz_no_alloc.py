"""GPU: the entry point for callers that cannot allocate device memory (fta_decode_static).

Some users of this library run where cudaMalloc is not theirs to call: inside a serving
runtime that has claimed the whole device heap, or as a plugin that must leave its host's
allocator alone.  For them the library carries its own fixed scratch array.  This test calls
that entry point through the C ABI, twice in a row (the array is shared between calls and
keeps the previous call's contents), and checks each result against what the ordinary entry
point returns for the same inputs and against the fp32 oracle, to the tolerance the parity tests
use; it also checks that the device's free memory is the same after the call as before it.  The
file sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

OUT_TOL = 2e-3
LSE_TOL = 1e-3


def _inputs(seed, lens):
    from flash_tree_attn_b200.workloads import Workload, make_inputs

    w = Workload("noalloc", 3, 8, 2, 128, 32, torch.float16, 2048, lens, "random", seed=seed)
    return w, make_inputs(w, "cuda")


@pytest.mark.parametrize("kernel", ["mma", "auto"])
def test_static_scratch_entry_point_matches_regular_one(kernel):
    assert torch.cuda.is_available()
    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200 import _lib
    from oracle.tree_attention_oracle import tree_attention_oracle

    lib = _lib.load()
    assert lib.fta_static_scratch_bytes() == 24 << 20
    fta.set_kernel(kernel)
    try:
        for seed, lens in ((11, "fixed:2048,900,3"), (12, "fixed:70,2000,1111")):
            w, inp = _inputs(seed, lens)
            args = (inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"], inp["mask"],
                    inp["kv_seq_len"], 64, w.ctx)
            # the ordinary entry point, with a torch-allocated workspace
            ref = fta.prepare(*args, kv_group_num=w.G, want_lse=True)
            ref_out, ref_lse = ref.run()
            ref_out, ref_lse = ref_out.clone(), ref_lse.clone()
            # the same call through fta_decode_static: fresh outputs, no workspace at all
            call = fta.prepare(*args, kv_group_num=w.G, want_lse=True)
            call.out.fill_(float("nan"))
            call.lse.fill_(float("nan"))
            call.p.workspace = None
            call.p.workspace_bytes = 0
            # The first call on a device is the documented set-up call (it resolves the address of the
            # library's scratch array, which is when the CUDA runtime loads that part of the library
            # image onto the device); what is measured is a call after it.
            assert lib.fta_decode_static(C.byref(call.p), call.stream) == 0
            torch.cuda.synchronize()
            call.out.fill_(float("nan"))
            call.lse.fill_(float("nan"))
            torch.cuda.synchronize()
            # nothing may be taken from the device heap: neither through torch's allocator nor
            # behind its back (cudaMemGetInfo sees every allocation of the process)
            torch_before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
            rc = lib.fta_decode_static(C.byref(call.p), call.stream)
            assert rc == 0, lib.fta_strerror(rc)
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == torch_before
            assert torch.cuda.mem_get_info()[0] == free_before
            assert lib.fta_umma_status() == 0
            assert torch.isfinite(call.out.float()).all()
            assert (call.out.float() - ref_out.float()).abs().max().item() <= OUT_TOL
            assert (call.lse - ref_lse).abs().max().item() <= LSE_TOL
            ora = tree_attention_oracle(inp["q"], inp["k_cache"], inp["v_cache"], inp["current_k"], inp["current_v"],
                                        inp["mask"], inp["kv_seq_len"], None, w.G)
            assert (call.out.float() - ora["out"]).abs().max().item() <= OUT_TOL
            assert (call.lse - ora["lse"]).abs().max().item() <= LSE_TOL
    finally:
        fta.set_kernel("auto")


def test_static_scratch_rejects_oversized_requests():
    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200 import _lib

    lib = _lib.load()
    # partial-result slots scale with the number of stage-1 blocks: ask for far more blocks than
    # the fixed array has room for
    B, H = 4, 8
    p = _lib.FtaParams()
    dummy = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    lens = torch.zeros(B, dtype=torch.int32, device="cuda")
    for name in ("q", "k_cache", "v_cache", "cur_k", "cur_v", "out"):
        setattr(p, name, dummy.data_ptr())
    p.mask = torch.zeros(64, device="cuda").data_ptr()
    p.kv_seq_len = lens.data_ptr()
    p.cur_head_mul = 1
    p.B, p.H, p.Hkv, p.Q, p.D, p.ctx = B, H, H, 4, 128, 64
    p.dtype = p.out_dtype = _lib.DTYPE_F16
    p.sm_scale = 1.0
    p.with_tree = 1
    p.split_mode = _lib.SPLIT_BALANCED
    p.grid_override = 4000  # 2 * 4000 * 16 rows * 129 floats = 66 MB of partial slots
    for f in ("q_sb", "q_sh", "q_sq", "k_sb", "k_sh", "k_st", "v_sb", "v_sh", "v_st", "ck_sb", "ck_sh", "ck_st",
              "cv_sb", "cv_sh", "cv_st", "o_sb", "o_sh", "o_sq"):
        setattr(p, f, 128)
    assert lib.fta_decode_static(C.byref(p), None) == _lib.FTA_E_TOO_LARGE
