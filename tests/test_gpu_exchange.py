"""fta_exchange_merge on two GPUs of one box: child processes, one per GPU.  Skipped on a box
with a single GPU; the host-side layout and epoch logic is covered on CPU in test_dist_cpu.py."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_exchange_merge_matches_allgather_merge():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "_exchange_worker.py"), "8192", "6"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("EXCHANGE_OK") == 2, r.stdout[-2000:]


def _params(lib_mod, bufs, flags, status, rank, epoch, rows, D, out, lse, timeout_ns):
    """Two 'ranks' whose memory is all on this GPU: bufs[s] is rank s's packed partial, flags is
    this rank's flag array, and the signal meant for the peer lands in flags[2 + s]."""
    import ctypes as C

    p = lib_mod.FtaExchangeParams()
    for s, b in enumerate(bufs):
        p.part[s] = b.data_ptr()
        p.flag_peer[s] = flags.data_ptr() + 4 * (2 + s)
    p.flag_local = flags.data_ptr()
    p.status = status.data_ptr()
    p.timeout_ns = timeout_ns
    p.world, p.rank, p.epoch, p.rows, p.D, p.out_dtype = len(bufs), rank, epoch, rows, D, lib_mod.DTYPE_F32
    p.out, p.lse = out.data_ptr(), lse.data_ptr()
    return p, C.byref(p)


def test_exchange_merge_kernel_on_one_gpu_and_its_timeout():
    """The kernel alone, both 'ranks' in this GPU's memory.  (1) The peer's flag already holds the
    epoch: the merge must equal fta_merge_parts on the same partials bit for bit, and the signal
    must have been written.  (2) A flag nothing sets: the wait runs out after its limit, the
    status word names the late rank, nothing is stored and the context stays usable."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import flash_tree_attn_b200 as fta
    from flash_tree_attn_b200 import _lib

    lib = _lib.load()
    rows, D = 4096, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    bufs = []
    for s in range(2):
        o = torch.randn(rows, D, device="cuda", generator=g)
        l = torch.randn(rows, device="cuda", generator=g) * 3
        l[s::7] = float("-inf")  # empty partial rows contribute nothing
        bufs.append(torch.cat([o.reshape(-1), l]))
    po = torch.stack([b[: rows * D].view(rows, D) for b in bufs])
    pl = torch.stack([b[rows * D:] for b in bufs])
    want_o, want_l = fta.merge_partials(po, pl, torch.float32)
    stream = torch.cuda.current_stream().cuda_stream

    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((rows, D), float("nan"), device="cuda")
    lse = torch.full((rows,), float("nan"), device="cuda")
    flags[1] = 5  # "rank 1 has finished call 5"
    p, ref = _params(_lib, bufs, flags, status, 0, 5, rows, D, out, lse, 200_000_000)
    _lib.check(lib.fta_exchange_merge(ref, stream), "fta_exchange_merge")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert int(flags[2 + 1].item()) == 5  # this rank's signal to rank 1
    assert torch.equal(out, want_o) and torch.equal(lse, want_l)

    # a later call whose peer never signals
    out.fill_(float("nan"))
    p, ref = _params(_lib, bufs, flags, status, 0, 6, rows, D, out, lse, 50_000_000)
    _lib.check(lib.fta_exchange_merge(ref, stream), "fta_exchange_merge")
    torch.cuda.synchronize()
    assert int(status.item()) == 0b10
    assert torch.isnan(out).all()
    # the context is intact: the same call succeeds once the flag is there
    status.zero_()
    flags[1] = 6
    _lib.check(lib.fta_exchange_merge(ref, stream), "fta_exchange_merge")
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(out, want_o)
