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
    assert r.stdout.count("EXCHANGE_OK") == 4, r.stdout[-2000:]  # two ranks x two forms


class _Emulated:
    """Two 'ranks' whose memory is all on this GPU: partials, flag arrays [2 * world], result
    buffers and counters as fta_exchange_merge wants them, so that the kernel of either rank can
    be launched alone once the other rank's flags have been put there by hand."""

    def __init__(self, rows, D, seed=3):
        self.rows, self.D, self.world = rows, D, 2
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.bufs = []
        for s in range(2):
            o = torch.randn(rows, D, device="cuda", generator=g)
            l = torch.randn(rows, device="cuda", generator=g) * 3
            l[s::7] = float("-inf")  # empty partial rows contribute nothing
            self.bufs.append(torch.cat([o.reshape(-1), l]))
        self.flags = torch.zeros(2, 4, dtype=torch.int32, device="cuda")   # [rank][round * world + from]
        self.words = torch.zeros(2, 3, dtype=torch.int32, device="cuda")   # [rank][status, finished blocks, waits lost in the launch]
        self.out = torch.full((2, rows, D), float("nan"), device="cuda")
        self.lse = torch.full((2, rows), float("nan"), device="cuda")

    def want(self):
        """What the merge must give: the oracle's closed form (fp32, to rounding), and, bit for
        bit, the library's own merge of gathered partials (the NCCL path folds the ranks' partials
        in the same order with the same arithmetic)."""
        import flash_tree_attn_b200 as fta
        from oracle.tree_attention_oracle import merge_partials_oracle

        n = self.rows * self.D
        po = torch.stack([b[:n].view(self.rows, self.D) for b in self.bufs])
        pl = torch.stack([b[n:] for b in self.bufs])
        o, l = fta.merge_partials(po, pl, torch.float32)
        oo, ol = merge_partials_oracle(po, pl)
        # rows whose partials are all empty have no LSE to compare (-inf on both sides)
        fin = torch.isfinite(ol)
        assert torch.equal(torch.isfinite(l), fin)
        assert (o - oo).abs().max().item() <= 1e-5 and (l[fin] - ol[fin]).abs().max().item() <= 1e-5
        self.oracle = (oo, ol)
        return o, l

    def check_oracle(self, out, lse, rows=slice(None)):
        """fp32 results of the exchange kernels against the oracle's merge."""
        oo, ol = self.oracle
        fin = torch.isfinite(ol[rows])
        assert (out[rows] - oo[rows]).abs().max().item() <= 1e-5
        assert (lse[rows][fin] - ol[rows][fin]).abs().max().item() <= 1e-5

    def launch(self, rank, epoch, scatter, timeout_ns=200_000_000):
        import ctypes as C

        from flash_tree_attn_b200 import _lib

        p = _lib.FtaExchangeParams()
        for s in range(2):
            p.part[s] = self.bufs[s].data_ptr()
            p.flag_peer[s] = self.flags[s].data_ptr() + 4 * rank
            if scatter:
                p.out_peer[s] = self.out[s].data_ptr()
                p.lse_peer[s] = self.lse[s].data_ptr()
        p.flag_local = self.flags[rank].data_ptr()
        p.status = self.words[rank].data_ptr()
        p.done = self.words[rank].data_ptr() + 4 if scatter else None
        p.timeout_ns = timeout_ns
        p.world, p.rank, p.epoch, p.rows, p.D, p.out_dtype = 2, rank, epoch, self.rows, self.D, _lib.DTYPE_F32
        if not scatter:
            p.out, p.lse = self.out[rank].data_ptr(), self.lse[rank].data_ptr()
        _lib.check(_lib.load().fta_exchange_merge(C.byref(p), torch.cuda.current_stream().cuda_stream), "fta_exchange_merge")
        torch.cuda.synchronize()
        return int(self.words[rank, 0].item())


def _needs_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")


def test_gather_form_on_one_gpu_and_its_timeout():
    """The gather kernel alone.  (1) The peer's flag already holds the epoch: the merge must equal
    fta_merge_parts on the same partials bit for bit, and the signal must have been written.
    (2) A flag nothing sets: the wait runs out after its limit, the status word names the late
    rank, nothing is stored and the context stays usable."""
    _needs_gpu()
    e = _Emulated(4096, 128)
    want_o, want_l = e.want()
    e.flags[0, 1] = 5  # "rank 1 has finished call 5"
    assert e.launch(0, 5, scatter=False) == 0
    assert int(e.flags[1, 0].item()) == 5  # rank 0's signal in rank 1's array
    assert torch.equal(e.out[0], want_o) and torch.equal(e.lse[0], want_l)
    e.check_oracle(e.out[0], e.lse[0])

    e.out.fill_(float("nan"))
    assert e.launch(0, 6, scatter=False, timeout_ns=50_000_000) == 0b10  # rank 1 never signals call 6
    assert torch.isnan(e.out).all()
    # the context is intact: the same call succeeds once the flag is there
    e.words.zero_()
    e.flags[0, 1] = 6
    assert e.launch(0, 6, scatter=False) == 0
    assert torch.equal(e.out[0], want_o)


def test_scatter_form_on_one_gpu_and_its_timeouts():
    """The scatter kernel alone, a row count the ranks do not divide.  Each rank merges its slice
    and stores it into both result buffers; after both ranks have run, both buffers hold the full
    merge, bit for bit what fta_merge_parts gives.  Then the two waits that can run out: the
    first round (nothing stored) and the second (own slice stored, status says the peer's is not)."""
    _needs_gpu()
    rows, D = 4097, 128
    e = _Emulated(rows, D)
    want_o, want_l = e.want()
    per = (rows + 1) // 2
    e.flags[0, 1] = e.flags[0, 3] = 9  # rank 1's two signals of call 9, as rank 0 will see them
    e.flags[1, 0] = e.flags[1, 2] = 0
    assert e.launch(0, 9, scatter=True) == 0
    assert int(e.flags[1, 0].item()) == 9 and int(e.flags[1, 2].item()) == 9  # both of rank 0's signals
    assert int(e.words[0, 1].item()) == 0  # the block counter is back at zero
    for s in range(2):
        assert torch.equal(e.out[s, :per], want_o[:per]) and torch.isnan(e.out[s, per:]).all()
    assert e.launch(1, 9, scatter=True) == 0
    for s in range(2):
        assert torch.equal(e.out[s], want_o) and torch.equal(e.lse[s], want_l)
        e.check_oracle(e.out[s], e.lse[s])

    # first round runs out: nothing stored, counter reset, no second-round signal
    e.out.fill_(float("nan"))
    e.flags[1, 2] = 0
    assert e.launch(0, 10, scatter=True, timeout_ns=50_000_000) == 0b10
    assert torch.isnan(e.out).all() and int(e.words[0, 1].item()) == 0 and int(e.flags[1, 2].item()) == 0
    # second round runs out: the first-round flag is there, the second never comes
    e.words.zero_()
    e.flags[0, 1] = 10
    assert e.launch(0, 10, scatter=True, timeout_ns=50_000_000) == 0b10 << 8
    assert torch.equal(e.out[1, :per], want_o[:per])
    # and the context is still usable
    e.words.zero_()
    e.flags[0, 3] = 10
    assert e.launch(0, 10, scatter=True) == 0
    # a status word the host has not read yet (an old timeout) is sticky, but it must not make
    # later calls skip their second round: the peers would then wait out their limit on every call
    e.words[0, 0] = 0b10
    e.flags[0, 1] = e.flags[0, 3] = 11
    e.flags[1, 2] = 0
    assert e.launch(0, 11, scatter=True) == 0b10
    assert int(e.flags[1, 2].item()) == 11
    assert int(e.words[0, 1].item()) == 0 and int(e.words[0, 2].item()) == 0
