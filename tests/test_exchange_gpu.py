"""GPU: sequence-sharded decode merged over peer memory (fa_b200_fwd_exchange, flash_b200.dist.PeerExchange).

The exchange is built for one process per GPU; what a single GPU can show is shown here by giving one process the
buffers of several "ranks": the data path (each rank's partial lands in every rank's buffer, the merge over ranks
equals attention over the whole sequence), the bounded wait (a rank that never delivers makes the merge give up with
a status instead of hanging), and that the context stays usable afterwards.  With two or more GPUs the last test runs
real ranks as child processes.
"""
import ctypes as C
import os
import sys

import pytest
import torch

import parity_util as U
from flash_b200 import lib as L
from flash_b200 import ops
from oracle import api as OA

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
SHORT_WAIT = 40_000_000  # cycles: about 20 ms


class _Bufs:
    """world exchange buffers, all allocated by this process."""

    def __init__(self, world, rows, d):
        lib = L.load()
        self.nbytes = lib.fa_b200_exchange_bytes(world, rows, d)
        self.ptrs = []
        for _ in range(world):
            ptr, handle = C.c_void_p(), C.create_string_buffer(64)
            L.check(lib.fa_b200_exchange_alloc(self.nbytes, C.byref(ptr), handle))
            self.ptrs.append(ptr)
        self.world = world

    def view(self, rank, timeout_cycles=0):
        x = L.Exchange()
        for r, ptr in enumerate(self.ptrs):
            x.bufs[r] = ptr.value
        x.buf_bytes, x.world, x.rank, x.timeout_cycles = self.nbytes, self.world, rank, timeout_cycles
        return x

    def free(self):
        torch.cuda.synchronize()
        for ptr in self.ptrs:
            L.load().fa_b200_exchange_free(ptr)


def _status():
    return L.load().fa_b200_check_status(torch.cuda.current_stream().cuda_stream)


def _case(seed, b, s_q, h, hk, d, s_k):
    g = torch.Generator().manual_seed(seed)
    return U.normal((b, s_q, h, d), BF, g), U.normal((b, s_k, hk, d), BF, g), U.normal((b, s_k, hk, d), BF, g)


@pytest.mark.parametrize("s_q,s_k", [(1, 6000), (4, 2500), (1, 300)])
def test_a_single_rank_exchange_is_plain_attention(s_q, s_k):
    q, k, v = _case(1, 3, s_q, 16, 4, 128, s_k)
    bufs = _Bufs(1, 3 * s_q * 16, 128)
    for step in range(3):  # the two parities of the buffer, then the first again
        out, lse = ops.attention_forward_exchange(q.cuda(), k.cuda(), v.cuda(), bufs.view(0), softmax_scale=128 ** -0.5,
                                                  causal=True, kv_pos_offset=0, kv_total=s_k)
        go, gl = OA.flash_attn_with_kvcache(q, k, v, cache_seqlens=s_k, causal=True)
        U.check_rules(out, lse, go, gl, tag=f"world 1 step {step}")
    assert _status() == 0
    bufs.free()


def test_two_ranks_on_one_gpu_merge_to_the_whole_sequence():
    """Rank 1 goes first with a short wait: its partial reaches both buffers, its own merge gives up (rank 0 has not
    delivered yet) and says so.  Rank 0 then finds rank 1's flag set, and its merge covers the whole sequence."""
    b, s_q, h, hk, d, s_k = 2, 2, 16, 4, 128, 5000
    q, k, v = _case(2, b, s_q, h, hk, d, s_k)
    cut = 2304
    bufs = _Bufs(2, b * s_q * h, d)
    go, gl = OA.flash_attn_with_kvcache(q, k, v, cache_seqlens=s_k, causal=True)
    kw = dict(softmax_scale=d ** -0.5, causal=True, kv_total=s_k)
    for step in range(3):
        ops.attention_forward_exchange(q.cuda(), k[:, cut:].cuda(), v[:, cut:].cuda(), bufs.view(1, SHORT_WAIT), kv_pos_offset=cut, **kw)
        assert _status() != 0 and "did not deliver" in L.load().fa_b200_last_error().decode()
        out, lse = ops.attention_forward_exchange(q.cuda(), k[:, :cut].cuda(), v[:, :cut].cuda(), bufs.view(0, SHORT_WAIT), kv_pos_offset=0, **kw)
        assert _status() == 0
        U.check_rules(out, lse, go, gl, tag=f"two ranks step {step}")
        # rank 1 is now one step behind in what it has seen from rank 0, which is as far apart as ranks can get;
        # bring it level: its next call finds rank 0's flag of this step
    # the same shards through the all-gather-shaped path (fp32 partials + merge kernel) give the same bits
    parts = [ops.attention_forward(q.cuda(), k[:, lo:hi].cuda(), v[:, lo:hi].cuda(), partial_out=True, kv_pos_offset=lo, **kw)
             for lo, hi in ((0, cut), (cut, s_k))]
    o_all = torch.stack([p[0] for p in parts])
    lse_all = torch.stack([p[1].permute(0, 2, 1) for p in parts])
    ref_out, ref_lse = ops.combine(o_all, lse_all, out_dtype=BF)
    assert torch.equal(ref_out, out) and torch.equal(ref_lse.permute(0, 2, 1), lse)
    bufs.free()


def test_a_rank_that_never_delivers_ends_in_a_status_not_a_hang():
    q, k, v = _case(3, 2, 1, 8, 2, 128, 1000)
    bufs = _Bufs(2, 2 * 1 * 8, 128)
    ops.attention_forward_exchange(q.cuda(), k.cuda(), v.cuda(), bufs.view(0, SHORT_WAIT), softmax_scale=128 ** -0.5, causal=True,
                                   kv_pos_offset=0, kv_total=2000)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="did not deliver"):
        L.check(_status())
    assert _status() == 0  # reported once, then cleared
    # the context is intact: an ordinary call right after
    out, lse = ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), softmax_scale=128 ** -0.5, causal=True)
    go, gl = OA.flash_attn_func(q, k, v, causal=True)
    U.check_rules(out, lse, go, gl, tag="after a timed-out exchange")
    bufs.free()


def test_exchange_refuses_what_it_cannot_serve():
    q, k, v = _case(4, 2, 1, 8, 2, 128, 512)
    bufs = _Bufs(1, 4, 128)  # too few rows
    with pytest.raises(RuntimeError, match="too small"):
        ops.attention_forward_exchange(q.cuda(), k.cuda(), v.cuda(), bufs.view(0), softmax_scale=0.1, kv_pos_offset=0, kv_total=512)
    x = bufs.view(0)
    x.world = 99
    with pytest.raises(RuntimeError, match="rank / world"):
        ops.attention_forward_exchange(q.cuda(), k.cuda(), v.cuda(), x, softmax_scale=0.1, kv_pos_offset=0, kv_total=512)
    bufs.free()


def _rank_main(rank, world, port, q, k, v, ret):
    import torch.distributed as dist
    from flash_b200 import dist as D
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    px = D.PeerExchange(q.shape[0] * q.shape[1] * q.shape[2], q.shape[3], torch.device("cuda", rank))
    lo, hi = D.kv_shard_range(k.shape[1], world, rank)
    for _ in range(4):
        out, lse = D.sharded_decode(q.cuda(), k[:, lo:hi].cuda(), v[:, lo:hi].cuda(), kv_pos_offset=lo, kv_total=k.shape[1],
                                    causal=True, exchange=px)
    torch.cuda.synchronize()
    status = L.load().fa_b200_check_status(torch.cuda.current_stream().cuda_stream)
    ret[rank] = (out.cpu(), lse.cpu(), status)
    dist.barrier()
    px.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_real_ranks_over_nvlink():
    import torch.multiprocessing as mp
    world = min(4, torch.cuda.device_count())
    q, k, v = _case(5, 4, 1, 32, 8, 128, 20000)
    go, gl = OA.flash_attn_with_kvcache(q, k, v, cache_seqlens=20000, causal=True)
    os.environ["PYTHONPATH"] = os.pathsep.join(p for p in sys.path if p)  # the children import this module and the package
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, 29611, q, k, v, ret), nprocs=world, join=True)
    for r in range(world):
        out, lse, status = ret[r]
        assert status == 0
        U.check_rules(out, lse, go, gl, tag=f"rank {r}")
        assert torch.equal(out, ret[0][0]) and torch.equal(lse, ret[0][1])
