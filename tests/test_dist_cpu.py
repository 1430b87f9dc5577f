"""CPU (gloo, world_size 2 and 3): the host-side plumbing of the multi-GPU paths -- unit
partitioning, KV-sequence sharding, packing, all-gather and merge ordering -- with stand-in
compute (the oracle) in place of the CUDA kernels.  Failures are injected on the host only:
a rank that raises before the exchange makes its peer's collective time out with an error."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_b200 import dist as D
from oracle import api as OA
from oracle import golden as OG


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_unit_slices_partition_everything():
    for n in (1, 7, 128, 512, 131072):
        for world in (1, 2, 3, 4, 8):
            got = [D.unit_slice(n, world, r) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [b - a for a, b in got]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        D.unit_slice(4, 2, 2)


def _oracle_partial(scale, lo, total):
    def fn(q, k, v):
        outs, lses = [], []
        for i in range(q.shape[0]):
            s_q, s_k = q.shape[1], k.shape[1]
            # causal mask at global positions: key j_local visible iff j_local + lo <= i + total - s_q
            ii = torch.arange(s_q).view(-1, 1)
            jj = torch.arange(s_k).view(1, -1) + lo
            mask = jj > ii + (total - s_q)
            o, l = OG.blockwise_attention(q[i], k[i], v[i], scale, mask, q.dtype, round_p=False)
            dead = mask.all(dim=-1)
            o = o.float()
            o[dead] = 0
            l[:, dead] = float("-inf")
            outs.append(o)
            lses.append(l)
        return torch.stack(outs), torch.stack(lses)
    return fn


def _merge(o_all, lse_all, dtype):
    return OA.merge_partials(o_all, lse_all, out_dtype=dtype)


def _worker(rank, world, port, fail_rank, q, k, v, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        total = k.shape[1]
        lo, hi = D.kv_shard_range(total, world, rank)
        if rank == fail_rank:
            raise RuntimeError("injected host failure before the exchange")
        scale = q.shape[-1] ** -0.5
        out, lse = D.sharded_decode(q, k[:, lo:hi], v[:, lo:hi], kv_pos_offset=lo, kv_total=total,
                                    softmax_scale=scale, causal=True, local_partial=_oracle_partial(scale, lo, total),
                                    merge=_merge)
        ret[rank] = (out, lse)
    except Exception as e:  # noqa: BLE001
        ret[rank] = repr(e)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(world, fail_rank=-1):
    g = torch.Generator().manual_seed(world)
    q = torch.randn(2, 3, 4, 32, generator=g).to(torch.bfloat16)
    k = torch.randn(2, 101, 2, 32, generator=g).to(torch.bfloat16)
    v = torch.randn(2, 101, 2, 32, generator=g).to(torch.bfloat16)
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail_rank, q, k, v, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive()
    return q, k, v, dict(ret)


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_sharded_decode_over_gloo(world):
    q, k, v, ret = _run(world)
    gold_out, gold_lse = OA.flash_attn_with_kvcache(q, k, v, cache_seqlens=k.shape[1], causal=True, round_p=False)
    for r in range(world):
        assert not isinstance(ret[r], str), ret[r]
        out, lse = ret[r]
        torch.testing.assert_close(out.float(), gold_out.float(), rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(lse, gold_lse, rtol=1e-5, atol=1e-5)
        assert torch.equal(out, ret[0][0])  # replicated result


def test_rank_failing_on_the_host_surfaces_as_an_error_on_the_peer():
    _, _, _, ret = _run(2, fail_rank=1)
    assert "injected host failure" in ret[1]
    assert isinstance(ret[0], str)  # the surviving rank's all-gather ended with an error, it did not hang
