"""Multi-GPU helpers: one process per GPU, torch.distributed (NCCL) for the plumbing.

The reference has no distributed code at all; these helpers implement the two partitionings
the benchmark configurations ask for:

* independent shards (prefill, contiguous / paged decode): (batch x kv-head) units are split into
  contiguous slices, one per rank, with no communication -- ``unit_slice``.
* sequence-sharded long-context decode: rank r holds keys [r*L/n, (r+1)*L/n) of every sequence.
  Each rank runs the split-KV decode kernel on its shard producing a normalised fp32 partial
  (O, LSE); one all-gather of the packed [O | LSE] buffer moves n * rows * (d + 1) * 4 bytes, and
  the merge kernel (the same arithmetic as the reference's in-kernel split merge,
  csrc/arch22/flash_attn_npu_v2/CombineScale.hpp:165-309) finishes on every rank --
  ``sharded_decode``.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def unit_slice(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, stop) of n_units for this rank; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank / world size")
    base, rem = divmod(n_units, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def kv_shard_range(seqlen_k: int, world: int, rank: int) -> Tuple[int, int]:
    """Token range of the KV sequence held by this rank (even split, remainder to the low ranks)."""
    return unit_slice(seqlen_k, world, rank)


def pack_partial(o_partial: torch.Tensor, lse_partial: torch.Tensor) -> torch.Tensor:
    """(b, s, h, d) fp32 + (b, h, s) fp32 -> one flat fp32 buffer [O | LSE] (a single message)."""
    return torch.cat([o_partial.reshape(-1), lse_partial.reshape(-1)])


def unpack_gathered(buf: torch.Tensor, world: int, o_shape, lse_shape):
    """(world * (numel(O) + numel(LSE))) -> o (n, b, s, h, d), lse (n, b, s, h) as strided views."""
    n_o = 1
    for x in o_shape:
        n_o *= x
    n_l = 1
    for x in lse_shape:
        n_l *= x
    per = n_o + n_l
    buf = buf.view(world, per)
    o = buf[:, :n_o].unflatten(1, o_shape)                       # (n, b, s, h, d)
    lse = buf[:, n_o:].unflatten(1, lse_shape).permute(0, 1, 3, 2)  # (n, b, h, s) -> (n, b, s, h)
    return o, lse


class PeerExchange:
    """Exchange buffers for ``sharded_decode(..., exchange=...)``: every rank allocates one buffer, hands its CUDA
    IPC handle to the others through the process group (a host-side all-gather of 64-byte handles) and maps theirs,
    so that the kernels can store a rank's partial straight into every peer's memory over NVLink and merge without
    a collective call.  One process per GPU; every rank must construct it and must make the same sequence of calls
    with it.  ``rows`` = batch x seqlen_q x heads of the largest problem it will serve, ``head_dim`` likewise.
    ``timeout_s``: how long the merge waits for the slowest rank before it gives up (flash_b200 reports that through
    fa_b200_check_status; nothing hangs)."""

    def __init__(self, rows: int, head_dim: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 timeout_s: float = 2.0):
        import ctypes as C

        from . import lib as L
        self._L, self._C = L, C
        lib = L.load()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > L.MAX_RANKS:
            raise RuntimeError(f"at most {L.MAX_RANKS} ranks")
        self.device = torch.device(device)
        self.nbytes = lib.fa_b200_exchange_bytes(self.world, rows, head_dim)
        self._own = C.c_void_p()
        handle = C.create_string_buffer(64)
        with torch.cuda.device(self.device):
            L.check(lib.fa_b200_exchange_alloc(self.nbytes, C.byref(self._own), handle))
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, handle.raw, group=group)
            else:
                handles[0] = handle.raw
            self._mapped = []
            self.x = L.Exchange()
            for r in range(self.world):
                if r == self.rank:
                    self.x.bufs[r] = self._own.value
                    continue
                ptr = C.c_void_p()
                L.check(lib.fa_b200_exchange_open(C.create_string_buffer(handles[r], 64), C.byref(ptr)))
                self._mapped.append(ptr)
                self.x.bufs[r] = ptr.value
        self.x.buf_bytes, self.x.world, self.x.rank = self.nbytes, self.world, self.rank
        self.x.timeout_cycles = int(timeout_s * 2.0e9)  # SM clock cycles, at about 2 GHz
        if self.world > 1:
            dist.barrier(group=group)  # nobody stores into a buffer that its owner has not finished setting up

    def close(self):
        """Unmaps the peers' buffers and frees this rank's.  Call it on every rank after the last exchange has
        completed on every rank (e.g. after a barrier)."""
        lib = self._L.load()
        with torch.cuda.device(self.device):
            for ptr in self._mapped:
                lib.fa_b200_exchange_close(ptr)
            self._mapped = []
            if self._own:
                lib.fa_b200_exchange_free(self._own)
                self._own = self._C.c_void_p()


def sharded_decode(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, *, kv_pos_offset: int,
                   kv_total: int, softmax_scale: Optional[float] = None, causal: bool = False,
                   group: Optional[dist.ProcessGroup] = None, out_dtype: Optional[torch.dtype] = None,
                   local_partial: Optional[Callable] = None, merge: Optional[Callable] = None,
                   exchange: Optional[PeerExchange] = None):
    """Sequence-sharded decode.  q (b, s_q, h, d) replicated; k_shard / v_shard
    (b, L_local, h_k, d) = this rank's slice [kv_pos_offset, kv_pos_offset + L_local) of a
    kv_total-long cache.  Returns (out (b, s_q, h, d), lse (b, h, s_q)) replicated on every rank.

    ``local_partial`` / ``merge`` exist so that the host-side plumbing can be exercised on CPU
    ranks (gloo) with stand-in compute; they default to the CUDA kernels.  ``exchange``: a ``PeerExchange`` built
    by every rank; the partials then travel by peer stores over NVLink instead of an all-gather (same results).
    """
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if exchange is not None:
        # peer-memory path: the local merge stores this rank's partial into every rank's exchange buffer, the final
        # merge waits for all of them -- three launches and no collective call
        from . import ops
        return ops.attention_forward_exchange(q, k_shard, v_shard, exchange.x, softmax_scale=softmax_scale, causal=causal,
                                              kv_pos_offset=kv_pos_offset, kv_total=kv_total)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    out_dtype = out_dtype or q.dtype
    if local_partial is None and merge is None:
        # CUDA path: the kernel writes its partial straight into the message buffer [O | LSE] and the
        # merge writes LSE in its final (b, h, s) layout -- no packing or transposing kernels.
        from . import ops
        b, s, h, d = q.shape
        n_o, n_l = b * s * h * d, b * h * s
        send = torch.empty(n_o + n_l, dtype=torch.float32, device=q.device)
        ops.attention_forward(q, k_shard, v_shard, out=send[:n_o].view(b, s, h, d), lse=send[n_o:].view(b, h, s),
                              softmax_scale=softmax_scale, causal=causal, kv_pos_offset=kv_pos_offset,
                              kv_total=kv_total, partial_out=True)
        if world > 1:
            recv = torch.empty(world * send.numel(), dtype=torch.float32, device=send.device)
            dist.all_gather_into_tensor(recv, send, group=group)
        else:
            recv = send
        o_all, lse_all = unpack_gathered(recv, world, (b, s, h, d), (b, h, s))
        lse = torch.empty((b, h, s), dtype=torch.float32, device=q.device)
        out, _ = ops.combine(o_all, lse_all, out_dtype=out_dtype, lse_out=lse.permute(0, 2, 1))
        return out, lse
    if local_partial is None:
        from . import ops

        def local_partial(q_, k_, v_):
            return ops.attention_forward(q_, k_, v_, softmax_scale=softmax_scale, causal=causal,
                                         kv_pos_offset=kv_pos_offset, kv_total=kv_total, partial_out=True)
    if merge is None:
        from . import ops

        def merge(o_all, lse_all, dtype):
            return ops.combine(o_all, lse_all, out_dtype=dtype)
    o_part, lse_part = local_partial(q, k_shard, v_shard)   # (b, s, h, d) fp32, (b, h, s) fp32
    if o_part.dtype != torch.float32 or lse_part.dtype != torch.float32:
        raise RuntimeError("local partials must be fp32")
    send = pack_partial(o_part, lse_part)
    if world > 1:
        recv = torch.empty(world * send.numel(), dtype=torch.float32, device=send.device)
        dist.all_gather_into_tensor(recv, send, group=group)
    else:
        recv = send
    o_all, lse_all = unpack_gathered(recv, world, tuple(o_part.shape), tuple(lse_part.shape))
    out, lse_bsh = merge(o_all, lse_all, out_dtype)
    return out, lse_bsh.permute(0, 2, 1).contiguous()
