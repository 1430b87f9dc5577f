"""Drop-in for the reference's pybind extension module ``flash_attn_npu_arch22_v3``
(csrc/arch22/flash_attn_npu_v3/flash_api.cpp:816-822): ``fwd`` with the unified 34-argument
positional signature (:61-96) and ``get_scheduler_metadata`` (:493-517), plus ``fwd_combine``
which the reference's Python layer calls (flash_attn_npu_v3/interface_arch22.py:930-931) but its
native module never exported.  Backed by libfa_b200.so.
"""
from __future__ import annotations

import ctypes as C
import weakref

import torch

from flash_b200 import lib as L
from flash_b200 import ops



def _reject(cond, msg):
    if cond:
        raise RuntimeError(msg)


def fwd(q, k, v, k_new_, v_new_, q_v_, out_, cu_seqlens_q_, cu_seqlens_k_, cu_seqlens_k_new_, seqused_q_, seqused_k_,
        max_seqlen_q_, max_seqlen_k_, page_table_, kv_batch_idx_, leftpad_k_, rotary_cos_, rotary_sin_,
        seqlens_rotary_, q_descale_, k_descale_, v_descale_, softmax_scale_, is_causal, window_size_left,
        window_size_right, attention_chunk, softcap, is_rotary_interleaved, scheduler_metadata_, num_splits,
        pack_gqa_, sm_margin):
    """mha_fwd (unified), flash_api.cpp:60-491 -> [out, softmax_lse, out_accum, softmax_lse_accum].

    q is (b, s_q, h, d), or (total_q, h, d) with cu_seqlens_q_; k / v are dense, varlen
    (with cu_seqlens_k_), a contiguous cache or a paged cache (with page_table_); seqused_k_ gives
    the per-sequence key counts.  softmax_lse is (b, h, s_q) or (h, total_q).
    """
    # same rejections as the reference (:150-162)
    _reject(q_v_ is not None, "NPU FlashAttention does not support qv")
    _reject(leftpad_k_ is not None, "NPU FlashAttention does not support leftpad_k")
    _reject(seqused_q_ is not None, "NPU FlashAttention does not support seqused_q")
    _reject(cu_seqlens_k_new_ is not None, "NPU FlashAttention does not support cu_seqlens_k_new")
    _reject(seqlens_rotary_ is not None, "NPU FlashAttention does not support seqlens_rotary")
    _reject(q_descale_ is not None or k_descale_ is not None or v_descale_ is not None,
            "NPU FlashAttention does not support descale")
    _reject(attention_chunk != 0, "NPU FlashAttention does not support attention_chunk")
    if softmax_scale_ is None:
        softmax_scale_ = q.shape[-1] ** (-0.5)
    plan_bytes = _plan_bytes(scheduler_metadata_) if scheduler_metadata_ is not None else None
    if k.dim() == 3 and cu_seqlens_k_ is None and seqused_k_ is not None and page_table_ is None:
        # Packed (total_k, h_k, d) keys described by their per-sequence lengths alone: the reference's kernel takes
        # the prefix sums of seqused_k as the sequence starts (its tests feed flash_attn_with_kvcache this way,
        # tests/test_flash_attn_npu_v3.py:326-331,336-340).  The longest sequence is not known on the host, so the
        # total serves as its bound.
        _reject(k_new_ is not None, "appending new tokens needs a KV cache with one row per sequence")
        cu_seqlens_k_ = torch.nn.functional.pad(torch.cumsum(seqused_k_, 0, dtype=torch.int32), (1, 0))
        seqused_k_, max_seqlen_k_ = None, int(k.shape[0])
    out, lse = ops.attention_forward(
        q, k, v, out=out_, k_new=k_new_, v_new=v_new_, cu_seqlens_q=cu_seqlens_q_, cu_seqlens_k=cu_seqlens_k_,
        max_seqlen_q=max_seqlen_q_, max_seqlen_k=max_seqlen_k_, seqused_k=seqused_k_, cache_batch_idx=kv_batch_idx_,
        block_table=page_table_, rotary_cos=rotary_cos_, rotary_sin=rotary_sin_,
        rotary_interleaved=is_rotary_interleaved, softmax_scale=softmax_scale_, causal=is_causal,
        window_left=window_size_left, window_right=window_size_right, softcap=softcap, num_splits=num_splits,
        plan_bytes=plan_bytes)
    return [out, lse, None, None]


# Decoded copies of metadata tensors seen before.  Reading the bytes of a device tensor costs a device-to-host copy,
# which a decode loop that passes the same tensor object every step should pay once.  An entry belongs to one live
# tensor object at one version (the weak reference guards against a new tensor at a recycled address or id); a
# clone, a moved copy or a modified tensor simply misses here and is read again.
_decoded = {}


def _plan_bytes(meta: torch.Tensor) -> bytes:
    if meta.dtype != torch.uint8 or meta.dim() != 1 or meta.numel() < L.PLAN_BYTES:
        raise RuntimeError("scheduler_metadata must be the uint8 tensor returned by get_scheduler_metadata")
    hit = _decoded.get(id(meta))
    if hit is not None and hit[0]() is meta and hit[1] == meta._version:
        return hit[2]
    raw = bytes(meta[:L.PLAN_BYTES].cpu().numpy().tobytes())
    if len(_decoded) > 64:
        _decoded.clear()
    _decoded[id(meta)] = (weakref.ref(meta), meta._version, raw)
    return raw


def get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads_q, num_heads_kv, headdim, headdim_v,
                           qkv_dtype, cache_seqlens, cu_seqlens_q=None, cu_seqlens_k=None, cu_seqlens_k_new=None,
                           seqused_q=None, cache_leftpad=None, page_size=None, max_seqlen_k_new=0, causal=False,
                           window_size_left=-1, window_size_right=-1, attention_chunk=0, has_softcap=False,
                           num_splits=0, pack_gqa=None, sm_margin=0):
    """Plans a forward ahead of the call -- kernel family, tile configuration, KV splits, grid -- from the shapes
    alone, without touching the sequence lengths on the host.  Returns an opaque uint8 tensor on the device of
    cache_seqlens whose bytes ARE the plan (a header naming the problem, then the plan); pass it back as
    ``scheduler_metadata=``.  The forward checks the header against its own arguments: bytes made for other shapes,
    dtype or mask are refused.  (The reference computes its plan with an AICPU kernel and a host synchronisation,
    csrc/arch22/flash_attn_npu_v3/flash_api.cpp:43-56,493-558; this one is host arithmetic.)  Tensors are assumed
    contiguous and 16-byte aligned, as the torch allocator makes them; a call whose tensors are not is planned afresh."""
    _reject(cu_seqlens_k_new is not None or seqused_q is not None or cache_leftpad is not None,
            "NPU FlashAttention does not support cu_seqlens_k_new / seqused_q / cache_leftpad")
    _reject(attention_chunk != 0, "NPU FlashAttention does not support attention_chunk")
    _reject(headdim_v is not None and headdim_v != headdim, "head dims of q / k and v must be equal")
    p = L.FwdParams()
    stand_in = 256  # only NULL-ness and alignment of the pointers matter to the planner
    p.q = p.k = p.v = p.o = p.lse = stand_in
    b, s_q, s_k, h, h_k, d = int(batch_size), int(max_seqlen_q), int(max_seqlen_k), int(num_heads_q), int(num_heads_kv), int(headdim)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d = b, s_q, s_k, h, h_k, d
    p.q_head_stride = p.o_head_stride = d
    p.q_row_stride = p.o_row_stride = h * d
    if cu_seqlens_q is not None:
        p.cu_seqlens_q = stand_in
        p.total_q = b * s_q  # an upper bound: the plan only depends on it through the LSE layout
        p.lse_head_stride = p.total_q
    else:
        p.total_q = b * s_q
        p.q_batch_stride = p.o_batch_stride = s_q * h * d
        p.lse_batch_stride, p.lse_head_stride = h * s_q, s_q
    p.k_head_stride = p.v_head_stride = d
    p.k_row_stride = p.v_row_stride = h_k * d
    if cu_seqlens_k is not None:
        p.cu_seqlens_k, p.total_k = stand_in, b * s_k
    else:
        p.seqused_k = stand_in
        if page_size is not None:
            p.block_table, p.page_size = stand_in, int(page_size)
            pages = -(-s_k // int(page_size))
            p.seqlen_k = pages * int(page_size)
            p.block_table_batch_stride, p.kv_outer = pages, b * pages
            p.k_batch_stride = p.v_batch_stride = int(page_size) * h_k * d
        else:
            p.k_batch_stride = p.v_batch_stride = s_k * h_k * d
    if max_seqlen_k_new:
        p.k_new = p.v_new = stand_in
        p.seqlen_new = int(max_seqlen_k_new)
        p.knew_head_stride = p.vnew_head_stride = d
        p.knew_row_stride = p.vnew_row_stride = h_k * d
        p.knew_batch_stride = p.vnew_batch_stride = int(max_seqlen_k_new) * h_k * d
    p.dtype = L.FA_BF16 if qkv_dtype == torch.bfloat16 else L.FA_FP16
    p.causal, p.window_left, p.window_right = int(bool(causal)), int(window_size_left), int(window_size_right)
    p.max_seqlen_k_known = -1
    p.num_splits = int(num_splits)
    p.kernel = L.KERNEL_AUTO
    dev = cache_seqlens.device
    p.num_sm = ops._num_sm(dev) if dev.type == "cuda" else 148
    p.softmax_scale = float(d) ** -0.5
    p.softcap = 1.0 if has_softcap else 0.0
    raw = ops.encode_plan(p)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)


def fwd_combine(out_partial, lse_partial, out=None, out_dtype=None):
    """Merge of split partials: out_partial (n, b, s, h, d) fp32, lse_partial (n, b, s, h) fp32
    -> [out (b, s, h, d), softmax_lse (b, s, h)]."""
    o, lse = ops.combine(out_partial, lse_partial, out=out, out_dtype=out_dtype)
    return [o, lse]


def bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_seqlens_q_, cu_seqlens_k_, seqused_q_, seqused_k_,
        max_seqlen_q_, max_seqlen_k_, softmax_scale, is_causal, window_size_left, window_size_right, softcap,
        deterministic, sm_margin):
    """Backward of ``fwd`` for dense or packed-varlen q / k / v (argument order of the reference's pybind ``bwd``,
    flash_attn_npu_v3/interface_arch22.py:294-317).  Returns [dq, dk, dv, softmax_d]."""
    _reject(seqused_q_ is not None or seqused_k_ is not None, "the backward does not support seqused_q / seqused_k")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    dq, dk, dv = ops.attention_backward(dout, q, k, v, out, softmax_lse, dq=dq_, dk=dk_, dv=dv_,
                                        softmax_scale=softmax_scale, causal=is_causal, window_left=window_size_left,
                                        window_right=window_size_right, softcap=softcap, cu_seqlens_q=cu_seqlens_q_,
                                        cu_seqlens_k=cu_seqlens_k_, max_seqlen_q=max_seqlen_q_, max_seqlen_k=max_seqlen_k_)
    return [dq, dk, dv, torch.empty(0, dtype=torch.float32, device=q.device)]
