"""Drop-in for the reference's pybind extension module ``flash_attn_npu_arch22_v3``
(csrc/arch22/flash_attn_npu_v3/flash_api.cpp:816-822): ``fwd`` with the unified 34-argument
positional signature (:61-96) and ``get_scheduler_metadata`` (:493-517), plus ``fwd_combine``
which the reference's Python layer calls (flash_attn_npu_v3/interface_arch22.py:930-931) but its
native module never exported.  Backed by libfa_b200.so.
"""
from __future__ import annotations

import ctypes as C

import torch

from flash_b200 import lib as L
from flash_b200 import ops

_PLAN_MAGIC = 0x0FA5B200


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
    if scheduler_metadata_ is not None:
        meta = getattr(scheduler_metadata_, "_fa_b200_plan", None)
        if meta is not None and num_splits == 0:
            num_splits = meta["num_splits"]
    out, lse = ops.attention_forward(
        q, k, v, out=out_, k_new=k_new_, v_new=v_new_, cu_seqlens_q=cu_seqlens_q_, cu_seqlens_k=cu_seqlens_k_,
        max_seqlen_q=max_seqlen_q_, max_seqlen_k=max_seqlen_k_, seqused_k=seqused_k_, cache_batch_idx=kv_batch_idx_,
        block_table=page_table_, rotary_cos=rotary_cos_, rotary_sin=rotary_sin_,
        rotary_interleaved=is_rotary_interleaved, softmax_scale=softmax_scale_, causal=is_causal,
        window_left=window_size_left, window_right=window_size_right, softcap=softcap, num_splits=num_splits)
    return [out, lse, None, None]


def get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads_q, num_heads_kv, headdim, headdim_v,
                           qkv_dtype, cache_seqlens, cu_seqlens_q=None, cu_seqlens_k=None, cu_seqlens_k_new=None,
                           seqused_q=None, cache_leftpad=None, page_size=None, max_seqlen_k_new=0, causal=False,
                           window_size_left=-1, window_size_right=-1, attention_chunk=0, has_softcap=False,
                           num_splits=0, pack_gqa=None, sm_margin=0):
    """Pre-plans a KV-cache forward (tile configuration and KV splits) without touching the
    sequence lengths on the host.  Returns an opaque uint8 tensor on the device of cache_seqlens;
    pass it back as ``scheduler_metadata=``.  (The reference computes its plan with an AICPU kernel
    and a host synchronisation, flash_api.cpp:43-56; this one is pure host arithmetic.)"""
    lib = L.load()
    p = L.FwdParams()
    dummy = 256  # plan only checks pointers for NULL-ness
    p.q = p.k = p.v = p.o = p.lse = dummy
    p.seqused_k = dummy
    p.b, p.seqlen_q, p.seqlen_k = batch_size, max_seqlen_q, max_seqlen_k
    p.h, p.h_k, p.d = num_heads_q, num_heads_kv, headdim
    p.total_q = batch_size * max_seqlen_q
    if cu_seqlens_q is not None:
        p.cu_seqlens_q = dummy
        p.total_q = batch_size * max_seqlen_q
        p.lse_head_stride = p.total_q
    else:
        p.lse_batch_stride, p.lse_head_stride = num_heads_q * max_seqlen_q, max_seqlen_q
    if page_size is not None:
        p.block_table, p.page_size, p.kv_outer = dummy, int(page_size), 1
    if max_seqlen_k_new:
        p.k_new = p.v_new = dummy
        p.seqlen_new = int(max_seqlen_k_new)
    p.dtype = L.FA_BF16 if qkv_dtype == torch.bfloat16 else L.FA_FP16
    p.causal, p.window_left, p.window_right = int(bool(causal)), window_size_left, window_size_right
    p.max_seqlen_k_known = -1
    p.num_splits = num_splits
    p.kernel = L.KERNEL_MMA
    dev = cache_seqlens.device
    p.num_sm = ops._num_sm(dev) if dev.type == "cuda" else 148
    p.softmax_scale = 1.0
    p.softcap = 1.0 if has_softcap else 0.0
    plan = L.FwdPlan()
    L.check(lib.fa_b200_fwd_plan(C.byref(p), C.byref(plan)))
    words = [_PLAN_MAGIC, plan.kernel, plan.config, plan.pack_gqa, plan.block_m, plan.block_n, plan.m_blocks,
             plan.num_splits, plan.blocks_per_split, plan.grid]
    meta = torch.tensor(words, dtype=torch.int32).view(torch.uint8).to(dev, non_blocking=True)
    meta._fa_b200_plan = {"num_splits": plan.num_splits, "blocks_per_split": plan.blocks_per_split,
                          "config": plan.config, "grid": plan.grid}
    return meta


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
