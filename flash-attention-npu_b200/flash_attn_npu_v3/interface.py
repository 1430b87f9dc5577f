"""Public FA3-style API of the reference's ``flash_attn_npu_v3`` package, on B200.

Same names, argument order, defaults and return conventions as
flash_attn_npu_v3/interface_arch22.py of the reference (:797-1138); every call funnels into the
single positional ``flash_attn_npu_arch22_v3.fwd`` exactly like the reference (:63-154).
Arguments the backend does not implement (qv, *_descale, attention_chunk, seqused_q,
cu_seqlens_k_new, rotary_seqlens, cache_leftpad) must keep their defaults, as in the reference
(csrc/arch22/flash_attn_npu_v3/flash_api.cpp:150-162).  ``flash_attn_func`` and
``flash_attn_varlen_func`` are differentiable (backward through ``flash_attn_npu_arch22_v3.bwd``).
"""
from __future__ import annotations

from typing import Optional, Union

import torch

import flash_attn_npu_arch22_v3 as _ext

from . import custom_ops as _ops  # registers the torch.library operators the calls below go through


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _forward(q, k, v, k_new=None, v_new=None, qv=None, out_=None, cu_seqlens_q=None, cu_seqlens_k=None,
             cu_seqlens_k_new=None, seqused_q=None, seqused_k=None, max_seqlen_q=None, max_seqlen_k=None,
             page_table=None, kv_batch_idx=None, leftpad_k=None, rotary_cos=None, rotary_sin=None,
             seqlens_rotary=None, q_descale=None, k_descale=None, v_descale=None, softmax_scale=None, causal=False,
             window_size_left=-1, window_size_right=-1, attention_chunk=0, softcap=0.0, rotary_interleaved=True,
             scheduler_metadata=None, num_splits=1, pack_gqa=None, sm_margin=0):
    q, k, v, k_new, v_new = [maybe_contiguous(x) for x in (q, k, v, k_new, v_new)]
    cu_seqlens_q, cu_seqlens_k, seqused_k, page_table, kv_batch_idx = [
        maybe_contiguous(x) for x in (cu_seqlens_q, cu_seqlens_k, seqused_k, page_table, kv_batch_idx)]
    d = q.shape[-1]
    if d % 8 != 0:  # pad the head dim like the v2 front end does; sliced back below
        pad = 8 - d % 8
        q, k, v = [torch.nn.functional.pad(t, [0, pad]) for t in (q, k, v)]
    args = (q, k, v, k_new, v_new, qv, out_, cu_seqlens_q, cu_seqlens_k, cu_seqlens_k_new, seqused_q, seqused_k,
            max_seqlen_q, max_seqlen_k, page_table, kv_batch_idx, leftpad_k, rotary_cos, rotary_sin, seqlens_rotary,
            q_descale, k_descale, v_descale, softmax_scale, causal, window_size_left, window_size_right,
            attention_chunk, softcap, rotary_interleaved, scheduler_metadata, num_splits, pack_gqa, sm_margin)
    unsupported = (qv, cu_seqlens_k_new, seqused_q, leftpad_k, seqlens_rotary, q_descale, k_descale, v_descale)
    if out_ is not None or any(x is not None for x in unsupported) or attention_chunk != 0:
        # a caller-provided output cannot be an operator result (it would alias an input), and the arguments this
        # backend rejects are rejected by the extension with the reference's messages
        out, lse, out_accum, lse_accum = _ops._call(*args)
    elif k_new is not None:  # new tokens are written into the cache: the operator that says so
        out, lse, out_accum, lse_accum = _ops._flash_attn_forward_inplace(
            q, k, v, k_new, v_new, cu_seqlens_q, seqused_k, max_seqlen_q, page_table, kv_batch_idx, rotary_cos,
            rotary_sin, softmax_scale, causal, window_size_left, window_size_right, softcap, rotary_interleaved,
            scheduler_metadata, num_splits, pack_gqa, sm_margin)
    else:
        out, lse, out_accum, lse_accum = _ops._flash_attn_forward(*args)
    return out[..., :d], lse, out_accum, lse_accum


class _AttnFunc(torch.autograd.Function):
    """Dense / packed-varlen attention with a backward (the reference's FlashAttnFunc / FlashAttnVarlenFunc of v3)."""

    @staticmethod
    def forward(ctx, q, k, v, kw):
        out, lse, _, _ = _forward(q, k, v, **kw)
        if any(t.requires_grad for t in (q, k, v)):
            d = q.shape[-1]
            pad = (8 - d % 8) % 8
            qp, kp, vp = [maybe_contiguous(t) if pad == 0 else torch.nn.functional.pad(maybe_contiguous(t), [0, pad])
                          for t in (q, k, v)]
            op = out if pad == 0 else torch.nn.functional.pad(out, [0, pad])
            ctx.save_for_backward(qp, kp, vp, op, lse, kw.get("cu_seqlens_q"), kw.get("cu_seqlens_k"))
            ctx.kw, ctx.d = kw, d
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, *unused):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        kw, d = ctx.kw, ctx.d
        dout = maybe_contiguous(dout)
        if q.shape[-1] != d:
            dout = torch.nn.functional.pad(dout, [0, q.shape[-1] - d])
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _ops._flash_attn_backward(dout, q, k, v, out.contiguous(), lse, cu_q, cu_k, kw.get("seqused_q"),
                                  kw.get("seqused_k"), kw.get("max_seqlen_q"), kw.get("max_seqlen_k"), dq, dk, dv,
                                  kw.get("softmax_scale"), kw.get("causal", False), kw.get("window_size_left", -1),
                                  kw.get("window_size_right", -1), kw.get("softcap", 0.0), False, kw.get("sm_margin", 0))
        return dq[..., :d], dk[..., :d], dv[..., :d], None


def _default_scale(q, qv):
    return (q.shape[-1] + (qv.shape[-1] if qv is not None else 0)) ** (-0.5)


def flash_attn_func(q, k, v, softmax_scale=None, causal=False, qv=None, q_descale=None, k_descale=None,
                    v_descale=None, window_size=(-1, -1), attention_chunk=0, softcap=0.0, num_splits=1, pack_gqa=None,
                    deterministic=False, sm_margin=0, return_attn_probs=False, scheduler_metadata=None):
    """q (b, s_q, h, d), k / v (b, s_k, h_k, d) -> out, or (out, softmax_lse (b, h, s_q))."""
    if softmax_scale is None:
        softmax_scale = _default_scale(q, qv)
    out, lse = _AttnFunc.apply(q, k, v, dict(
        qv=qv, q_descale=q_descale, k_descale=k_descale, v_descale=v_descale, softmax_scale=softmax_scale, causal=causal,
        window_size_left=window_size[0], window_size_right=window_size[1], attention_chunk=attention_chunk,
        softcap=softcap, scheduler_metadata=scheduler_metadata, num_splits=num_splits, pack_gqa=pack_gqa,
        sm_margin=sm_margin))
    return (out, lse) if return_attn_probs else out


def flash_attn_qkvpacked_func(qkv, softmax_scale=None, causal=False, q_descale=None, k_descale=None, v_descale=None,
                              window_size=(-1, -1), attention_chunk=0, softcap=0.0, deterministic=False,
                              num_heads_q=None, sm_margin=0, return_attn_probs=False):
    """qkv (b, s, 3, h, d), or (b, s, h_q + 2 h_k, d) with num_heads_q."""
    if qkv.dim() == 5:
        q, k, v = qkv.unbind(dim=-3)
    else:
        h_k = (qkv.shape[2] - num_heads_q) // 2
        q, k, v = qkv.split([num_heads_q, h_k, h_k], dim=-2)
    return flash_attn_func(q, k, v, softmax_scale, causal, None, q_descale, k_descale, v_descale, window_size,
                           attention_chunk, softcap, 1, None, deterministic, sm_margin, return_attn_probs)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, seqused_q=None,
                           seqused_k=None, softmax_scale=None, causal=False, qv=None, q_descale=None, k_descale=None,
                           v_descale=None, window_size=(-1, -1), attention_chunk=0, softcap=0.0, num_splits=1,
                           pack_gqa=None, deterministic=False, sm_margin=0, return_attn_probs=False,
                           scheduler_metadata=None):
    """q (total_q, h, d), k / v (total_k, h_k, d) -> out, or (out, softmax_lse (h, total_q))."""
    if softmax_scale is None:
        softmax_scale = _default_scale(q, qv)
    out, lse = _AttnFunc.apply(q, k, v, dict(
        qv=qv, cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k, seqused_q=seqused_q, seqused_k=seqused_k,
        max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k, q_descale=q_descale, k_descale=k_descale,
        v_descale=v_descale, softmax_scale=softmax_scale, causal=causal, window_size_left=window_size[0],
        window_size_right=window_size[1], attention_chunk=attention_chunk, softcap=softcap,
        scheduler_metadata=scheduler_metadata, num_splits=num_splits, pack_gqa=pack_gqa, sm_margin=sm_margin))
    return (out, lse) if return_attn_probs else out


def flash_attn_combine(out_partial, lse_partial, out=None, out_dtype=None):
    """out_partial (n, b, s, h, d) fp32, lse_partial (n, b, s, h) fp32 -> (out, softmax_lse (b, s, h))."""
    o, lse = _ext.fwd_combine(out_partial, lse_partial, out, out_dtype)
    return o, lse


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, qv=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
                            cache_batch_idx: Optional[torch.Tensor] = None,
                            cache_leftpad: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
                            cu_seqlens_q: Optional[torch.Tensor] = None,
                            cu_seqlens_k_new: Optional[torch.Tensor] = None, max_seqlen_q: Optional[int] = None,
                            rotary_seqlens: Optional[torch.Tensor] = None, q_descale=None, k_descale=None,
                            v_descale=None, softmax_scale=None, causal=False, window_size=(-1, -1), attention_chunk=0,
                            softcap=0.0, rotary_interleaved=True, scheduler_metadata=None, num_splits=0, pack_gqa=None,
                            sm_margin=0, return_softmax_lse=False):
    """KV-cache attention; q is (b, s_q, h, d) or (total_q, h, d) with cu_seqlens_q + max_seqlen_q.
    Returns out, or (out, softmax_lse, out_accum, softmax_lse_accum) when return_softmax_lse
    (the last two are empty tensors, as in the reference :1095)."""
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    if softmax_scale is None:
        softmax_scale = _default_scale(q, qv)
    if cache_seqlens is not None and isinstance(cache_seqlens, int):
        cache_seqlens = torch.full((q.shape[0],), cache_seqlens, dtype=torch.int32, device=k_cache.device)
    out, lse, *rest = _forward(q, k_cache, v_cache, k, v, qv, None, cu_seqlens_q, None, cu_seqlens_k_new, None,
                               cache_seqlens, max_seqlen_q, None, page_table, cache_batch_idx, cache_leftpad,
                               rotary_cos, rotary_sin, rotary_seqlens, q_descale, k_descale, v_descale, softmax_scale,
                               causal=causal, window_size_left=window_size[0], window_size_right=window_size[1],
                               attention_chunk=attention_chunk, softcap=softcap,
                               rotary_interleaved=rotary_interleaved, scheduler_metadata=scheduler_metadata,
                               num_splits=num_splits, pack_gqa=pack_gqa, sm_margin=sm_margin)
    return (out, lse, *rest) if return_softmax_lse else out


def get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads_q, num_heads_kv, headdim,
                           cache_seqlens: torch.Tensor, qkv_dtype=torch.bfloat16, headdim_v=None,
                           cu_seqlens_q: Optional[torch.Tensor] = None, cu_seqlens_k_new: Optional[torch.Tensor] = None,
                           cache_leftpad: Optional[torch.Tensor] = None, page_size: Optional[int] = None,
                           max_seqlen_k_new=0, causal=False, window_size=(-1, -1), attention_chunk=0,
                           has_softcap=False, num_splits=0, pack_gqa=None, sm_margin=0):
    """Opaque plan tensor for ``scheduler_metadata=`` (tile configuration + KV splits)."""
    cache_seqlens = maybe_contiguous(cache_seqlens)
    if headdim_v is None:
        headdim_v = headdim
    return _ext.get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads_q, num_heads_kv, headdim,
                                       headdim_v, qkv_dtype, cache_seqlens, cu_seqlens_q, None, cu_seqlens_k_new,
                                       None, cache_leftpad, page_size, max_seqlen_k_new, causal, window_size[0],
                                       window_size[1], attention_chunk, has_softcap, num_splits, pack_gqa, sm_margin)
