"""Public FA2-style API of the reference's ``flash_attn_npu_v2`` package, on B200.

Same function names, argument order, defaults and return conventions as
flash_attn_npu_v2/interface_arch22.py of the reference (:965-1573); the native calls go to
``flash_attn_npu_arch22_v2`` (here a ctypes-backed module over libfa_b200.so) positionally,
exactly as the reference calls its pybind extension (:61-75, :1551-1572); the dense and varlen forward and
backward go through ``torch.library`` operators of the reference's names (``custom_ops.py``).

``flash_attn_func`` and ``flash_attn_varlen_func`` (and their packed variants) are differentiable:
autograd Functions with the structure of the reference's (:774-824, :827-900), whose backward
calls ``bwd`` / ``varlen_bwd`` of the extension.  The KV-cache entry point is inference only.
"""
from __future__ import annotations

from typing import Optional, Union

import torch
import torch.nn.functional as F

import flash_attn_npu_arch22_v2 as _ext

from . import custom_ops as _ops  # registers the torch.library operators the calls below go through


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _pad_head(ts, d):
    """The reference pads the head dim to a multiple of 8 and slices the output back (:796-800,823)."""
    if d % 8 == 0:
        return ts
    return [F.pad(t, [0, 8 - d % 8]) for t in ts]


def _check_dropout(dropout_p):
    if dropout_p != 0.0:
        raise RuntimeError("NPU FlashAttention does not support dropout")


class FlashAttnFunc(torch.autograd.Function):
    """Dense attention with a backward (structure of the reference's FlashAttnFunc, :774-900)."""

    @staticmethod
    def forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
                return_softmax):
        d = q.size(3)
        qp, kp, vp = _pad_head([maybe_contiguous(x) for x in (q, k, v)], d)
        out_padded, lse, s_dmask, _ = _ops._flash_attn_forward(qp, kp, vp, dropout_p, softmax_scale, causal,
                                                               window_size[0], window_size[1], softcap, alibi_slopes,
                                                               False)
        if any(t.requires_grad for t in (q, k, v)):
            ctx.save_for_backward(qp, kp, vp, out_padded, lse)
            ctx.args = (dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic, d)
        out = out_padded[..., :d]
        ctx.mark_non_differentiable(lse, s_dmask)
        return out, lse, s_dmask

    @staticmethod
    def backward(ctx, dout, *unused):
        q, k, v, out, lse = ctx.saved_tensors
        dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic, d = ctx.args
        dout_padded = _pad_head([maybe_contiguous(dout)], d)[0]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _ops._flash_attn_backward(dout_padded, q, k, v, out, lse, dq, dk, dv, dropout_p, softmax_scale, causal,
                                  window_size[0], window_size[1], softcap, alibi_slopes, deterministic, None)
        return dq[..., :d], dk[..., :d], dv[..., :d], None, None, None, None, None, None, None, None


class FlashAttnVarlenFunc(torch.autograd.Function):
    """Packed varlen attention with a backward (the reference's FlashAttnVarlenFunc)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal,
                window_size, softcap, alibi_slopes, deterministic, block_table):
        d = q.size(2)
        qp, kp, vp = _pad_head([maybe_contiguous(x) for x in (q, k, v)], d)
        out_padded, lse, s_dmask, _ = _ops._flash_attn_varlen_forward(
            qp, kp, vp, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal,
            window_size[0], window_size[1], softcap, alibi_slopes, False, block_table, None, None, False)
        if any(t.requires_grad for t in (q, k, v)):
            ctx.save_for_backward(qp, kp, vp, out_padded, lse, cu_seqlens_q, cu_seqlens_k)
            ctx.args = (max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal, window_size, softcap,
                        alibi_slopes, deterministic, d)
        out = out_padded[..., :d]
        ctx.mark_non_differentiable(lse, s_dmask)
        return out, lse, s_dmask

    @staticmethod
    def backward(ctx, dout, *unused):
        q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k = ctx.saved_tensors
        (max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
         d) = ctx.args
        dout_padded = _pad_head([maybe_contiguous(dout)], d)[0]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _ops._flash_attn_varlen_backward(dout_padded, q, k, v, out, lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                                         max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal, window_size[0],
                                         window_size[1], softcap, alibi_slopes, deterministic, None, False)
        return (dq[..., :d], dk[..., :d], dv[..., :d]) + (None,) * 12


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """q (b, s_q, h, d), k / v (b, s_k, h_k, d) -> out (b, s_q, h, d)
    or (out, softmax_lse (b, h, s_q) fp32, S_dmask (empty)) when return_attn_probs.  Differentiable in q, k, v."""
    _check_dropout(dropout_p)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    out, lse, s_dmask = FlashAttnFunc.apply(q, k, v, dropout_p, softmax_scale, causal, tuple(window_size), softcap,
                                            alibi_slopes, deterministic, return_attn_probs)
    return (out, lse, s_dmask) if return_attn_probs else out


def flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                             softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """kv (b, s_k, 2, h_k, d)."""
    return flash_attn_func(q, kv[:, :, 0], kv[:, :, 1], dropout_p, softmax_scale, causal, window_size, softcap,
                           alibi_slopes, deterministic, return_attn_probs)


def flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                              softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """qkv (b, s, 3, h, d)."""
    return flash_attn_func(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], dropout_p, softmax_scale, causal, window_size,
                           softcap, alibi_slopes, deterministic, return_attn_probs)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                           softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
                           deterministic=False, return_attn_probs=False, block_table=None):
    """q (total_q, h, d), k / v (total_k, h_k, d) -> out (total_q, h, d)
    or (out, softmax_lse (h, total_q) fp32, S_dmask (empty))."""
    _check_dropout(dropout_p)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    out, lse, s_dmask = FlashAttnVarlenFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                                  dropout_p, softmax_scale, causal, tuple(window_size), softcap,
                                                  alibi_slopes, deterministic, block_table)
    return (out, lse, s_dmask) if return_attn_probs else out


def flash_attn_varlen_kvpacked_func(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                                    softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                                    alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """kv (total_k, 2, h_k, d)."""
    return flash_attn_varlen_func(q, kv[:, 0], kv[:, 1], cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                  dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                                  deterministic, return_attn_probs)


def flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_seqlen, dropout_p=0.0, softmax_scale=None, causal=False,
                                     window_size=(-1, -1), softcap=0.0, alibi_slopes=None, deterministic=False,
                                     return_attn_probs=False):
    """qkv (total, 3, h, d)."""
    return flash_attn_varlen_func(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                  dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                                  deterministic, return_attn_probs)


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
                            cache_batch_idx: Optional[torch.Tensor] = None,
                            cache_leftpad: Optional[torch.Tensor] = None,
                            block_table: Optional[torch.Tensor] = None, softmax_scale=None, causal=False,
                            window_size=(-1, -1), softcap=0.0, rotary_interleaved=True, alibi_slopes=None,
                            num_splits=0, return_softmax_lse=False):
    """Attention over a KV cache (contiguous (b_c, s_cache, h_k, d) or paged
    (n_blocks, page, h_k, d) + block_table), optionally appending k / v IN PLACE at
    cache_seqlens (rotary applied to k and q first when rotary_cos / rotary_sin are given).

    Returns out (b, s_q, h, d), or (out, softmax_lse (b, h, s_q)) when return_softmax_lse.
    Semantics follow the reference docstring (interface_arch22.py:1452-1537): bottom-right
    aligned causal mask, window [i + s_k - s_q - left, i + s_k - s_q + right], rows without a
    visible key give 0.  cache_seqlens is not updated by the call.
    """
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if cache_seqlens is not None and isinstance(cache_seqlens, int):
        cache_seqlens = torch.full((q.shape[0],), cache_seqlens, dtype=torch.int32, device=k_cache.device)
    cache_seqlens = maybe_contiguous(cache_seqlens)
    cache_batch_idx = maybe_contiguous(cache_batch_idx)
    block_table = maybe_contiguous(block_table)
    out, softmax_lse = _ext.fwd_kvcache(q, k_cache, v_cache, k, v, cache_seqlens, rotary_cos, rotary_sin,
                                        cache_batch_idx, cache_leftpad, block_table, alibi_slopes, None,
                                        softmax_scale, causal, window_size[0], window_size[1], softcap,
                                        rotary_interleaved, num_splits)
    return (out, softmax_lse) if return_softmax_lse else out
