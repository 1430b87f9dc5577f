"""Drop-in for the reference's pybind extension module ``flash_attn_npu_arch22_v2``
(csrc/arch22/flash_attn_npu_v2/flash_api.cpp:1301-1309): same function names, same
positional argument order, same return lists -- backed by libfa_b200.so.

Differences from the reference's native layer, all additions: rotary_cos/sin, the in-place
append of k / v, cache_batch_idx and alibi_slopes are implemented (the reference rejects or
ignores them, flash_api.cpp:415-436); num_splits > 1 is honoured.  cache_leftpad, dropout and
return_softmax stay rejected exactly as in the reference (:416, :653-656).
"""
from __future__ import annotations

import torch

from flash_b200 import ops


def _empty_like_nothing(ref):
    return torch.empty((0,), dtype=ref.dtype, device=ref.device)


def fwd(q, k, v, out_, alibi_slopes_, p_dropout, softmax_scale, is_causal, window_size_left, window_size_right,
        softcap, return_softmax, gen_):
    """mha_fwd, flash_api.cpp:628-826 -> [out, softmax_lse (b, h, s_q), p (empty), rng_state (empty)]."""
    if p_dropout != 0.0:
        raise RuntimeError("NPU FlashAttention does not support dropout")
    if return_softmax:
        raise RuntimeError("NPU FlashAttention does not support return_softmax")
    out, lse = ops.attention_forward(
        q, k, v, out=out_, alibi_slopes=alibi_slopes_, softmax_scale=softmax_scale, causal=is_causal,
        window_left=window_size_left, window_right=window_size_right, softcap=softcap)
    return [out, lse, _empty_like_nothing(q), torch.empty((2,), dtype=torch.int64, device=q.device)]


def varlen_fwd(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k_, leftpad_k_, block_table_, alibi_slopes_,
               max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left,
               window_size_right, softcap, return_softmax, gen_):
    """mha_varlen_fwd, flash_api.cpp:828-1060 -> [out, softmax_lse (h, total_q), p, rng_state]."""
    if p_dropout != 0.0:
        raise RuntimeError("NPU FlashAttention does not support dropout")
    if return_softmax:
        raise RuntimeError("NPU FlashAttention does not support return_softmax")
    if leftpad_k_ is not None:
        raise RuntimeError("NPU FlashAttention does not support leftpad_k")
    if block_table_ is not None:
        raise RuntimeError("NPU FlashAttention varlen_fwd does not support block_table")
    if seqused_k_ is not None:
        raise RuntimeError("NPU FlashAttention varlen_fwd does not support seqused_k")
    out, lse = ops.attention_forward(
        q, k, v, out=out_, cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k, max_seqlen_q=max_seqlen_q,
        max_seqlen_k=max_seqlen_k, alibi_slopes=alibi_slopes_, softmax_scale=softmax_scale, causal=is_causal,
        window_left=window_size_left, window_right=window_size_right, softcap=softcap)
    return [out, lse, _empty_like_nothing(q), torch.empty((2,), dtype=torch.int64, device=q.device)]


def fwd_kvcache(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_, cache_batch_idx_, leftpad_k_,
                block_table_, alibi_slopes_, out_, softmax_scale, is_causal, window_size_left, window_size_right,
                softcap, is_rotary_interleaved, num_splits):
    """mha_fwd_kvcache, flash_api.cpp:356-626 -> [out, softmax_lse (b, h, s_q)].

    kcache / vcache are updated in place at rows [seqlens_k[b], seqlens_k[b] + s_new) when k_, v_
    are given (rotary applied to k_ and q first when rotary_cos_/sin_ are given).
    """
    if leftpad_k_ is not None:
        raise RuntimeError("NPU FlashAttention does not support leftpad_k")
    if (rotary_cos_ is None) != (rotary_sin_ is None):
        raise RuntimeError("rotary_cos and rotary_sin must be passed together")
    out, lse = ops.attention_forward(
        q, kcache, vcache, out=out_, k_new=k_, v_new=v_, seqused_k=seqlens_k_, rotary_cos=rotary_cos_,
        rotary_sin=rotary_sin_, rotary_interleaved=is_rotary_interleaved, cache_batch_idx=cache_batch_idx_,
        block_table=block_table_, alibi_slopes=alibi_slopes_, softmax_scale=softmax_scale, causal=is_causal,
        window_left=window_size_left, window_right=window_size_right, softcap=softcap, num_splits=num_splits)
    return [out, lse]


def _check_bwd_features(alibi_slopes_, p_dropout, softcap):
    if p_dropout != 0.0:
        raise RuntimeError("NPU FlashAttention does not support dropout")
    if alibi_slopes_ is not None:
        raise RuntimeError("the backward does not support alibi_slopes")


def bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, alibi_slopes_, p_dropout, softmax_scale, is_causal,
        window_size_left, window_size_right, softcap, deterministic, gen_=None, rng_state=None):
    """Backward of ``fwd`` (argument order of the reference's pybind ``bwd``,
    flash_attn_npu_v2/interface_arch22.py:232-252).  Returns [dq, dk, dv, softmax_d].
    ``deterministic``: head dim 128 without softcap runs on kernels without atomics (bit-reproducible whatever the flag
    says); the other shapes accumulate dQ with atomic adds and the flag does not change that."""
    _check_bwd_features(alibi_slopes_, p_dropout, softcap)
    dq, dk, dv = ops.attention_backward(dout, q, k, v, out, softmax_lse, dq=dq_, dk=dk_, dv=dv_,
                                        softmax_scale=softmax_scale, causal=is_causal,
                                        window_left=window_size_left, window_right=window_size_right, softcap=softcap)
    return [dq, dk, dv, torch.empty(0, dtype=torch.float32, device=q.device)]


def varlen_bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_seqlens_q, cu_seqlens_k, alibi_slopes_, max_seqlen_q,
               max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left, window_size_right,
               softcap, deterministic, gen_=None, rng_state=None):
    """Backward of ``varlen_fwd`` (argument order of the reference's pybind ``varlen_bwd``)."""
    _check_bwd_features(alibi_slopes_, p_dropout, softcap)
    dq, dk, dv = ops.attention_backward(dout, q, k, v, out, softmax_lse, dq=dq_, dk=dk_, dv=dv_,
                                        softmax_scale=softmax_scale, causal=is_causal,
                                        window_left=window_size_left, window_right=window_size_right, softcap=softcap,
                                        cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k,
                                        max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k)
    return [dq, dk, dv, torch.empty(0, dtype=torch.float32, device=q.device)]
