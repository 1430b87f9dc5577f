"""``torch.library`` operators of the FA3-style package, registered for CUDA.

Names and argument lists follow the reference's registrations (flash_attn_npu_v3/interface_arch22.py:63-154 forward
with its fake :157-259, :262-360 backward; ``device_types="npu"`` there), so graphs captured against the reference
keep their node names; the bodies call this library's extension module.  One operator is added:
``_flash_attn_forward_inplace`` is the forward for calls that bring new tokens (``k_new`` / ``v_new``), which are
written into the KV cache: it declares that it mutates ``k`` and ``v``, which a tracing compiler has to know (the
reference registers its forward as mutating nothing although its documented semantics append in place).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

import flash_attn_npu_arch22_v3 as _ext

NS = "flash_attn_npu_arch22_v3"


def _contig(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _call(q, k, v, k_new, v_new, qv, out_, cu_seqlens_q, cu_seqlens_k, cu_seqlens_k_new, seqused_q, seqused_k,
          max_seqlen_q, max_seqlen_k, page_table, kv_batch_idx, leftpad_k, rotary_cos, rotary_sin, seqlens_rotary,
          q_descale, k_descale, v_descale, softmax_scale, causal, window_size_left, window_size_right, attention_chunk,
          softcap, rotary_interleaved, scheduler_metadata, num_splits, pack_gqa, sm_margin):
    q, k, v, k_new, v_new = [_contig(x) for x in (q, k, v, k_new, v_new)]
    cu_seqlens_q, cu_seqlens_k, seqused_k, page_table, kv_batch_idx = [
        _contig(x) for x in (cu_seqlens_q, cu_seqlens_k, seqused_k, page_table, kv_batch_idx)]
    out, lse, out_accum, lse_accum = _ext.fwd(
        q, k, v, k_new, v_new, qv, out_, cu_seqlens_q, cu_seqlens_k, cu_seqlens_k_new, seqused_q, seqused_k,
        max_seqlen_q, max_seqlen_k, page_table, kv_batch_idx, leftpad_k, rotary_cos, rotary_sin, seqlens_rotary,
        q_descale, k_descale, v_descale, softmax_scale, causal, window_size_left, window_size_right,
        attention_chunk, softcap, rotary_interleaved, scheduler_metadata, num_splits, pack_gqa, sm_margin)
    if out_accum is None:
        out_accum = torch.empty((0,), device=out.device)
    if lse_accum is None:
        lse_accum = torch.empty((0,), device=out.device)
    return out, lse, out_accum, lse_accum


def _shapes(q, v, out_, cu_seqlens_q, max_seqlen_q):
    if out_ is not None:
        raise TypeError("Tracing (torch.compile / torch.export) with a pre-allocated output tensor is not supported.")
    if cu_seqlens_q is not None:
        if max_seqlen_q is None:
            raise ValueError("max_seqlen_q must be provided if cu_seqlens_q is provided")
        total_q, h, _d = q.shape
        out = torch.empty((total_q, h, v.shape[-1]), dtype=q.dtype, device=q.device)
        lse = torch.empty((h, total_q), dtype=torch.float32, device=q.device)
    else:
        b, s_q, h, _d = q.shape
        out = torch.empty((b, s_q, h, v.shape[-1]), dtype=q.dtype, device=q.device)
        lse = torch.empty((b, h, s_q), dtype=torch.float32, device=q.device)
    empty = torch.empty((0,), device=q.device)  # split partials are never returned by this backend
    return out, lse, empty, torch.empty((0,), device=q.device)


@torch.library.custom_op(f"{NS}::_flash_attn_forward", mutates_args=(), device_types="cuda")
def _flash_attn_forward(
        q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_new: Optional[torch.Tensor] = None,
        v_new: Optional[torch.Tensor] = None, qv: Optional[torch.Tensor] = None, out_: Optional[torch.Tensor] = None,
        cu_seqlens_q: Optional[torch.Tensor] = None, cu_seqlens_k: Optional[torch.Tensor] = None,
        cu_seqlens_k_new: Optional[torch.Tensor] = None, seqused_q: Optional[torch.Tensor] = None,
        seqused_k: Optional[torch.Tensor] = None, max_seqlen_q: Optional[int] = None,
        max_seqlen_k: Optional[int] = None, page_table: Optional[torch.Tensor] = None,
        kv_batch_idx: Optional[torch.Tensor] = None, leftpad_k: Optional[torch.Tensor] = None,
        rotary_cos: Optional[torch.Tensor] = None, rotary_sin: Optional[torch.Tensor] = None,
        seqlens_rotary: Optional[torch.Tensor] = None, q_descale: Optional[torch.Tensor] = None,
        k_descale: Optional[torch.Tensor] = None, v_descale: Optional[torch.Tensor] = None,
        softmax_scale: Optional[float] = None, causal: bool = False, window_size_left: int = -1,
        window_size_right: int = -1, attention_chunk: int = 0, softcap: float = 0.0, rotary_interleaved: bool = True,
        scheduler_metadata: Optional[torch.Tensor] = None, num_splits: int = 1, pack_gqa: Optional[bool] = None,
        sm_margin: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    if k_new is not None or v_new is not None:
        raise RuntimeError("new tokens are appended to the cache in place: use _flash_attn_forward_inplace")
    return _call(q, k, v, None, None, qv, out_, cu_seqlens_q, cu_seqlens_k, cu_seqlens_k_new, seqused_q, seqused_k,
                 max_seqlen_q, max_seqlen_k, page_table, kv_batch_idx, leftpad_k, rotary_cos, rotary_sin, seqlens_rotary,
                 q_descale, k_descale, v_descale, softmax_scale, causal, window_size_left, window_size_right,
                 attention_chunk, softcap, rotary_interleaved, scheduler_metadata, num_splits, pack_gqa, sm_margin)


@_flash_attn_forward.register_fake
def _(q, k, v, k_new=None, v_new=None, qv=None, out_=None, cu_seqlens_q=None, cu_seqlens_k=None, cu_seqlens_k_new=None,
      seqused_q=None, seqused_k=None, max_seqlen_q=None, max_seqlen_k=None, page_table=None, kv_batch_idx=None,
      leftpad_k=None, rotary_cos=None, rotary_sin=None, seqlens_rotary=None, q_descale=None, k_descale=None,
      v_descale=None, softmax_scale=None, causal=False, window_size_left=-1, window_size_right=-1, attention_chunk=0,
      softcap=0.0, rotary_interleaved=True, scheduler_metadata=None, num_splits=1, pack_gqa=None, sm_margin=0):
    return _shapes(q, v, out_, cu_seqlens_q, max_seqlen_q)


@torch.library.custom_op(f"{NS}::_flash_attn_forward_inplace", mutates_args=("k", "v"), device_types="cuda")
def _flash_attn_forward_inplace(
        q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
        cu_seqlens_q: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None,
        max_seqlen_q: Optional[int] = None, page_table: Optional[torch.Tensor] = None,
        kv_batch_idx: Optional[torch.Tensor] = None, rotary_cos: Optional[torch.Tensor] = None,
        rotary_sin: Optional[torch.Tensor] = None, softmax_scale: Optional[float] = None, causal: bool = False,
        window_size_left: int = -1, window_size_right: int = -1, softcap: float = 0.0, rotary_interleaved: bool = True,
        scheduler_metadata: Optional[torch.Tensor] = None, num_splits: int = 1, pack_gqa: Optional[bool] = None,
        sm_margin: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _call(q, k, v, k_new, v_new, None, None, cu_seqlens_q, None, None, None, seqused_k, max_seqlen_q, None,
                 page_table, kv_batch_idx, None, rotary_cos, rotary_sin, None, None, None, None, softmax_scale, causal,
                 window_size_left, window_size_right, 0, softcap, rotary_interleaved, scheduler_metadata, num_splits,
                 pack_gqa, sm_margin)


@_flash_attn_forward_inplace.register_fake
def _(q, k, v, k_new, v_new, cu_seqlens_q=None, seqused_k=None, max_seqlen_q=None, page_table=None, kv_batch_idx=None,
      rotary_cos=None, rotary_sin=None, softmax_scale=None, causal=False, window_size_left=-1, window_size_right=-1,
      softcap=0.0, rotary_interleaved=True, scheduler_metadata=None, num_splits=1, pack_gqa=None, sm_margin=0):
    return _shapes(q, v, None, cu_seqlens_q, max_seqlen_q)


@torch.library.custom_op(f"{NS}::_flash_attn_backward", mutates_args=("dq", "dk", "dv"), device_types="cuda")
def _flash_attn_backward(
        dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
        softmax_lse: torch.Tensor, cu_seqlens_q: Optional[torch.Tensor] = None,
        cu_seqlens_k: Optional[torch.Tensor] = None, sequed_q: Optional[torch.Tensor] = None,
        sequed_k: Optional[torch.Tensor] = None, max_seqlen_q: Optional[int] = None, max_seqlen_k: Optional[int] = None,
        dq: Optional[torch.Tensor] = None, dk: Optional[torch.Tensor] = None, dv: Optional[torch.Tensor] = None,
        softmax_scale: Optional[float] = None, is_causal: bool = False, window_size_left: int = -1,
        window_size_right: int = -1, softcap: float = 0.0, deterministic: bool = False, sm_margin: int = 0) -> torch.Tensor:
    dout, q, k, v, out = [_contig(x) for x in (dout, q, k, v, out)]
    _, _, _, softmax_d = _ext.bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, sequed_q,
                                  sequed_k, max_seqlen_q, max_seqlen_k, softmax_scale, is_causal, window_size_left,
                                  window_size_right, softcap, deterministic, sm_margin)
    return softmax_d


@_flash_attn_backward.register_fake
def _(dout, q, k, v, out, softmax_lse, cu_seqlens_q=None, cu_seqlens_k=None, sequed_q=None, sequed_k=None,
      max_seqlen_q=None, max_seqlen_k=None, dq=None, dk=None, dv=None, softmax_scale=None, is_causal=False,
      window_size_left=-1, window_size_right=-1, softcap=0.0, deterministic=False, sm_margin=0):
    return torch.empty((0,), dtype=torch.float32, device=q.device)
