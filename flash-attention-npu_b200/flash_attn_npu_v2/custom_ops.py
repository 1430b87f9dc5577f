"""``torch.library`` operators of the FA2-style package, registered for CUDA.

The reference registers its native calls as custom operators so that ``torch.compile`` / ``torch.export`` see one
opaque node per attention call (flash_attn_npu_v2/interface_arch22.py:46-106 forward, :112-201 varlen forward,
:204-293 backward, :296-392 varlen backward; ``device_types="npu"`` there).  The operator names and argument lists
are kept -- graphs captured against the reference keep their node names -- the device type is "cuda", and the
bodies call this library's extension module.  Each operator has a fake (meta) implementation that returns tensors
of the shapes and dtypes the real one produces, which is all a tracing compiler needs.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

import flash_attn_npu_arch22_v2 as _ext

NS = "flash_attn_npu_arch22_v2"


def _contig(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _aux_like(q):
    """The two placeholders of the reference's return list: the attention-probability tensor (never produced) and
    the dropout generator state (dropout is not supported)."""
    return torch.empty((0,), dtype=q.dtype, device=q.device), torch.empty((2,), dtype=torch.int64, device=q.device)


@torch.library.custom_op(f"{NS}::_flash_attn_forward", mutates_args=(), device_types="cuda")
def _flash_attn_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dropout_p: float, softmax_scale: float,
                        causal: bool, window_size_left: int, window_size_right: int, softcap: float,
                        alibi_slopes: Optional[torch.Tensor], return_softmax: bool
                        ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    q, k, v = [_contig(x) for x in (q, k, v)]
    out, lse, p, rng = _ext.fwd(q, k, v, None, alibi_slopes, dropout_p, softmax_scale, causal, window_size_left,
                                window_size_right, softcap, return_softmax, None)
    return out, lse, p, rng


@_flash_attn_forward.register_fake
def _(q, k, v, dropout_p, softmax_scale, causal, window_size_left, window_size_right, softcap, alibi_slopes,
      return_softmax):
    b, s_q, h, _d = q.shape
    p, rng = _aux_like(q)
    return torch.empty_like(q), torch.empty((b, h, s_q), dtype=torch.float32, device=q.device), p, rng


@torch.library.custom_op(f"{NS}::_flash_attn_varlen_forward", mutates_args=(), device_types="cuda")
def _flash_attn_varlen_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                               cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, dropout_p: float,
                               softmax_scale: float, causal: bool, window_size_left: int = -1,
                               window_size_right: int = -1, softcap: float = 0.0,
                               alibi_slopes: Optional[torch.Tensor] = None, return_softmax: bool = False,
                               block_table: Optional[torch.Tensor] = None, leftpad_k: Optional[torch.Tensor] = None,
                               seqused_k: Optional[torch.Tensor] = None, zero_tensors: bool = False
                               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    q, k, v = [_contig(x) for x in (q, k, v)]
    out, lse, p, rng = _ext.varlen_fwd(q, k, v, None, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table,
                                       alibi_slopes, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale,
                                       zero_tensors, causal, window_size_left, window_size_right, softcap,
                                       return_softmax, None)
    return out, lse, p, rng


@_flash_attn_varlen_forward.register_fake
def _(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal,
      window_size_left=-1, window_size_right=-1, softcap=0.0, alibi_slopes=None, return_softmax=False,
      block_table=None, leftpad_k=None, seqused_k=None, zero_tensors=False):
    total_q, h, _d = q.shape
    p, rng = _aux_like(q)
    return torch.empty_like(q), torch.empty((h, total_q), dtype=torch.float32, device=q.device), p, rng


@torch.library.custom_op(f"{NS}::_flash_attn_backward", mutates_args=("dq", "dk", "dv"), device_types="cuda")
def _flash_attn_backward(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                         softmax_lse: torch.Tensor, dq: Optional[torch.Tensor], dk: Optional[torch.Tensor],
                         dv: Optional[torch.Tensor], dropout_p: float, softmax_scale: float, causal: bool,
                         window_size_left: int, window_size_right: int, softcap: float,
                         alibi_slopes: Optional[torch.Tensor], deterministic: bool,
                         rng_state: Optional[torch.Tensor] = None) -> torch.Tensor:
    dout, q, k, v, out = [_contig(x) for x in (dout, q, k, v, out)]
    _, _, _, softmax_d = _ext.bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, alibi_slopes, dropout_p, softmax_scale,
                                  causal, window_size_left, window_size_right, softcap, deterministic, None, rng_state)
    return softmax_d


@_flash_attn_backward.register_fake
def _(dout, q, k, v, out, softmax_lse, dq, dk, dv, dropout_p, softmax_scale, causal, window_size_left,
      window_size_right, softcap, alibi_slopes, deterministic, rng_state=None):
    return torch.empty((0,), dtype=torch.float32, device=q.device)


@torch.library.custom_op(f"{NS}::_flash_attn_varlen_backward", mutates_args=("dq", "dk", "dv"), device_types="cuda")
def _flash_attn_varlen_backward(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                out: torch.Tensor, softmax_lse: torch.Tensor, dq: Optional[torch.Tensor],
                                dk: Optional[torch.Tensor], dv: Optional[torch.Tensor], cu_seqlens_q: torch.Tensor,
                                cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, dropout_p: float,
                                softmax_scale: float, causal: bool, window_size_left: int, window_size_right: int,
                                softcap: float, alibi_slopes: Optional[torch.Tensor], deterministic: bool,
                                rng_state: Optional[torch.Tensor] = None, zero_tensors: bool = False) -> torch.Tensor:
    dout, q, k, v, out = [_contig(x) for x in (dout, q, k, v, out)]
    _, _, _, softmax_d = _ext.varlen_bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                                         alibi_slopes, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale,
                                         zero_tensors, causal, window_size_left, window_size_right, softcap,
                                         deterministic, None, rng_state)
    return softmax_d


@_flash_attn_varlen_backward.register_fake
def _(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
      softmax_scale, causal, window_size_left, window_size_right, softcap, alibi_slopes, deterministic, rng_state=None,
      zero_tensors=False):
    return torch.empty((0,), dtype=torch.float32, device=q.device)
