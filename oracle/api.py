"""API-level CPU oracle (TEST INFRASTRUCTURE ONLY): the three public forward
functions of the reference, evaluated with ``oracle.golden`` one sequence at a
time exactly like the reference tests drive their golden
(tests/test_flash_attn_npu_v2.py:350-403, :452-470, :595-621).

Features the reference rejects or ignores natively (KV append, rotary,
cache_batch_idx, alibi -- csrc/arch22/flash_attn_npu_v2/flash_api.cpp:415-436)
are restated from the docstring flash_attn_npu_v2/interface_arch22.py:1452-1537;
their parity is unpinned by any reference test.  Arithmetic defined here for
them: rotary in fp32 with separately rounded products
(``x1*cos - x2*sin``, ``x1*sin + x2*cos``), then round-to-nearest-even to the
cache dtype; v is a plain copy; ALiBi adds ``-slope*|i + s_k - s_q - j|`` to the
scaled scores.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import torch

from . import golden as G


def alibi_bias(slopes: torch.Tensor, s_q: int, s_k: int) -> torch.Tensor:
    """(H,) fp32 slopes -> (H, s_q, s_k) bias, interface_arch22.py:1524-1526."""
    i = torch.arange(s_q, dtype=torch.float32).view(-1, 1)
    j = torch.arange(s_k, dtype=torch.float32).view(1, -1)
    dist = (i + (s_k - s_q) - j).abs()
    return -slopes.to(torch.float32).view(-1, 1, 1) * dist


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
                 interleaved: bool) -> torch.Tensor:
    """x (S, H, D); cos/sin (seqlen_ro, rotary_dim/2); positions (S,) int64 -> rotated x, same dtype.

    Non-interleaved pairs (j, j + rotary_dim/2); interleaved pairs (2j, 2j+1)
    (interface_arch22.py:1520-1523).  Dims >= rotary_dim pass through.
    """
    rd = cos.shape[-1] * 2
    c = cos[positions].to(torch.float32).unsqueeze(1)  # (S,1,rd/2)
    s = sin[positions].to(torch.float32).unsqueeze(1)
    xf = x.to(torch.float32)
    out = xf.clone()
    if interleaved:
        x1 = xf[..., 0:rd:2]
        x2 = xf[..., 1:rd:2]
        out[..., 0:rd:2] = x1 * c - x2 * s
        out[..., 1:rd:2] = x1 * s + x2 * c
    else:
        x1 = xf[..., : rd // 2]
        x2 = xf[..., rd // 2: rd]
        out[..., : rd // 2] = x1 * c - x2 * s
        out[..., rd // 2: rd] = x1 * s + x2 * c
    return out.to(x.dtype)


def _one_sequence(q, k, v, scale, s_q_for_norm, max_k_for_norm, causal, window, softcap, slopes, round_p=True):
    s_q, s_k = q.shape[0], k.shape[0]
    is_causal, is_local, wl, wr = G.normalize_window(s_q_for_norm, max_k_for_norm, causal, window[0], window[1])
    mask = G.build_mask(s_q, s_k, is_causal, is_local, wl, wr)
    bias = alibi_bias(slopes, s_q, s_k) if slopes is not None else None
    out, lse = G.blockwise_attention(q, k, v, scale, mask, q.dtype, softcap, bias=bias, round_p=round_p)
    return G.patch_dead_rows(out, lse, mask)


def flash_attn_func(q, k, v, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, round_p=True):
    """q (B,S_q,H,D), k/v (B,S_k,H_k,D) -> out (B,S_q,H,D), lse (B,H,S_q) fp32."""
    b, s_q, h, d = q.shape
    s_k = k.shape[1]
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    outs, lses = [], []
    for i in range(b):
        slopes = None
        if alibi_slopes is not None:
            slopes = alibi_slopes if alibi_slopes.dim() == 1 else alibi_slopes[i]
        o, l = _one_sequence(q[i], k[i], v[i], scale, s_q, s_k, causal, window_size, softcap, slopes, round_p)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                           softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                           alibi_slopes=None):
    """q (T_q,H,D), k/v (T_k,H_k,D) -> out (T_q,H,D), lse (H,T_q) fp32."""
    h, d = q.shape[1], q.shape[2]
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    out = torch.zeros_like(q)
    lse = torch.full((h, q.shape[0]), float("inf"), dtype=torch.float32)
    cq = cu_seqlens_q.tolist()
    ck = cu_seqlens_k.tolist()
    for i in range(len(cq) - 1):
        qs, qe, ks, ke = cq[i], cq[i + 1], ck[i], ck[i + 1]
        if qe == qs:
            continue
        slopes = None
        if alibi_slopes is not None:
            slopes = alibi_slopes if alibi_slopes.dim() == 1 else alibi_slopes[i]
        o, l = _one_sequence(q[qs:qe], k[ks:ke], v[ks:ke], scale, max_seqlen_q, max_seqlen_k, causal,
                             window_size, softcap, slopes)
        out[qs:qe] = o
        lse[:, qs:qe] = l
    return out, lse


def gather_paged(cache: torch.Tensor, block_row: torch.Tensor, length: int) -> torch.Tensor:
    """Logical token t lives at page block_row[t // P], row t % P
    (tests/test_flash_attn_npu_v2.py:363-371), vectorised."""
    p = cache.shape[1]
    t = torch.arange(length)
    return cache[block_row.long()[t // p], t % p]


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
                            cache_batch_idx=None, block_table=None, softmax_scale=None, causal=False,
                            window_size=(-1, -1), softcap=0.0, rotary_interleaved=True, alibi_slopes=None,
                            round_p=True):
    """Mutates k_cache / v_cache in place when k, v are given.  Returns (out (B,S_q,H,D), lse (B,H,S_q))."""
    b, s_q, h, d = q.shape
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    paged = block_table is not None
    if cache_seqlens is None:
        assert not paged
        lens = [k_cache.shape[1]] * b
    elif isinstance(cache_seqlens, int):
        lens = [cache_seqlens] * b
    else:
        lens = [int(x) for x in cache_seqlens.tolist()]
    s_new = 0 if k is None else k.shape[1]
    max_k = max(l + s_new for l in lens)
    is_causal, is_local, _, _ = G.normalize_window(s_q, max_k, causal, window_size[0], window_size[1])
    outs, lses = [], []
    for i in range(b):
        L = lens[i]
        row = i if cache_batch_idx is None else int(cache_batch_idx[i])
        qi = q[i]
        if k is not None:
            kn, vn = k[i], v[i]
            if rotary_cos is not None:
                kpos = torch.arange(L, L + s_new)
                kn = apply_rotary(kn, rotary_cos, rotary_sin, kpos, rotary_interleaved)
                if is_causal or is_local:
                    qpos = torch.arange(L, L + s_q)
                else:
                    qpos = torch.full((s_q,), L, dtype=torch.int64)
                qi = apply_rotary(qi, rotary_cos, rotary_sin, qpos, rotary_interleaved)
            if paged:
                p = k_cache.shape[1]
                t = torch.arange(L, L + s_new)
                blk = block_table[i].long()[t // p]
                k_cache[blk, t % p] = kn
                v_cache[blk, t % p] = vn
            else:
                k_cache[row, L:L + s_new] = kn
                v_cache[row, L:L + s_new] = vn
        s_k = L + s_new
        if paged:
            ki = gather_paged(k_cache, block_table[i], s_k)
            vi = gather_paged(v_cache, block_table[i], s_k)
        else:
            ki, vi = k_cache[row, :s_k], v_cache[row, :s_k]
        slopes = None
        if alibi_slopes is not None:
            slopes = alibi_slopes if alibi_slopes.dim() == 1 else alibi_slopes[i]
        o, l = _one_sequence(qi, ki, vi, scale, s_q, max_k, causal, window_size, softcap, slopes, round_p)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def merge_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor, out_dtype=None):
    """Split-KV merge, csrc/arch22/flash_attn_npu_v2/CombineScale.hpp:165-309.

    o_parts (n, ..., D) fp32 normalised partial outputs, lse_parts (n, ...) fp32
    with -inf marking an empty partial.  Rows whose every partial is empty give
    O = 0, LSE = +inf.
    """
    m = lse_parts.max(dim=0)[0]
    safe_m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse_parts - safe_m)
    w = torch.nan_to_num(w, nan=0.0)
    tot = w.sum(dim=0)
    o = (torch.where(w.unsqueeze(-1) > 0, o_parts, torch.zeros_like(o_parts)) * w.unsqueeze(-1)).sum(dim=0) / torch.where(tot > 0, tot, torch.ones_like(tot)).unsqueeze(-1)
    o = torch.where((tot > 0).unsqueeze(-1), o, torch.zeros_like(o))
    lse = torch.where(tot > 0, safe_m + torch.log(tot), torch.full_like(tot, float("inf")))
    return (o.to(out_dtype) if out_dtype is not None else o), lse
