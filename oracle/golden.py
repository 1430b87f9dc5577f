"""CPU restatement of the reference's forward golden (TEST INFRASTRUCTURE ONLY).

Follows, in this repo's own code:

* ``ref_flash_attention``  tests/test_flash_attn_npu_v2.py:84-143 (helpers
  ``group_matmul`` :10-24, ``softmax1`` :26-44, ``qkMM1`` :46-63, ``pvMM2``
  :65-82) -- fp32 math on up-cast inputs, KV processed in chunks of 512 with
  a running max / running sum, masked scores get ``-1e4`` added, P rounded to
  the input dtype before P.V, ``LSE = log(l) + m``.
* window normalisation: csrc/arch22/flash_attn_npu_v2/flash_api.cpp:483-494,
  mirrored by tests/test_flash_attn_npu_v2.py:294-303.
* masks: tests/test_flash_attn_npu_v2.py:330-348 (bottom-right aligned causal
  ``triu``; literal-integer band for local attention).
* dead rows (no visible key): O = 0, LSE = +inf,
  tests/test_flash_attn_npu_v2.py:383-401.

Pinned against the reference's own functions by tests/golden/*.npz.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

MASK_ADD = -1e4  # tests/test_flash_attn_npu_v2.py:116
GOLDEN_CHUNK = 512  # tests/test_flash_attn_npu_v2.py:102


def normalize_window(seqlen_q: int, max_seqlen_k: int, causal: bool, wl: int, wr: int):
    """Host-side window normalisation.  Returns (is_causal, is_local, wl, wr).

    csrc/arch22/flash_attn_npu_v2/flash_api.cpp:483-494.  ``max_seqlen_k`` is the
    maximum key length over the batch, not a per-sequence value.
    """
    if max_seqlen_k > 0 and wl >= max_seqlen_k - 1:
        wl = -1
    if seqlen_q > 0 and wr >= seqlen_q - 1:
        wr = -1
    if causal:
        wr = 0
    is_causal = wl < 0 and wr == 0
    is_local = (wl >= 0 or wr >= 0) and not is_causal
    return is_causal, is_local, wl, wr


def build_mask(s_q: int, s_k: int, is_causal: bool, is_local: bool, wl: int, wr: int) -> Optional[torch.Tensor]:
    """Boolean (s_q, s_k) mask, True = masked out; None when nothing is masked.

    causal: key j visible iff j <= i + (s_k - s_q)   (test :342-346).
    local : visible iff (s_k-s_q) - wl <= j - i <= (s_k-s_q) + wr with wl, wr
            taken as literal integers, negatives included (test :330-340).
    """
    if not (is_causal or is_local):
        return None
    i = torch.arange(s_q).view(-1, 1)
    j = torch.arange(s_k).view(1, -1)
    rel = j - i
    off = s_k - s_q
    if is_causal:
        return rel > off
    return (rel < off - wl) | (rel > off + wr)


def blockwise_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    mask: Optional[torch.Tensor],
    dtype: torch.dtype,
    softcap: float = 0.0,
    bias: Optional[torch.Tensor] = None,
    chunk: int = GOLDEN_CHUNK,
    round_p: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """One sequence.  q (S_q,H,D); k, v (S_k,H_k,D) -> out (S_q,H,D) ``dtype``, lse (H,S_q) fp32.

    ``bias`` (H,S_q,S_k) fp32 is added to the scaled (and soft-capped) scores;
    it carries the ALiBi term, which the reference golden does not have.
    ``round_p=False`` gives the no-down-cast variant used by the 2x-error rule.
    """
    s_q, h, d = q.shape
    s_k, h_k, _ = k.shape
    g = h // h_k
    qf = q.to(torch.float32).permute(1, 0, 2)                      # (H, S_q, D)
    kf = k.to(torch.float32).permute(1, 2, 0)                      # (H_k, D, S_k)
    vf = v.to(torch.float32).permute(1, 0, 2)                      # (H_k, S_k, D)
    scale_t = torch.tensor(scale, dtype=torch.float32)
    run_max = None
    run_sum = None
    acc = None
    for start in range(0, s_k, chunk):
        stop = min(start + chunk, s_k)
        kc = kf[:, :, start:stop]
        vc = vf[:, start:stop, :]
        # (H_k, G, S_q, D) x (H_k, 1, D, n) -> (H, S_q, n); contraction over D in 128-wide
        # slabs like qkMM1 (:46-63) so the fp32 summation order is the same.
        s = None
        for d0 in range(0, d, 128):
            part = torch.matmul(qf[:, :, d0:d0 + 128].reshape(h_k, g, s_q, -1), kc[:, d0:d0 + 128, :].unsqueeze(1))
            s = part if s is None else s + part
        s = s.reshape(h, s_q, stop - start) * scale_t
        if softcap > 0.0:
            s = softcap * torch.tanh(s / softcap)
        if bias is not None:
            s = s + bias[:, :, start:stop]
        if mask is not None:
            s = s + mask[:s_q, start:stop].to(torch.float32) * MASK_ADD
        blk_max = s.max(dim=-1, keepdim=True)[0]
        if run_max is None:
            new_max = blk_max
            decay = None
        else:
            new_max = torch.maximum(run_max, blk_max)
            decay = torch.exp(run_max - new_max)
        p = torch.exp(s - new_max)
        blk_sum = p.sum(dim=-1, keepdim=True)
        if round_p:
            p = p.to(dtype)
        pv = None
        n = stop - start
        for n0 in range(0, n, 128):  # pvMM2 (:65-82) sums 128-wide slabs of the key axis
            part = torch.matmul(p[:, :, n0:n0 + 128].to(torch.float32).reshape(h_k, g, s_q, -1),
                                vc[:, n0:n0 + 128, :].unsqueeze(1))
            pv = part if pv is None else pv + part
        pv = pv.reshape(h, s_q, d)
        if decay is None:
            run_sum, acc = blk_sum, pv
        else:
            run_sum = run_sum * decay + blk_sum
            acc = acc * decay + pv
        run_max = new_max
    if acc is None:  # s_k == 0
        out = torch.zeros(s_q, h, d, dtype=dtype)
        lse = torch.full((h, s_q), float("inf"), dtype=torch.float32)
        return out, lse
    out = (acc / run_sum).permute(1, 0, 2)
    lse = (torch.log(run_sum) + run_max).squeeze(-1).to(torch.float32)
    return (out.to(dtype) if round_p else out), lse


def patch_dead_rows(out: torch.Tensor, lse: torch.Tensor, mask: Optional[torch.Tensor]):
    """Rows with no visible key: O = 0, LSE = +inf (test :383-401, README.md:126)."""
    if mask is None:
        return out, lse
    dead = mask.all(dim=-1)  # (S_q,)
    if dead.any():
        out = out.clone()
        lse = lse.clone()
        out[dead] = 0
        lse[:, dead] = float("inf")
    return out, lse


def dense_softmax_attention(q, k, v, scale, mask, bias=None, softcap=0.0, compute_dtype=torch.float32):
    """Plain (non-blockwise) attention of one sequence evaluated in ``compute_dtype``.

    With ``compute_dtype`` = the input dtype this is the "plain fp16/bf16 PyTorch
    attention" of the 2x-error acceptance rule; with fp32 it is an independent
    cross-check of ``blockwise_attention``.  Returns (out (S_q,H,D), lse (H,S_q)).
    """
    s_q, h, d = q.shape
    h_k = k.shape[1]
    g = h // h_k
    qc = q.to(compute_dtype).permute(1, 0, 2)
    kc = k.to(compute_dtype).permute(1, 2, 0).repeat_interleave(g, dim=0)
    vc = v.to(compute_dtype).permute(1, 0, 2).repeat_interleave(g, dim=0)
    s = torch.matmul(qc, kc) * scale
    if softcap > 0.0:
        s = softcap * torch.tanh(s / softcap)
    if bias is not None:
        s = s + bias.to(compute_dtype)
    if mask is not None:
        s = s.masked_fill(mask.unsqueeze(0), float("-inf"))
    lse = torch.logsumexp(s.to(torch.float32), dim=-1)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    out = torch.matmul(p, vc).permute(1, 0, 2)
    lse = torch.where(torch.isinf(lse) & (lse < 0), torch.full_like(lse, float("inf")), lse)
    return out, lse
