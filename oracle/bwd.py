"""CPU restatement of the reference's backward golden -- TEST INFRASTRUCTURE, not a product path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this module.

Follows tests/fa_small_op_golden.py of the reference:
  * masks                      make_window_atten_mask / normalize_window      :21-58
  * P from the forward's LSE   softmax_res_from_fa_lse_bsnd / _tnd_slice      :106-176
      S = (q k^T computed in the input dtype) -> fp32 * scale, masked + (-40000), P = exp(S - lse), masked -> 0
  * gradients                  tsoftmax_grad, tbackward_bsnd / tbackward_tnd   :69-72, :179-204
      dP = dO V^T, dV = P^T dO, dS = (dP - rowsum(dP o P)) o P * scale, dQ = dS K, dK = dS^T Q
  * GQA                        broadcast_kv_single, sum_gqa_grad               :11-19, :92-103
  * drivers                    golden_bsnd_bwd_from_fwd / golden_tnd_bwd_from_fwd :207-353
Pinned by tests/golden/bwd/*.npz, which hold outputs of those reference functions
(tests/golden/make_golden_bwd.py); dropout is not restated (not built).
"""
from __future__ import annotations

import torch


def normalize_window(seq_q, seq_k, is_causal, wl, wr):
    if wl >= seq_k - 1:
        wl = -1
    if wr >= seq_q - 1:
        wr = -1
    if is_causal:
        wr = 0
    causal_out = wl < 0 and wr == 0
    local = (wl >= 0 or wr >= 0) and not causal_out
    return wl, wr, causal_out, local


def window_mask(seq_q, seq_k, is_causal, wl, wr):
    """1 where masked, or None (fa_small_op_golden.py:36-58)."""
    wl, wr, causal_out, local = normalize_window(seq_q, seq_k, is_causal, wl, wr)
    if not causal_out and not local:
        return None
    off = seq_k - seq_q
    ones = torch.ones((seq_q, seq_k))
    if causal_out:
        return torch.triu(ones, diagonal=off + 1)
    mask = torch.zeros((seq_q, seq_k))
    if wr >= 0:
        mask = mask + torch.triu(ones, diagonal=wr + 1 + off)
    if wl >= 0:
        mask = mask + torch.tril(ones, diagonal=-wl - 1 + off)
    return mask


def _bwd_one(q, k, v, dout, lse, scale, is_causal, wl, wr, gtype, softcap=0.0):
    """q, dout (1, h, s_q, d); k, v (1, h, s_k, d) already broadcast to h heads, in gtype; lse (h, s_q) fp32."""
    compute_dtype = q.dtype
    qg, kg, vg, dx = (t.to(gtype) for t in (q, k, v, dout))
    mask = window_mask(q.shape[2], k.shape[2], is_causal, wl, wr)
    qk = torch.matmul(q.to(compute_dtype), k.to(compute_dtype).permute(0, 1, 3, 2)).to(torch.float32).mul(scale)
    cap_factor = None
    if softcap > 0.0:  # :80-89 (factor from the unmasked scaled scores), :124-125
        cap_factor = 1.0 - torch.tanh(qk.to(gtype) / softcap) ** 2
        qk = softcap * torch.tanh(qk / softcap)
    if mask is not None:
        qk = qk + mask.to(torch.float32) * (-40000.0)
    p = torch.exp(qk.to(gtype) - lse.to(torch.float32).to(gtype).unsqueeze(0).unsqueeze(-1))
    if mask is not None:
        p[mask.bool().broadcast_to(p.shape)] = 0
    dp = torch.matmul(dx, vg.permute(0, 1, 3, 2))
    dv = torch.matmul(p.permute(0, 1, 3, 2), dx)
    ds = (dp - (dp * p).sum(dim=-1, keepdim=True)) * p * scale
    if cap_factor is not None:
        ds = ds * cap_factor
    dq = torch.matmul(ds, kg)
    dk = torch.matmul(ds.permute(0, 1, 3, 2), qg)
    return dq, dk, dv


def _sum_groups(g, h, h_k):
    if h == h_k:
        return g
    b, _, s, d = g.shape
    return g.reshape(b, h_k, h // h_k, s, d).sum(dim=2)


def attention_backward(q, k, v, dout, lse, *, softmax_scale, causal=False, window=(-1, -1), softcap=0.0,
                       gtype=torch.float64):
    """Dense (b, s, h, d) tensors, lse (b, h, s_q) -> dq, dk, dv in the input dtype (golden_bsnd_bwd_from_fwd)."""
    b, s_q, h, d = q.shape
    h_k = k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    for bi in range(b):
        qb = q[bi:bi + 1].permute(0, 2, 1, 3)
        kb = k[bi:bi + 1].permute(0, 2, 1, 3).repeat_interleave(h // h_k, dim=1)
        vb = v[bi:bi + 1].permute(0, 2, 1, 3).repeat_interleave(h // h_k, dim=1)
        db = dout[bi:bi + 1].permute(0, 2, 1, 3)
        gq, gk, gv = _bwd_one(qb, kb, vb, db, lse[bi], softmax_scale, causal, window[0], window[1], gtype, softcap)
        dq[bi] = gq.permute(0, 2, 1, 3)[0].to(q.dtype)
        dk[bi] = _sum_groups(gk, h, h_k).permute(0, 2, 1, 3)[0].to(k.dtype)
        dv[bi] = _sum_groups(gv, h, h_k).permute(0, 2, 1, 3)[0].to(v.dtype)
    return dq, dk, dv


def attention_varlen_backward(q, k, v, dout, lse, cu_seqlens_q, cu_seqlens_k, *, softmax_scale, causal=False,
                              window=(-1, -1), softcap=0.0, gtype=torch.float64):
    """Packed (total, h, d) tensors, lse (h, total_q) (golden_tnd_bwd_from_fwd); empty sequences get zero gradients."""
    h, h_k = q.shape[1], k.shape[1]
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    cq, ck = [int(x) for x in cu_seqlens_q], [int(x) for x in cu_seqlens_k]
    for i in range(len(cq) - 1):
        q0, q1, k0, k1 = cq[i], cq[i + 1], ck[i], ck[i + 1]
        if q1 == q0 or k1 == k0:
            continue
        qb = q[q0:q1].unsqueeze(0).permute(0, 2, 1, 3)
        kb = k[k0:k1].unsqueeze(0).permute(0, 2, 1, 3).repeat_interleave(h // h_k, dim=1)
        vb = v[k0:k1].unsqueeze(0).permute(0, 2, 1, 3).repeat_interleave(h // h_k, dim=1)
        db = dout[q0:q1].unsqueeze(0).permute(0, 2, 1, 3)
        gq, gk, gv = _bwd_one(qb, kb, vb, db, lse[:, q0:q1], softmax_scale, causal, window[0], window[1], gtype, softcap)
        dq[q0:q1] = gq.permute(0, 2, 1, 3)[0].to(q.dtype)
        dk[k0:k1] = _sum_groups(gk, h, h_k).permute(0, 2, 1, 3)[0].to(k.dtype)
        dv[k0:k1] = _sum_groups(gv, h, h_k).permute(0, 2, 1, 3)[0].to(v.dtype)
    return dq, dk, dv
