"""Torch-facing launcher: turns tensors into the POD parameter block of the C ABI.

PyTorch is plumbing here (device memory, the current stream); all compute happens in
libfa_b200.so.  Every function raises if the tensors are not CUDA tensors -- there is no
CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import lib as L

_sm_count = {}


def _num_sm(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return L.FA_FP16
    if t.dtype == torch.bfloat16:
        return L.FA_BF16
    raise RuntimeError("FlashAttention only supports FP16 and BF16 data types")


def _check_i32(t, name):
    if t is not None:
        if t.dtype != torch.int32:
            raise RuntimeError(f"{name} must have dtype int32")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dim() > 0 and t.stride(-1) != 1:
            raise RuntimeError(f"{name} must have contiguous last dimension")


def build_params(q, k, v, out, lse, *, k_new=None, v_new=None, cu_seqlens_q=None, cu_seqlens_k=None,
                 max_seqlen_q=None, max_seqlen_k=None, seqused_k=None, cache_batch_idx=None, block_table=None,
                 rotary_cos=None, rotary_sin=None, rotary_interleaved=True, alibi_slopes=None,
                 softmax_scale=1.0, causal=False, window_left=-1, window_right=-1, softcap=0.0, num_splits=0,
                 max_seqlen_k_known=-1, kv_pos_offset=0, kv_total=0, partial_out=False, kernel=L.KERNEL_AUTO,
                 num_sm=0) -> L.FwdParams:
    p = L.FwdParams()
    varlen_q = cu_seqlens_q is not None
    paged = block_table is not None
    p.q, p.k, p.v, p.o, p.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse)
    p.dtype = _dtype_code(q)
    if varlen_q:
        total_q, h, d = q.shape
        b = cu_seqlens_q.numel() - 1
        if max_seqlen_q is None:
            raise RuntimeError("max_seqlen_q is required with cu_seqlens_q")
        p.q_batch_stride, p.q_row_stride, p.q_head_stride = 0, q.stride(0), q.stride(1)
        p.o_batch_stride, p.o_row_stride, p.o_head_stride = 0, out.stride(0), out.stride(1)
        p.seqlen_q, p.total_q = int(max_seqlen_q), total_q
        p.lse_batch_stride, p.lse_head_stride = 0, lse.stride(0)
    else:
        b, s_q, h, d = q.shape
        p.q_batch_stride, p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
        p.o_batch_stride, p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1), out.stride(2)
        p.seqlen_q, p.total_q = s_q, b * s_q
        p.lse_batch_stride, p.lse_head_stride = lse.stride(0), lse.stride(1)
    if cu_seqlens_k is not None:
        if k.dim() != 3:
            raise RuntimeError("k must be (total_k, h_k, d) with cu_seqlens_k")
        h_k = k.shape[1]
        if max_seqlen_k is None:
            raise RuntimeError("max_seqlen_k is required with cu_seqlens_k")
        p.k_batch_stride, p.k_row_stride, p.k_head_stride = 0, k.stride(0), k.stride(1)
        p.v_batch_stride, p.v_row_stride, p.v_head_stride = 0, v.stride(0), v.stride(1)
        p.seqlen_k = int(max_seqlen_k)
        p.total_k = int(k.shape[0])
    else:
        if k.dim() != 4:
            raise RuntimeError("k must be 4-dimensional")
        h_k = k.shape[2]
        p.k_batch_stride, p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
        p.v_batch_stride, p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
        if paged or cache_batch_idx is not None:
            p.kv_outer = k.shape[0]  # pages / cache rows: bounds every block_table / cache_batch_idx entry
        if paged:
            p.page_size = k.shape[1]
            p.seqlen_k = block_table.shape[1] * k.shape[1]
            p.block_table_batch_stride = block_table.stride(0)
        else:
            p.seqlen_k = k.shape[1]
    p.b, p.h, p.h_k, p.d = b, h, h_k, d
    if k_new is not None:
        p.k_new, p.v_new = _ptr(k_new), _ptr(v_new)
        p.seqlen_new = k_new.shape[1]
        p.knew_batch_stride, p.knew_row_stride, p.knew_head_stride = k_new.stride(0), k_new.stride(1), k_new.stride(2)
        p.vnew_batch_stride, p.vnew_row_stride, p.vnew_head_stride = v_new.stride(0), v_new.stride(1), v_new.stride(2)
    p.cu_seqlens_q, p.cu_seqlens_k = _ptr(cu_seqlens_q), _ptr(cu_seqlens_k)
    p.seqused_k, p.cache_batch_idx, p.block_table = _ptr(seqused_k), _ptr(cache_batch_idx), _ptr(block_table)
    if rotary_cos is not None:
        p.rotary_cos, p.rotary_sin = _ptr(rotary_cos), _ptr(rotary_sin)
        p.rotary_seqlen, p.rotary_dim = rotary_cos.shape[0], rotary_cos.shape[1] * 2
        p.rotary_interleaved = int(bool(rotary_interleaved))
    if alibi_slopes is not None:
        p.alibi_slopes = _ptr(alibi_slopes)
        p.alibi_batch_stride = alibi_slopes.stride(0) if alibi_slopes.dim() == 2 else 0
    p.causal, p.window_left, p.window_right = int(bool(causal)), int(window_left), int(window_right)
    p.max_seqlen_k_known = int(max_seqlen_k_known)
    p.kv_pos_offset, p.kv_total, p.partial_out = int(kv_pos_offset), int(kv_total), int(bool(partial_out))
    p.num_splits, p.kernel, p.num_sm = int(num_splits), int(kernel), int(num_sm)
    p.softmax_scale, p.softcap = float(softmax_scale), float(softcap)
    return p


def _lse_shape(q, varlen_q):
    return (q.shape[1], q.shape[0]) if varlen_q else (q.shape[0], q.shape[2], q.shape[1])


def validate_forward(q, k, v, out, lse, kw) -> None:
    """Every check that must hold before a parameter block is built from these tensors; allocates nothing.
    ``out`` / ``lse`` may be None (the caller allocates them afterwards).  The C side only sees raw pointers and
    strides, so a wrong dtype, device, shape or layout here would become an out-of-bounds access on the GPU."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("flash_b200 runs on CUDA tensors only (there is no CPU implementation)")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError("query and key/value must have the same dtype")
    if k.device != q.device or v.device != q.device:
        raise RuntimeError("query and key/value must be on the same device")
    for name, t in (("q", q), ("k", k), ("v", v), ("k_new", kw.get("k_new")), ("v_new", kw.get("v_new"))):
        if t is not None and t.stride(-1) != 1:
            raise RuntimeError(f"Input tensor {name} must have contiguous last dimension")
    for name in ("k_new", "v_new"):
        t = kw.get(name)
        if t is not None and (t.dtype != q.dtype or t.device != q.device):
            raise RuntimeError(f"{name} must have the dtype and device of q")
    for name in ("cu_seqlens_q", "cu_seqlens_k", "seqused_k", "cache_batch_idx", "block_table"):
        _check_i32(kw.get(name), name)
    b = (kw["cu_seqlens_q"].numel() - 1) if kw.get("cu_seqlens_q") is not None else q.shape[0]
    for name in ("seqused_k", "cache_batch_idx"):
        t = kw.get(name)
        if t is not None and (t.dim() != 1 or t.numel() != b or not t.is_contiguous()):
            raise RuntimeError(f"{name} must be a contiguous int32 tensor of shape (batch_size,)")
    if kw.get("cu_seqlens_k") is not None and kw["cu_seqlens_k"].numel() != b + 1:
        raise RuntimeError("cu_seqlens_k must have shape (batch_size + 1,)")
    bt = kw.get("block_table")
    if bt is not None and (bt.dim() != 2 or bt.shape[0] != b):
        raise RuntimeError("block_table must have shape (batch_size, max_num_blocks_per_seq)")
    if kw.get("alibi_slopes") is not None:
        a = kw["alibi_slopes"]
        if a.dtype != torch.float32 or not a.is_cuda or a.stride(-1) != 1:
            raise RuntimeError("alibi_slopes must be a contiguous fp32 CUDA tensor")
        if tuple(a.shape) not in ((q.shape[-2],), (b, q.shape[-2])):
            raise RuntimeError("alibi_slopes must have shape (nheads,) or (batch_size, nheads)")
    for name in ("rotary_cos", "rotary_sin"):
        r = kw.get(name)
        if r is not None and (r.dtype != q.dtype or not r.is_contiguous() or r.device != q.device or r.dim() != 2):
            raise RuntimeError(f"{name} must be a contiguous 2-D tensor with the dtype and device of q")
    partial = bool(kw.get("partial_out", False))
    if out is not None:
        if out.shape != q.shape or out.stride(-1) != 1 or out.device != q.device:
            raise RuntimeError("out must have the shape and device of q and a contiguous last dimension")
        if out.dtype != (torch.float32 if partial else q.dtype):
            raise RuntimeError("out has the wrong dtype")
    if lse is not None:
        shape = _lse_shape(q, kw.get("cu_seqlens_q") is not None)
        if tuple(lse.shape) != shape or lse.dtype != torch.float32 or lse.device != q.device or not lse.is_contiguous():
            raise RuntimeError("lse must be a contiguous fp32 tensor of shape (b, h, s_q) / (h, total_q) on q's device")


def attention_forward(q, k, v, *, out=None, lse=None, return_plan=False, plan_bytes: Optional[bytes] = None,
                      **kw) -> Tuple[torch.Tensor, torch.Tensor]:
    """Runs the forward on the current CUDA stream.  Returns (out, lse[, plan]).

    out has q's shape (dtype of q, fp32 when partial_out); lse is fp32 (b, h, s_q), or
    (h, total_q) for varlen q.  k / v caches are mutated in place when k_new, v_new are given.
    ``out`` / ``lse`` may be given (e.g. views of one message buffer); they are allocated otherwise.
    ``plan_bytes``: a plan made ahead of the call (``encode_plan`` / get_scheduler_metadata); it is checked against
    this call's shapes and taken over where it applies (fa_b200_fwd_planned).
    """
    lib = L.load()
    validate_forward(q, k, v, out, lse, kw)
    partial = bool(kw.get("partial_out", False))
    if out is None:
        out = torch.empty(q.shape, dtype=torch.float32 if partial else q.dtype, device=q.device)
    if lse is None:
        lse = torch.empty(_lse_shape(q, kw.get("cu_seqlens_q") is not None), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        p = build_params(q, k, v, out, lse, num_sm=_num_sm(q.device), **kw)
        plan = L.FwdPlan()
        L.check(lib.fa_b200_fwd_plan(C.byref(p), C.byref(plan)))
        ws_bytes = plan.workspace_bytes
        if plan_bytes is not None:
            blob = C.create_string_buffer(bytes(plan_bytes), len(plan_bytes))
            forced = L.FwdPlan()
            L.check(lib.fa_b200_plan_decode(blob, len(plan_bytes), C.byref(forced)))
            ws_bytes = max(ws_bytes, forced.workspace_bytes)  # whichever of the two plans ends up being used
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
        stream = torch.cuda.current_stream(q.device).cuda_stream
        if plan_bytes is not None:
            L.check(lib.fa_b200_fwd_planned(C.byref(p), blob, len(plan_bytes), _ptr(ws), ws_bytes, stream))
        else:
            L.check(lib.fa_b200_fwd(C.byref(p), _ptr(ws), ws_bytes, stream))
    if return_plan:
        return out, lse, plan
    return out, lse


def attention_forward_exchange(q, k, v, exchange: "L.Exchange", *, out=None, lse=None, **kw):
    """Attention of q over this rank's shard of the keys, merged with the other ranks' shards over peer memory
    (fa_b200_fwd_exchange).  ``kw`` as for ``attention_forward`` (kv_pos_offset / kv_total place the shard in the
    sequence); returns the final (out, lse), identical on every rank."""
    lib = L.load()
    validate_forward(q, k, v, out, lse, kw)
    if kw.get("cu_seqlens_q") is not None:
        raise RuntimeError("the cross-GPU exchange takes dense (b, s_q, h, d) queries")
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty(_lse_shape(q, False), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        p = build_params(q, k, v, out, lse, num_sm=_num_sm(q.device), **kw)
        nbytes = lib.fa_b200_fwd_exchange_workspace(C.byref(p))
        if nbytes == 0:  # the plan was refused: the library holds the reason
            L.check(L.load().fa_b200_fwd_plan(C.byref(p), C.byref(L.FwdPlan())) or -1)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        L.check(lib.fa_b200_fwd_exchange(C.byref(p), _ptr(ws), nbytes, C.byref(exchange),
                                         torch.cuda.current_stream(q.device).cuda_stream))
    return out, lse


def encode_plan(p: "L.FwdParams") -> bytes:
    """Plans the problem described by ``p`` (sizes, flags and NULL-ness of the pointers; nothing is dereferenced)
    and returns the plan as FA_B200_PLAN_BYTES opaque bytes for ``attention_forward(plan_bytes=...)``."""
    lib = L.load()
    buf = C.create_string_buffer(L.PLAN_BYTES)
    L.check(lib.fa_b200_plan_encode(C.byref(p), buf, L.PLAN_BYTES))
    return buf.raw


def attention_forward_noalloc(q, k, v, out, lse, **kw) -> None:
    """Same forward as ``attention_forward`` through ``fa_b200_fwd_noalloc``: the caller passes the
    output tensors (``out`` like q, ``lse`` fp32 (b, h, s_q) or (h, total_q)) and the library
    allocates nothing -- the split-KV scratch is a fixed 32 MiB array inside the library.  Meant
    for hosts that may not touch an allocator while serving.  The tensors go through the same checks as in
    ``attention_forward`` before anything is launched.  Calls that overlap on the GPU share that scratch and
    race.  The first call on a device loads the library's device image (which holds the array) and looks up the
    array's address: make it once at start-up, outside any stream capture, before the phase in which nothing may
    be allocated."""
    lib = L.load()
    if out is None or lse is None:
        raise RuntimeError("the allocation-free entry point needs caller-provided out and lse tensors")
    validate_forward(q, k, v, out, lse, kw)
    with torch.cuda.device(q.device):
        p = build_params(q, k, v, out, lse, num_sm=_num_sm(q.device), **kw)
        L.check(lib.fa_b200_fwd_noalloc(C.byref(p), torch.cuda.current_stream(q.device).cuda_stream))


def combine(o_partial: torch.Tensor, lse_partial: torch.Tensor, out: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None, partial_out: bool = False, lse_out: Optional[torch.Tensor] = None):
    """Merge of split partials.  o_partial (n, b, s, h, d) fp32, lse_partial (n, b, s, h) fp32
    (natural log, -inf = empty partial) -> out (b, s, h, d), lse (b, s, h).  ``lse_out``: an fp32
    (b, s, h) destination of any strides (e.g. the transposed view of a (b, h, s) tensor)."""
    lib = L.load()
    if not o_partial.is_cuda:
        raise RuntimeError("flash_b200 runs on CUDA tensors only (there is no CPU implementation)")
    if o_partial.dtype != torch.float32 or lse_partial.dtype != torch.float32:
        raise RuntimeError("partials must be fp32")
    n, b, s, h, d = o_partial.shape
    if tuple(lse_partial.shape) != (n, b, s, h):
        raise RuntimeError("lse_partial must be (num_splits, batch, seqlen, nheads)")
    if o_partial.stride(-1) != 1 or d % 4 != 0:
        raise RuntimeError("o_partial needs a contiguous last dimension that is a multiple of 4")
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else torch.float32
    code = {torch.float16: L.FA_FP16, torch.bfloat16: L.FA_BF16, torch.float32: L.FA_FP32_OUT}[out_dtype]
    if out is None:
        out = torch.empty((b, s, h, d), dtype=out_dtype, device=o_partial.device)
    if lse_out is None:
        lse = torch.empty((b, s, h), dtype=torch.float32, device=o_partial.device)
    else:
        if tuple(lse_out.shape) != (b, s, h) or lse_out.dtype != torch.float32 or lse_out.device != o_partial.device:
            raise RuntimeError("lse_out must be an fp32 (batch, seqlen, nheads) tensor on the partials' device")
        lse = lse_out
    c = L.CombineParams()
    c.o_partial, c.lse_partial, c.o, c.lse = _ptr(o_partial), _ptr(lse_partial), _ptr(out), _ptr(lse)
    c.op_split_stride, c.op_batch_stride, c.op_row_stride, c.op_head_stride = o_partial.stride()[:4]
    c.lp_split_stride, c.lp_batch_stride, c.lp_row_stride, c.lp_head_stride = lse_partial.stride()
    c.o_batch_stride, c.o_row_stride, c.o_head_stride = out.stride()[:3]
    c.lse_batch_stride, c.lse_row_stride, c.lse_head_stride = lse.stride()
    c.num_splits, c.b, c.s, c.h, c.d = n, b, s, h, d
    c.out_dtype, c.partial_out = code, int(bool(partial_out))
    with torch.cuda.device(o_partial.device):
        L.check(lib.fa_b200_combine(C.byref(c), torch.cuda.current_stream(o_partial.device).cuda_stream))
    return out, lse


def attention_backward(dout, q, k, v, out, lse, *, dq=None, dk=None, dv=None, softmax_scale=None, causal=False,
                       window_left=-1, window_right=-1, softcap=0.0, cu_seqlens_q=None, cu_seqlens_k=None,
                       max_seqlen_q=None, max_seqlen_k=None, kernel=0):
    """dQ, dK, dV of ``attention_forward`` (dense (b, s, h, d) or packed varlen (total, h, d) tensors) from
    the forward's ``out`` and ``lse``.  Head dim a multiple of 8, at most 256; no dropout / alibi.
    ``kernel``: 0 automatic (tcgen05 kernels for head dims up to 128), 1 the mma.sync kernel, 2 tcgen05."""
    lib = L.load()
    ts = (dout, q, k, v, out)
    if not all(t.is_cuda for t in ts) or not lse.is_cuda:
        raise RuntimeError("flash_b200 runs on CUDA tensors only (there is no CPU implementation)")
    if any(t.dtype != q.dtype for t in ts):
        raise RuntimeError("dout, q, k, v and out must have the same dtype")
    if lse.dtype != torch.float32 or not lse.is_contiguous():
        raise RuntimeError("softmax_lse must be a contiguous fp32 tensor")
    dout, q, k, v, out = [t if t.stride(-1) == 1 else t.contiguous() for t in ts]
    varlen = cu_seqlens_q is not None
    _check_i32(cu_seqlens_q, "cu_seqlens_q")
    _check_i32(cu_seqlens_k, "cu_seqlens_k")
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    for name, t, ref in (("dq", dq, q), ("dk", dk, k), ("dv", dv, v)):
        if t.shape != ref.shape or t.dtype != ref.dtype or t.stride(-1) != 1 or not t.is_cuda:
            raise RuntimeError(f"{name} must have the shape, dtype and device of its input and a contiguous last dimension")
    p = L.BwdParams()
    p.q, p.k, p.v, p.o, p.dout, p.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(dout), _ptr(lse)
    p.dq, p.dk, p.dv = _ptr(dq), _ptr(dk), _ptr(dv)
    p.cu_seqlens_q, p.cu_seqlens_k = _ptr(cu_seqlens_q), _ptr(cu_seqlens_k)
    for name, t in (("q", q), ("k", k), ("v", v), ("o", out), ("do", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
        if varlen:
            bs, rs, hs = 0, t.stride(0), t.stride(1)
        else:
            bs, rs, hs = t.stride(0), t.stride(1), t.stride(2)
        setattr(p, f"{name}_batch_stride", bs)
        setattr(p, f"{name}_row_stride", rs)
        setattr(p, f"{name}_head_stride", hs)
    if varlen:
        if cu_seqlens_k is None or max_seqlen_q is None or max_seqlen_k is None:
            raise RuntimeError("varlen backward needs cu_seqlens_k, max_seqlen_q and max_seqlen_k")
        total_q, h, d = q.shape
        h_k = k.shape[1]
        p.b, p.seqlen_q, p.seqlen_k, p.total_q = cu_seqlens_q.numel() - 1, int(max_seqlen_q), int(max_seqlen_k), total_q
        p.total_k = k.shape[0]
        p.lse_batch_stride, p.lse_head_stride = 0, lse.stride(0)
        if tuple(lse.shape) != (h, total_q):
            raise RuntimeError("softmax_lse must be (nheads, total_q)")
    else:
        b, s_q, h, d = q.shape
        h_k = k.shape[2]
        p.b, p.seqlen_q, p.seqlen_k, p.total_q = b, s_q, k.shape[1], b * s_q
        p.lse_batch_stride, p.lse_head_stride = lse.stride(0), lse.stride(1)
        if tuple(lse.shape) != (b, h, s_q):
            raise RuntimeError("softmax_lse must be (batch, nheads, seqlen_q)")
    p.h, p.h_k, p.d = h, h_k, d
    p.dtype, p.causal = _dtype_code(q), int(bool(causal))
    p.window_left, p.window_right = int(window_left), int(window_right)
    p.softmax_scale = float(softmax_scale if softmax_scale is not None else d ** -0.5)
    p.softcap = float(softcap)
    p.kernel = int(kernel)
    with torch.cuda.device(q.device):
        nbytes = lib.fa_b200_bwd_workspace_bytes(C.byref(p))
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
        L.check(lib.fa_b200_bwd(C.byref(p), _ptr(ws), nbytes, torch.cuda.current_stream(q.device).cuda_stream))
    return dq, dk, dv
