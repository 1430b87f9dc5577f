"""ctypes binding of libfa_b200.so (the C ABI declared in include/fa_b200.h).

The library is loaded from the package directory; there is no fallback of any kind:
if the shared object is missing the import raises, so a GPU box can never silently
run something else.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libfa_b200.so")

FA_OK = 0
FA_FP16, FA_BF16, FA_FP32_OUT = 0, 1, 2
KERNEL_AUTO, KERNEL_MMA, KERNEL_TCGEN05, KERNEL_DECODE = 0, 1, 2, 3

_p = C.c_void_p
_i64 = C.c_int64
_i32 = C.c_int32


class FwdParams(C.Structure):
    """Mirror of ``fa_fwd_params`` (include/fa_b200.h); field order is the ABI."""
    _fields_ = (
        [(n, _p) for n in (
            "q", "k", "v", "o", "lse", "k_new", "v_new", "cu_seqlens_q", "cu_seqlens_k", "seqused_k",
            "cache_batch_idx", "block_table", "rotary_cos", "rotary_sin", "alibi_slopes")]
        + [(n, _i64) for n in (
            "q_batch_stride", "q_row_stride", "q_head_stride",
            "k_batch_stride", "k_row_stride", "k_head_stride",
            "v_batch_stride", "v_row_stride", "v_head_stride",
            "o_batch_stride", "o_row_stride", "o_head_stride",
            "knew_batch_stride", "knew_row_stride", "knew_head_stride",
            "vnew_batch_stride", "vnew_row_stride", "vnew_head_stride",
            "lse_batch_stride", "lse_head_stride",
            "block_table_batch_stride", "alibi_batch_stride")]
        + [(n, _i32) for n in (
            "b", "seqlen_q", "seqlen_k", "h", "h_k", "d", "total_q", "seqlen_new", "page_size",
            "rotary_dim", "rotary_seqlen", "rotary_interleaved", "dtype",
            "causal", "window_left", "window_right", "max_seqlen_k_known",
            "kv_pos_offset", "kv_total", "partial_out",
            "num_splits", "kernel", "num_sm", "total_k", "kv_outer")]
        + [("softmax_scale", C.c_float), ("softcap", C.c_float)]
    )


class FwdPlan(C.Structure):
    """Mirror of ``fa_fwd_plan``."""
    _fields_ = [(n, _i32) for n in (
        "kernel", "config", "pack_gqa", "block_m", "block_n", "m_blocks", "num_splits", "blocks_per_split",
        "grid", "threads", "smem_bytes", "is_causal", "is_local", "window_left", "window_right", "launches")] + [
        ("workspace_bytes", C.c_size_t)]


class CombineParams(C.Structure):
    """Mirror of ``fa_combine_params``."""
    _fields_ = (
        [(n, _p) for n in ("o_partial", "lse_partial", "o", "lse")]
        + [(n, _i64) for n in (
            "op_split_stride", "op_batch_stride", "op_row_stride", "op_head_stride",
            "lp_split_stride", "lp_batch_stride", "lp_row_stride", "lp_head_stride",
            "o_batch_stride", "o_row_stride", "o_head_stride",
            "lse_batch_stride", "lse_row_stride", "lse_head_stride")]
        + [(n, _i32) for n in ("num_splits", "b", "s", "h", "d", "out_dtype", "partial_out")]
    )


class BwdParams(C.Structure):
    """Mirror of ``fa_bwd_params``."""
    _fields_ = (
        [(n, _p) for n in ("q", "k", "v", "o", "dout", "lse", "dq", "dk", "dv", "cu_seqlens_q", "cu_seqlens_k")]
        + [(f"{t}_{s}_stride", _i64) for t in ("q", "k", "v", "o", "do", "dq", "dk", "dv") for s in ("batch", "row", "head")]
        + [("lse_batch_stride", _i64), ("lse_head_stride", _i64)]
        + [(n, _i32) for n in ("b", "seqlen_q", "seqlen_k", "h", "h_k", "d", "total_q", "dtype", "causal",
                               "window_left", "window_right")]
        + [("softmax_scale", C.c_float), ("softcap", C.c_float), ("total_k", _i32), ("kernel", _i32)]
    )


MAX_RANKS = 16  # FA_B200_MAX_RANKS


class Exchange(C.Structure):
    """Mirror of ``fa_exchange``."""
    _fields_ = [("bufs", _p * MAX_RANKS), ("buf_bytes", C.c_size_t), ("world", _i32), ("rank", _i32),
                ("timeout_cycles", _i64)]


# every symbol include/fa_b200.h declares
EXPORTS = (
    "fa_b200_fwd", "fa_b200_fwd_noalloc", "fa_b200_fwd_plan", "fa_b200_combine", "fa_b200_normalize_window",
    "fa_b200_check_status", "fa_b200_last_error", "fa_b200_status_string", "fa_b200_abi_version",
    "fa_b200_launch_count", "fa_b200_bwd", "fa_b200_bwd_workspace_bytes",
    "fa_b200_plan_encode", "fa_b200_plan_decode", "fa_b200_fwd_planned",
    "fa_b200_exchange_bytes", "fa_b200_exchange_alloc", "fa_b200_exchange_open", "fa_b200_exchange_close",
    "fa_b200_exchange_free", "fa_b200_fwd_exchange_workspace", "fa_b200_fwd_exchange",
)
PLAN_BYTES = 192  # FA_B200_PLAN_BYTES

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python flash-attention-npu_b200/build.py` "
            "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    lib.fa_b200_fwd.argtypes = [C.POINTER(FwdParams), _p, C.c_size_t, _p]
    lib.fa_b200_fwd.restype = C.c_int
    lib.fa_b200_fwd_noalloc.argtypes = [C.POINTER(FwdParams), _p]
    lib.fa_b200_fwd_noalloc.restype = C.c_int
    lib.fa_b200_fwd_plan.argtypes = [C.POINTER(FwdParams), C.POINTER(FwdPlan)]
    lib.fa_b200_fwd_plan.restype = C.c_int
    lib.fa_b200_plan_encode.argtypes = [C.POINTER(FwdParams), _p, C.c_size_t]
    lib.fa_b200_plan_encode.restype = C.c_int
    lib.fa_b200_plan_decode.argtypes = [_p, C.c_size_t, C.POINTER(FwdPlan)]
    lib.fa_b200_plan_decode.restype = C.c_int
    lib.fa_b200_fwd_planned.argtypes = [C.POINTER(FwdParams), _p, C.c_size_t, _p, C.c_size_t, _p]
    lib.fa_b200_fwd_planned.restype = C.c_int
    lib.fa_b200_exchange_bytes.argtypes = [_i32, _i64, _i32]
    lib.fa_b200_exchange_bytes.restype = C.c_size_t
    lib.fa_b200_exchange_alloc.argtypes = [C.c_size_t, C.POINTER(_p), _p]
    lib.fa_b200_exchange_alloc.restype = C.c_int
    lib.fa_b200_exchange_open.argtypes = [_p, C.POINTER(_p)]
    lib.fa_b200_exchange_open.restype = C.c_int
    lib.fa_b200_exchange_close.argtypes = [_p]
    lib.fa_b200_exchange_close.restype = C.c_int
    lib.fa_b200_exchange_free.argtypes = [_p]
    lib.fa_b200_exchange_free.restype = C.c_int
    lib.fa_b200_fwd_exchange_workspace.argtypes = [C.POINTER(FwdParams)]
    lib.fa_b200_fwd_exchange_workspace.restype = C.c_size_t
    lib.fa_b200_fwd_exchange.argtypes = [C.POINTER(FwdParams), _p, C.c_size_t, C.POINTER(Exchange), _p]
    lib.fa_b200_fwd_exchange.restype = C.c_int
    lib.fa_b200_bwd.argtypes = [C.POINTER(BwdParams), _p, C.c_size_t, _p]
    lib.fa_b200_bwd.restype = C.c_int
    lib.fa_b200_bwd_workspace_bytes.argtypes = [C.POINTER(BwdParams)]
    lib.fa_b200_bwd_workspace_bytes.restype = C.c_size_t
    lib.fa_b200_combine.argtypes = [C.POINTER(CombineParams), _p]
    lib.fa_b200_combine.restype = C.c_int
    lib.fa_b200_normalize_window.argtypes = [_i32, _i32, _i32] + [C.POINTER(_i32)] * 4
    lib.fa_b200_normalize_window.restype = C.c_int
    lib.fa_b200_check_status.argtypes = [_p]
    lib.fa_b200_check_status.restype = C.c_int
    lib.fa_b200_last_error.restype = C.c_char_p
    lib.fa_b200_status_string.argtypes = [C.c_int]
    lib.fa_b200_status_string.restype = C.c_char_p
    lib.fa_b200_abi_version.restype = C.c_int
    lib.fa_b200_launch_count.restype = C.c_longlong
    lib.fa_b200_launch_count.argtypes = []
    if lib.fa_b200_abi_version() != 2:
        raise ImportError("libfa_b200.so ABI version mismatch")
    _lib = lib
    return lib


def check(status: int) -> None:
    """Non-zero status -> RuntimeError, the error convention of the reference's TORCH_CHECK."""
    if status != FA_OK:
        lib = load()
        msg = lib.fa_b200_last_error().decode() or lib.fa_b200_status_string(status).decode()
        raise RuntimeError(msg)


def normalize_window(seqlen_q: int, max_seqlen_k: int, causal: bool, wl: int, wr: int):
    """Host-only; returns (is_causal, is_local, wl, wr)."""
    lib = load()
    a, b, c, d = _i32(wl), _i32(wr), _i32(0), _i32(0)
    check(lib.fa_b200_normalize_window(seqlen_q, max_seqlen_k, int(bool(causal)), C.byref(a), C.byref(b),
                                       C.byref(c), C.byref(d)))
    return bool(c.value), bool(d.value), a.value, b.value
