"""CPU: the C-ABI library loads, exports every symbol include/fa_b200.h declares, and its
host-only entry points (window normalisation, planning, argument validation) behave like the
reference's host code.  No kernel is launched here."""
import ctypes as C
import os
import re

import pytest

from flash_b200 import lib as L
from oracle import golden as OG

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    header = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    declared = set(re.findall(r"\b(fa_b200_\w+)\s*\(", header))
    assert declared == set(L.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fa_b200_abi_version() == 2
    assert lib.fa_b200_status_string(-4).decode().startswith("workspace")


def test_struct_layout_matches_header():
    # sizes produced by gcc for include/fa_b200.h (x86-64 LP64)
    assert C.sizeof(L.FwdParams) == 408
    assert C.sizeof(L.FwdPlan) == 72
    assert C.sizeof(L.CombineParams) == 176
    assert C.sizeof(L.BwdParams) == 360
    assert C.sizeof(L.Exchange) == 152


@pytest.mark.parametrize("sq,mk,causal,wl,wr", [
    (64, 192, False, 32, 64), (1024, 1024, True, 512, 256), (1024, 1024, True, -128, 864),
    (512, 512, False, 508, -256), (128, 512, True, 511, 0), (4, 100, False, -1, -1), (1, 1024, True, 512, 0),
    (4, 32768, True, 4096, 0), (2, 1024, True, 256, 0), (128, 256, True, 127, 0)])
def test_window_normalisation_matches_oracle(sq, mk, causal, wl, wr):
    assert L.normalize_window(sq, mk, causal, wl, wr) == OG.normalize_window(sq, mk, causal, wl, wr)


def _params(**kw):
    p = L.FwdParams()
    p.q = p.k = p.v = p.o = p.lse = 256
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d = 2, 1, 4096, 32, 8, 128
    p.total_q = 2
    p.lse_batch_stride, p.lse_head_stride = 32, 1
    p.dtype, p.num_sm, p.softmax_scale = L.FA_BF16, 148, 0.088
    p.max_seqlen_k_known = -1
    p.window_left = p.window_right = -1
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def _plan(p):
    pl = L.FwdPlan()
    rc = L.load().fa_b200_fwd_plan(C.byref(p), C.byref(pl))
    return rc, pl


def test_plan_decode_packs_gqa_and_splits():
    rc, pl = _plan(_params(seqused_k=256))
    assert rc == 0
    assert pl.pack_gqa == 1 and pl.block_m == 16 and pl.block_n == 64 and pl.m_blocks == 1
    assert pl.num_splits > 1 and pl.launches == 2
    assert pl.blocks_per_split * pl.num_splits >= 64
    assert pl.grid == 2 * 8 * pl.num_splits
    assert pl.workspace_bytes >= pl.num_splits * 2 * 32 * (128 + 1) * 4
    rc, pl1 = _plan(_params(seqused_k=256, num_splits=1))
    assert rc == 0 and pl1.num_splits == 1 and pl1.workspace_bytes == 0 and pl1.launches == 1


def test_plan_window_bounds_the_kv_range():
    p = _params(seqused_k=256, block_table=256, page_size=256, kv_outer=4096, seqlen_k=32768, seqlen_q=4, total_q=8,
                lse_head_stride=4, lse_batch_stride=128, causal=1, window_left=4096, window_right=0, h=64)
    rc, pl = _plan(p)
    assert rc == 0 and pl.is_local == 1 and pl.window_left == 4096 and pl.window_right == 0
    assert pl.block_m == 32  # 4 query tokens x 8 packed heads
    assert pl.num_splits * pl.blocks_per_split * pl.block_n <= 4096 + 4 + 3 * 128


@pytest.mark.parametrize("kw,msg", [
    (dict(h=30), "Number of heads"), (dict(d=264), "at most 256"), (dict(d=100), "multiple of 8"),
    (dict(dtype=7), "FP16 and BF16"), (dict(b=0), "batch size"), (dict(softcap=-1.0), "softcap"),
    (dict(k_new=256), "together"), (dict(k_new=256, v_new=256, seqlen_new=1), "cache_seqlens"),
    (dict(block_table=256, page_size=16, kv_outer=8), "key lengths"),
    (dict(block_table=256, page_size=128, seqused_k=256), "kv_outer"),            # paged: the page count is required
    (dict(cache_batch_idx=256, seqused_k=256), "kv_outer"),                       # ... and the cache rows with an index
    (dict(block_table=256, page_size=128, seqused_k=256, kv_outer=-3), "kv_outer"),
    (dict(seqused_k=256, k_new=256, v_new=256, seqlen_new=5000), "do not fit"),   # more new tokens than the cache holds
    (dict(rotary_cos=256, rotary_sin=256, rotary_dim=64), "together with new k"),
    (dict(kernel=L.KERNEL_TCGEN05, seqused_k=256), "tcgen05"),
])
def test_plan_rejects_bad_arguments(kw, msg):
    rc, _ = _plan(_params(**kw))
    assert rc != 0
    assert msg in L.load().fa_b200_last_error().decode()
    with pytest.raises(RuntimeError, match=msg):
        L.check(rc)


def test_python_modules_expose_reference_signatures():
    import inspect

    import flash_attn_npu_v2 as v2
    import flash_attn_npu_v3 as v3
    assert v2.__version__ == "0.1.1" and v3.__version__ == "0.1.1"
    sig = inspect.signature(v2.flash_attn_with_kvcache)
    assert list(sig.parameters) == ["q", "k_cache", "v_cache", "k", "v", "rotary_cos", "rotary_sin", "cache_seqlens",
                                    "cache_batch_idx", "cache_leftpad", "block_table", "softmax_scale", "causal",
                                    "window_size", "softcap", "rotary_interleaved", "alibi_slopes", "num_splits",
                                    "return_softmax_lse"]
    assert sig.parameters["rotary_interleaved"].default is True and sig.parameters["num_splits"].default == 0
    sig = inspect.signature(v2.flash_attn_func)
    assert list(sig.parameters) == ["q", "k", "v", "dropout_p", "softmax_scale", "causal", "window_size", "softcap",
                                    "alibi_slopes", "deterministic", "return_attn_probs"]
    sig = inspect.signature(v3.flash_attn_with_kvcache)
    assert list(sig.parameters)[:12] == ["q", "k_cache", "v_cache", "k", "v", "qv", "rotary_cos", "rotary_sin",
                                         "cache_seqlens", "cache_batch_idx", "cache_leftpad", "page_table"]
    sig = inspect.signature(v3.flash_attn_func)
    assert sig.parameters["num_splits"].default == 1
    for name in ("flash_attn_func", "flash_attn_varlen_func", "flash_attn_with_kvcache", "get_scheduler_metadata"):
        assert hasattr(v3, name)


def test_cpu_tensors_are_refused():
    import torch

    import flash_attn_npu_v2 as v2
    q = torch.zeros(1, 1, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        v2.flash_attn_func(q, q, q)


def test_plan_varlen_prefill_needs_total_k_for_the_tcgen05_kernel():
    """Packed varlen input goes to the tcgen05 kernel only when the number of k / v rows is known (its TMA
    descriptors need the bound); otherwise to the general kernel."""
    kw = dict(b=3, seqlen_q=512, seqlen_k=640, h=8, h_k=2, d=128, total_q=1300, cu_seqlens_q=256, cu_seqlens_k=256,
              q_row_stride=1024, q_head_stride=128, k_row_stride=256, k_head_stride=128, v_row_stride=256,
              v_head_stride=128, o_row_stride=1024, o_head_stride=128, lse_batch_stride=0, lse_head_stride=1300, causal=1)
    rc, pl = _plan(_params(total_k=1500, **kw))
    assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05 and pl.block_m == 256 and pl.grid == min(148, 2 * 3 * 8)
    rc, pl = _plan(_params(total_k=0, **kw))
    assert rc == 0 and pl.kernel == L.KERNEL_MMA


def test_plan_persistent_decode_for_ragged_lengths_only():
    """Ragged cache lengths (a device-side length vector) with enough work: resident CTAs with equal shares and a
    fixed number of partial slots.  Window-bound ranges and explicit split requests keep the plain grid."""
    kw = dict(b=64, seqlen_q=1, seqlen_k=8192, h=32, h_k=8, d=128, total_q=64, seqused_k=256,
              q_batch_stride=4096, q_row_stride=4096, q_head_stride=128,
              k_batch_stride=8192 * 1024, k_row_stride=1024, k_head_stride=128,
              v_batch_stride=8192 * 1024, v_row_stride=1024, v_head_stride=128,
              o_batch_stride=4096, o_row_stride=4096, o_head_stride=128, lse_batch_stride=32, lse_head_stride=1, causal=1)
    rc, pl = _plan(_params(**kw))
    assert rc == 0 and pl.kernel == L.KERNEL_DECODE
    assert pl.num_splits == 4 and pl.grid in (148, 296) and pl.launches == 2 and pl.workspace_bytes > 0
    rc, pl = _plan(_params(num_splits=2, **kw))
    assert rc == 0 and pl.num_splits == 2 and pl.grid == 64 * 8 * 2
    rc, pl = _plan(_params(window_left=1024, window_right=0, **kw))
    assert rc == 0 and pl.kernel == L.KERNEL_DECODE and pl.grid % (64 * 8) == 0  # plain grid: units x splits


def test_plan_32_row_decode_configuration_follows_the_key_range():
    """17-32 packed rows: short key ranges (a sliding window) run two resident CTAs of 2x2 consumer warps with
    64-key blocks (one launch, no partials); long ranges and ragged launches that become persistent keep the
    single CTA of 2x4 warps with 128-key blocks."""
    kw = dict(b=32, seqlen_q=4, seqlen_k=32768, h=64, h_k=8, d=128, total_q=128, seqused_k=256,
              block_table=256, page_size=256, kv_outer=4096, block_table_batch_stride=128,
              q_batch_stride=4 * 8192, q_row_stride=8192, q_head_stride=128,
              k_batch_stride=256 * 1024, k_row_stride=1024, k_head_stride=128,
              v_batch_stride=256 * 1024, v_row_stride=1024, v_head_stride=128,
              o_batch_stride=4 * 8192, o_row_stride=8192, o_head_stride=128, lse_batch_stride=256, lse_head_stride=4, causal=1)
    rc, pl = _plan(_params(window_left=4096, window_right=0, **kw))
    assert rc == 0 and pl.kernel == L.KERNEL_DECODE and pl.block_m == 32
    assert pl.config == 11 and pl.block_n == 64 and pl.threads == 160 and 2 * pl.smem_bytes <= 227 * 1024
    assert pl.num_splits == 1 and pl.grid == 32 * 8 and pl.launches == 1
    rc, pl = _plan(_params(**kw))  # ragged, no window: persistent, 128-key blocks
    assert rc == 0 and pl.kernel == L.KERNEL_DECODE and pl.config == 5 and pl.block_n == 128 and pl.num_splits == 4
    kw.pop("seqused_k"), kw.pop("block_table"), kw.pop("page_size"), kw.pop("block_table_batch_stride")
    kw.update(k_batch_stride=32768 * 1024, v_batch_stride=32768 * 1024)
    rc, pl = _plan(_params(**kw))  # uniform long range: 128-key blocks, split over the keys
    assert rc == 0 and pl.kernel == L.KERNEL_DECODE and pl.config == 5 and pl.block_n == 128


def test_plan_prefill_against_a_cache_goes_to_the_tcgen05_kernel():
    """Many query tokens against a KV cache with per-entry lengths: tcgen05 kernel for contiguous caches and for
    pages that hold whole 128-key blocks; new tokens add a prologue launch and, with rotary, a workspace for the
    rotated q; alibi and small pages stay on the general kernel."""
    kw = dict(b=4, seqlen_q=512, seqlen_k=8192, h=32, h_k=8, d=128, total_q=2048, seqused_k=256,
              q_batch_stride=512 * 4096, q_row_stride=4096, q_head_stride=128,
              k_batch_stride=8192 * 1024, k_row_stride=1024, k_head_stride=128,
              v_batch_stride=8192 * 1024, v_row_stride=1024, v_head_stride=128,
              o_batch_stride=512 * 4096, o_row_stride=4096, o_head_stride=128, lse_batch_stride=32 * 512, lse_head_stride=512,
              causal=1)
    rc, pl = _plan(_params(**kw))
    assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05 and pl.launches == 1 and pl.workspace_bytes == 0
    paged = dict(kw, block_table=256, page_size=256, kv_outer=64, block_table_batch_stride=32,
                 k_batch_stride=256 * 1024, v_batch_stride=256 * 1024)
    rc, pl = _plan(_params(**paged))
    assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05 and pl.launches == 1
    rc, pl = _plan(_params(**dict(paged, page_size=64, k_batch_stride=64 * 1024, v_batch_stride=64 * 1024,
                                  block_table_batch_stride=128)))
    assert rc == 0 and pl.kernel == L.KERNEL_MMA
    new = dict(k_new=256, v_new=256, seqlen_new=512, knew_batch_stride=512 * 1024, knew_row_stride=1024, knew_head_stride=128,
               vnew_batch_stride=512 * 1024, vnew_row_stride=1024, vnew_head_stride=128)
    rc, pl = _plan(_params(**dict(paged, **new)))
    assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05 and pl.launches == 2 and pl.workspace_bytes == 0
    rc, pl = _plan(_params(**dict(paged, rotary_cos=256, rotary_sin=256, rotary_dim=128, rotary_seqlen=9000, **new)))
    assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05 and pl.launches == 2
    assert pl.workspace_bytes == 4 * 512 * 32 * 128 * 2
    rc, pl = _plan(_params(**dict(kw, cache_batch_idx=256, kv_outer=7)))
    assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05
    rc, pl = _plan(_params(**dict(kw, alibi_slopes=256)))
    assert rc == 0 and pl.kernel == L.KERNEL_MMA


def _bwd_params(**kw):
    p = L.BwdParams()
    for name in ("q", "k", "v", "o", "dout", "lse", "dq", "dk", "dv"):
        setattr(p, name, 256)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d, p.total_q = 2, 512, 512, 8, 2, 128, 1024
    for t, heads in (("q", 8), ("k", 2), ("v", 2), ("o", 8), ("do", 8), ("dq", 8), ("dk", 2), ("dv", 2)):
        setattr(p, f"{t}_batch_stride", 512 * heads * 128)
        setattr(p, f"{t}_row_stride", heads * 128)
        setattr(p, f"{t}_head_stride", 128)
    p.lse_batch_stride, p.lse_head_stride = 8 * 512, 512
    p.dtype, p.softmax_scale = L.FA_BF16, 0.088
    p.window_left = p.window_right = -1
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_backward_workspace_and_kernel_choice():
    """The tcgen05 backward (head dims up to 128; packed input only with the number of k / v rows) needs the rowsum
    and 16 bytes of counters; the mma.sync kernel needs its fp32 dQ accumulator as well.  A forced kernel that does not
    cover the problem is refused before anything is launched (the pointers here are never dereferenced)."""
    lib = L.load()
    rows, h = 2 * 512, 8
    delta = rows * h * 4
    assert lib.fa_b200_bwd_workspace_bytes(C.byref(_bwd_params())) == 16 + delta
    assert lib.fa_b200_bwd_workspace_bytes(C.byref(_bwd_params(softcap=30.0, d=64))) == 16 + delta
    assert lib.fa_b200_bwd_workspace_bytes(C.byref(_bwd_params(kernel=1))) == rows * h * 128 * 4 + delta
    assert lib.fa_b200_bwd_workspace_bytes(C.byref(_bwd_params(d=256))) == rows * h * 256 * 4 + delta
    packed = dict(cu_seqlens_q=256, cu_seqlens_k=256, lse_batch_stride=0, lse_head_stride=1024)
    assert lib.fa_b200_bwd_workspace_bytes(C.byref(_bwd_params(total_k=1024, **packed))) == 16 + delta
    assert lib.fa_b200_bwd_workspace_bytes(C.byref(_bwd_params(total_k=0, **packed))) == rows * h * 128 * 4 + delta
    for kw, msg in ((dict(kernel=2, d=256), "tcgen05 backward covers"), (dict(kernel=5), "kernel must be"),
                    (dict(h_k=3), "must divide"), (dict(d=100), "multiple of 8")):
        p = _bwd_params(**kw)
        rc = lib.fa_b200_bwd(C.byref(p), 4096, 1 << 40, None)
        assert rc != 0 and msg in lib.fa_b200_last_error().decode(), (kw, lib.fa_b200_last_error())


def test_plan_tcgen05_prefill_covers_head_dims_up_to_256_and_softcap():
    """Dense prefill with at least 128 query rows goes to the tcgen05 kernel for every head dim up to 256 that is a
    multiple of 8, with or without softcap; above 128 the CTA tile is 128 rows (one sub-tile), otherwise 256.  Alibi and
    fewer than 128 query rows stay on the general kernel."""
    def dense(d, sq=1024, **kw):
        h, hk = 8, 2
        return _params(b=2, seqlen_q=sq, seqlen_k=1024, h=h, h_k=hk, d=d, total_q=2 * sq, causal=1,
                       q_batch_stride=sq * h * d, q_row_stride=h * d, q_head_stride=d,
                       k_batch_stride=1024 * hk * d, k_row_stride=hk * d, k_head_stride=d,
                       v_batch_stride=1024 * hk * d, v_row_stride=hk * d, v_head_stride=d,
                       o_batch_stride=sq * h * d, o_row_stride=h * d, o_head_stride=d,
                       lse_batch_stride=h * sq, lse_head_stride=sq, **kw)
    for d, rows in ((8, 256), (40, 256), (64, 256), (96, 256), (128, 256), (136, 128), (192, 128), (256, 128)):
        rc, pl = _plan(dense(d))
        assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05 and pl.block_m == rows and pl.block_n == 128, (d, pl.kernel, pl.block_m)
        assert pl.m_blocks == -(-1024 // rows) and pl.num_splits == 1 and pl.workspace_bytes == 0
        rc, pl = _plan(dense(d, softcap=30.0))
        assert rc == 0 and pl.kernel == L.KERNEL_TCGEN05
    rc, pl = _plan(dense(128, alibi_slopes=256))
    assert rc == 0 and pl.kernel == L.KERNEL_MMA
    rc, pl = _plan(dense(128, sq=100))
    assert rc == 0 and pl.kernel == L.KERNEL_MMA
    rc, pl = _plan(dense(128, kernel=L.KERNEL_TCGEN05, sq=100))
    assert rc != 0  # forced, but the problem is not covered
