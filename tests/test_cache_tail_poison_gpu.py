"""GPU: memory a call may not use is filled with NaN and the results must not notice.

A KV cache is normally allocated once (``torch.empty``) and filled as the sequences grow, so the rows behind
``cache_seqlens`` (+ the appended tokens), the tails of the last pages and the pages or cache rows nobody owns
hold arbitrary bits.  The mask gives those keys the probability 0, but 0 x NaN is NaN inside a matrix product, so
every kernel has to keep such rows out of P.V by clearing them on the way in.  The reference copies only the valid
rows of a page (csrc/arch22/flash_attn_npu_v2/pv_matmul.hpp:137-142,188-206); its golden gathers ``cache_seqlens``
rows per sequence (tests/test_flash_attn_npu_v2.py:350-376), which is what the oracle does too, so the poison never
reaches the expected values.  Each case runs on the kernel family named in its id: the tcgen05 prefill kernel,
the producer / consumer decode kernel and the register-accumulator kernel.
"""
import pytest
import torch

import parity_util as U
from flash_b200 import lib as L
from flash_b200 import ops
from oracle import api as OA

pytestmark = pytest.mark.gpu
BF, FP = torch.bfloat16, torch.float16
NAN = float("nan")


def _poisoned_cache(g, dtype, b, s_cache, hk, d, lens, s_new, page, extra_rows=0):
    """Cache with valid data in rows [0, lens[i]) of sequence i and NaN everywhere else.  ``page`` > 0: a page pool
    with a permuted block table and two pages nobody owns (all NaN).  ``extra_rows`` > 0: a contiguous cache with
    that many more rows than the batch (all NaN) addressed through cache_batch_idx."""
    kc, vc = U.normal((b, s_cache, hk, d), dtype, g), U.normal((b, s_cache, hk, d), dtype, g)
    for i, n in enumerate(lens.tolist()):
        kc[i, n:] = NAN
        vc[i, n:] = NAN
    bt = idx = None
    if page:
        per = s_cache // page
        nblk = b * per + 2
        perm = torch.randperm(nblk, generator=g)[:b * per]
        bt = perm.view(b, per).to(torch.int32)
        pool_k = torch.full((nblk, page, hk, d), NAN, dtype=dtype)
        pool_v = torch.full((nblk, page, hk, d), NAN, dtype=dtype)
        pool_k[perm] = kc.view(-1, page, hk, d)
        pool_v[perm] = vc.view(-1, page, hk, d)
        kc, vc = pool_k, pool_v
    elif extra_rows:
        rows = torch.randperm(b + extra_rows, generator=g)[:b]
        idx = rows.to(torch.int32)
        big_k = torch.full((b + extra_rows, s_cache, hk, d), NAN, dtype=dtype)
        big_v = torch.full((b + extra_rows, s_cache, hk, d), NAN, dtype=dtype)
        big_k[rows] = kc
        big_v[rows] = vc
        kc, vc = big_k, big_v
    return kc, vc, bt, idx


def _check(q, kc, vc, kn, vn, lens, bt, idx, kernel, tag, causal=True, window=(-1, -1), cos=None, sin=None):
    kc_o, vc_o = kc.clone(), vc.clone()
    go, gl = OA.flash_attn_with_kvcache(q, kc_o, vc_o, kn, vn, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens,
                                        cache_batch_idx=idx, block_table=bt, causal=causal, window_size=window,
                                        rotary_interleaved=False)
    assert torch.isfinite(go.float()).all(), "the oracle itself must not see the poison"
    c = lambda t: None if t is None else t.cuda()
    kc_g, vc_g = kc.cuda(), vc.cuda()
    out, lse, plan = ops.attention_forward(
        c(q), kc_g, vc_g, k_new=c(kn), v_new=c(vn), seqused_k=c(lens), cache_batch_idx=c(idx), block_table=c(bt),
        rotary_cos=c(cos), rotary_sin=c(sin), rotary_interleaved=False, softmax_scale=q.shape[-1] ** -0.5,
        causal=causal, window_left=window[0], window_right=window[1], return_plan=True)
    torch.cuda.synchronize()
    assert plan.kernel == kernel, f"{tag}: ran on kernel {plan.kernel}, expected {kernel}"
    assert torch.isfinite(out.float()).all(), f"{tag}: NaN / Inf leaked from memory the call does not own"
    U.check_rules(out, lse, go, gl, tag=tag)
    # the cache afterwards: appended rows bit-exact, every poisoned row still poisoned (NaN payload bits included)
    assert torch.equal(kc_g.cpu().view(torch.int16), kc_o.view(torch.int16)), f"{tag}: k_cache differs"
    assert torch.equal(vc_g.cpu().view(torch.int16), vc_o.view(torch.int16)), f"{tag}: v_cache differs"
    assert L.load().fa_b200_check_status(torch.cuda.current_stream().cuda_stream) == 0


@pytest.mark.parametrize("append", [False, True], ids=["read", "append"])
@pytest.mark.parametrize("layout,d", [("contiguous", 128), ("page128", 128), ("page256", 128), ("batch_idx", 128),
                                      ("contiguous", 64), ("page128", 64), ("contiguous", 256), ("page256", 192)])
def test_tcgen05_prefill_ignores_the_cache_tail(layout, d, append):
    """Chunked prefill (200 query tokens) against a cache: lengths that end inside a 128-key block, exactly on a
    block boundary, inside a page, an empty entry, a full cache; every tile width of the kernel."""
    g = torch.Generator().manual_seed(4100 + len(layout) + append)
    b, s_q, h, hk, s_cache = 6, 200, 8, 2, 1536
    s_new = s_q if append else 0
    lens = torch.tensor([333, 1024, 77, 0, s_cache - s_new, 1281 - s_new if append else 1281], dtype=torch.int32)
    page = {"page128": 128, "page256": 256}.get(layout, 0)
    kc, vc, bt, idx = _poisoned_cache(g, BF, b, s_cache, hk, d, lens, s_new, page, extra_rows=3 if layout == "batch_idx" else 0)
    q = U.normal((b, s_q, h, d), BF, g)
    kn = vn = cos = sin = None
    if append:
        kn, vn = U.normal((b, s_new, hk, d), BF, g), U.normal((b, s_new, hk, d), BF, g)
        cos, sin = U.rotary_tables(s_cache + 8, d // 2, BF)
    _check(q, kc, vc, kn, vn, lens, bt, idx, L.KERNEL_TCGEN05, f"tcgen05 {layout} append={append}", cos=cos, sin=sin)
    if not append:  # a sliding window on top: the last block is still the one with the tail
        _check(q, kc, vc, None, None, lens, bt, idx, L.KERNEL_TCGEN05, f"tcgen05 {layout} window", window=(300, 0))


@pytest.mark.parametrize("append", [False, True], ids=["read", "append"])
@pytest.mark.parametrize("layout", ["contiguous", "page128", "page256", "batch_idx"])
@pytest.mark.parametrize("s_q", [1, 4])
def test_decode_kernel_ignores_the_cache_tail(layout, append, s_q):
    g = torch.Generator().manual_seed(4200 + len(layout) + append + s_q)
    b, h, hk, d, s_cache = 6, 32, 8, 128, 1536
    s_new = s_q if append else 0
    lens = torch.tensor([333, 1024, 77, 0 if append else 1, s_cache - s_new, 1281], dtype=torch.int32)
    page = {"page128": 128, "page256": 256}.get(layout, 0)
    kc, vc, bt, idx = _poisoned_cache(g, BF, b, s_cache, hk, d, lens, s_new, page, extra_rows=3 if layout == "batch_idx" else 0)
    q = U.normal((b, s_q, h, d), BF, g)
    kn = vn = cos = sin = None
    if append:
        kn, vn = U.normal((b, s_new, hk, d), BF, g), U.normal((b, s_new, hk, d), BF, g)
        cos, sin = U.rotary_tables(s_cache + 8, 128, BF)
    _check(q, kc, vc, kn, vn, lens, bt, idx, L.KERNEL_DECODE, f"decode {layout} append={append} s_q={s_q}", cos=cos, sin=sin)


@pytest.mark.parametrize("append", [False, True], ids=["read", "append"])
@pytest.mark.parametrize("layout,d,dtype", [("contiguous", 64, FP), ("page16", 128, BF), ("page64", 64, BF), ("batch_idx", 256, BF),
                                            ("page256", 96, FP)])
def test_register_kernel_ignores_the_cache_tail(layout, d, dtype, append):
    """Head dims other than 128 and pages smaller than a key block run on the register-accumulator kernel."""
    g = torch.Generator().manual_seed(4300 + d + append)
    b, s_q, h, hk, s_cache = 4, 3, 8, 2, 768
    s_new = s_q if append else 0
    lens = torch.tensor([333, 512, 7, s_cache - s_new], dtype=torch.int32)
    page = {"page16": 16, "page64": 64, "page256": 256}.get(layout, 0)
    kc, vc, bt, idx = _poisoned_cache(g, dtype, b, s_cache, hk, d, lens, s_new, page, extra_rows=2 if layout == "batch_idx" else 0)
    q = U.normal((b, s_q, h, d), dtype, g)
    kn = vn = None
    if append:
        kn, vn = U.normal((b, s_new, hk, d), dtype, g), U.normal((b, s_new, hk, d), dtype, g)
    _check(q, kc, vc, kn, vn, lens, bt, idx, L.KERNEL_MMA, f"mma {layout} d={d} append={append}")


@pytest.mark.parametrize("kernel", [L.KERNEL_TCGEN05, L.KERNEL_MMA], ids=["tcgen05", "mma"])
def test_packed_sequences_do_not_see_their_neighbours(kernel):
    """Packed (varlen) input: the rows behind a sequence's last key belong to the next sequence.  With that one
    poisoned, the sequences in front of it and behind it must come out clean and equal to the oracle."""
    import flash_attn_npu_v2 as fa2
    g = torch.Generator().manual_seed(4400)
    h, hk, d = 4, 2, 128
    lens_q, lens_k = [200, 130, 300], [333, 190, 257]  # ends inside a 128-key block every time
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    ck = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    q = U.normal((sum(lens_q), h, d), BF, g)
    k, v = U.normal((sum(lens_k), hk, d), BF, g), U.normal((sum(lens_k), hk, d), BF, g)
    k[ck[1]:ck[2]] = NAN
    v[ck[1]:ck[2]] = NAN
    go, gl = OA.flash_attn_varlen_func(q, k, v, cq, ck, max(lens_q), max(lens_k), causal=True)
    out, lse, plan = ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), cu_seqlens_q=cq.cuda(), cu_seqlens_k=ck.cuda(),
                                           max_seqlen_q=max(lens_q), max_seqlen_k=max(lens_k), softmax_scale=d ** -0.5,
                                           causal=True, kernel=kernel, return_plan=True)
    assert plan.kernel == kernel
    for s in (0, 2):
        rows = slice(int(cq[s]), int(cq[s + 1]))
        assert torch.isfinite(out[rows].float()).all(), f"sequence {s} picked up its neighbour's NaN"
        U.check_rules(out[rows], lse[:, rows], go[rows], gl[:, rows], tag=f"packed seq {s}")
    del fa2
