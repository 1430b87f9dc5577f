"""GPU: the pieces of the FA3-style boundary around the forward itself.

* ``get_scheduler_metadata`` -> opaque plan bytes -> ``scheduler_metadata=`` on all three entry points, with the
  case tables of the reference's tests/test_flash_attn_npu_v3_metadata.py (:175-208: dense BSND, packed TND, paged
  KV cache with BSND and with TND queries) checked against the oracle instead of the reference's inline golden;
* what the bytes are: a self-contained plan that survives a copy, is refused for another problem, and whose
  decisions (kernel family, splits) are the ones the forward then uses;
* ``flash_attn_combine`` through the v3 package (flash_attn_npu_v3/interface_arch22.py:930-931);
* the ``torch.library`` operators: registered for CUDA under the reference's names, usable under
  ``torch.compile(fullgraph=True)``.
"""
import ctypes as C

import pytest
import torch

import parity_util as U
from flash_b200 import lib as L
from flash_b200 import ops
from oracle import api as OA

pytestmark = pytest.mark.gpu
BF, FP = torch.bfloat16, torch.float16
# Value range of the inputs: the reference's SMALL_RANGE (tests/test_flash_attn_npu_v3_metadata.py:20), which it uses
# for its KV-cache cases.  Its dense and packed cases draw from (-5, 5); on that range two evaluations of the golden
# itself with different key chunkings already disagree at the 1e-2 tolerance for about one element in a million
# (P is rounded relative to a running maximum), which the forward's own table tests cover; these tests are about
# the plan plumbing.
RANGE = (-1.0, 1.0)


def _meta(fa3, b, s_q, s_k, h, h_k, d, lens, dtype, cu_q=None, page=None, causal=False, num_splits=0, s_new=0):
    return fa3.get_scheduler_metadata(batch_size=b, max_seqlen_q=s_q, max_seqlen_k=s_k, num_heads_q=h, num_heads_kv=h_k,
                                      headdim=d, cache_seqlens=lens, qkv_dtype=dtype, cu_seqlens_q=cu_q, page_size=page,
                                      max_seqlen_k_new=s_new, causal=causal, window_size=(-1, -1), num_splits=num_splits,
                                      sm_margin=0)


def _decoded(meta):
    raw = bytes(meta.cpu().numpy().tobytes())
    pl = L.FwdPlan()
    L.check(L.load().fa_b200_plan_decode(raw, len(raw), C.byref(pl)))
    return pl


# data_type, batch, heads, kv heads, q_seqlen, kv_seqlen, head dim, causal   (reference :175-180)
@pytest.mark.parametrize("dtype,b,h,hk,s_q,s_k,d,causal", [
    (BF, 1, 1, 1, 1024, 1024, 128, False), (BF, 2, 4, 4, 1024, 1024, 128, True), (FP, 7, 1, 1, 512, 512, 128, False)])
def test_flash_attn_func_with_metadata(dtype, b, h, hk, s_q, s_k, d, causal):
    import flash_attn_npu_v3 as fa3
    g = torch.Generator().manual_seed(b * 100 + s_q)
    q, k, v = [U.uniform(shape, dtype, g, *RANGE) for shape in ((b, s_q, h, d), (b, s_k, hk, d), (b, s_k, hk, d))]
    lens = torch.full((b,), s_k, dtype=torch.int32, device="cuda")
    meta = _meta(fa3, b, s_q, s_k, h, hk, d, lens, dtype, causal=causal)
    assert meta.dtype == torch.uint8 and meta.is_cuda and meta.numel() == L.PLAN_BYTES
    out, lse = fa3.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), softmax_scale=d ** -0.5, causal=causal, num_splits=1,
                                   return_attn_probs=True, scheduler_metadata=meta)
    go, gl = OA.flash_attn_func(q, k, v, causal=causal)
    U.check_rules(out, lse, go, gl, strict_data_compare=False, tag="func + metadata")


# reference :183-190; the 7777 x 8192 row runs with 2048 x 2304 here (the CPU oracle is quadratic), same ragged shape class
@pytest.mark.parametrize("dtype,b,h,hk,s_q,s_k,d,causal", [
    (BF, 1, 1, 1, 512, 1024, 128, True), (BF, 2, 4, 4, 1024, 1024, 128, False), (FP, 7, 5, 1, 512, 512, 128, True),
    (BF, 5, 4, 4, 512, 512, 128, True), (FP, 7, 5, 1, 777, 888, 192, False), (BF, 1, 1, 1, 2041, 2304, 64, True)])
def test_flash_attn_varlen_func_with_metadata(dtype, b, h, hk, s_q, s_k, d, causal):
    import flash_attn_npu_v3 as fa3
    g = torch.Generator().manual_seed(b * 100 + s_q + 1)
    cq = torch.arange(b + 1, dtype=torch.int32) * s_q
    ck = torch.arange(b + 1, dtype=torch.int32) * s_k
    q, k, v = [U.uniform(shape, dtype, g, *RANGE) for shape in ((b * s_q, h, d), (b * s_k, hk, d), (b * s_k, hk, d))]
    lens = torch.full((b,), s_k, dtype=torch.int32, device="cuda")
    meta = _meta(fa3, b, s_q, s_k, h, hk, d, lens, dtype, cu_q=cq.cuda(), causal=causal)
    out, lse = fa3.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cq.cuda(), ck.cuda(), s_q, s_k, softmax_scale=d ** -0.5,
                                          causal=causal, num_splits=1, scheduler_metadata=meta, return_attn_probs=True)
    go, gl = OA.flash_attn_varlen_func(q, k, v, cq, ck, s_q, s_k, causal=causal)
    U.check_rules(out, lse, go, gl, strict_data_compare=False, tag="varlen + metadata")


def _paged(g, dtype, b, s_k, hk, d, page):
    per = -(-s_k // page)
    kc, vc = U.uniform((b * per, page, hk, d), dtype, g, *RANGE), U.uniform((b * per, page, hk, d), dtype, g, *RANGE)
    bt = torch.arange(b * per, dtype=torch.int32).view(b, per)
    return kc, vc, bt


# reference :193-198 (BSND queries) and :201-205 (TND queries)
@pytest.mark.parametrize("layout", ["bsnd", "tnd"])
@pytest.mark.parametrize("dtype,b,h,hk,s_q,s_k,d,page,causal", [
    (BF, 1, 1, 1, 1024, 1024, 128, 128, False), (BF, 5, 4, 4, 1024, 1024, 128, 128, True),
    (BF, 1, 1, 1, 2048, 2048, 128, 128, False), (BF, 5, 4, 4, 512, 512, 128, 128, True)])
def test_flash_attn_with_kvcache_with_metadata(layout, dtype, b, h, hk, s_q, s_k, d, page, causal):
    import flash_attn_npu_v3 as fa3
    g = torch.Generator().manual_seed(b * 100 + s_q + 2)
    q = U.uniform((b, s_q, h, d), dtype, g, *RANGE)
    kc, vc, bt = _paged(g, dtype, b, s_k, hk, d, page)
    lens = torch.full((b,), s_k, dtype=torch.int32)
    cq = torch.arange(b + 1, dtype=torch.int32).cuda() * s_q if layout == "tnd" else None
    meta = _meta(fa3, b, s_q, s_k, h, hk, d, lens.cuda(), dtype, cu_q=cq, page=page, causal=causal)
    q_in = q.view(b * s_q, h, d).cuda() if layout == "tnd" else q.cuda()
    out, lse, *_ = fa3.flash_attn_with_kvcache(q_in, kc.cuda(), vc.cuda(), cache_seqlens=lens.cuda(), page_table=bt.cuda(),
                                               cu_seqlens_q=cq, max_seqlen_q=s_q, causal=causal, rotary_interleaved=False,
                                               scheduler_metadata=meta, num_splits=0, return_softmax_lse=True)
    go, gl = OA.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens, block_table=bt, causal=causal)
    if layout == "tnd":  # (total_q, h, d) and (h, total_q)
        assert tuple(out.shape) == (b * s_q, h, d) and tuple(lse.shape) == (h, b * s_q)
        out = out.view(b, s_q, h, d)
        lse = lse.view(h, b, s_q).permute(1, 0, 2)
    U.check_rules(out, lse, go, gl, tag=f"kvcache + metadata {layout}")


def test_tnd_queries_of_different_lengths_against_a_paged_cache():
    """The TND query layout exists for batches whose sequences bring different numbers of new tokens."""
    import flash_attn_npu_v3 as fa3
    g = torch.Generator().manual_seed(77)
    b, h, hk, d, page, s_cache = 4, 8, 2, 128, 128, 1024
    q_lens = [1, 37, 160, 300]
    cq = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    q = U.normal((sum(q_lens), h, d), BF, g)
    kc, vc, bt = _paged(g, BF, b, s_cache, hk, d, page)
    lens = torch.tensor([700, 37, 1024, 513], dtype=torch.int32)
    out, lse, *_ = fa3.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens.cuda(), page_table=bt.cuda(),
                                               cu_seqlens_q=cq.cuda(), max_seqlen_q=max(q_lens), causal=True,
                                               return_softmax_lse=True)
    for i in range(b):
        rows = slice(int(cq[i]), int(cq[i + 1]))
        go, gl = OA.flash_attn_with_kvcache(q[rows].unsqueeze(0), kc, vc, cache_seqlens=lens[i:i + 1], block_table=bt[i:i + 1],
                                            causal=True)
        U.check_rules(out[rows].unsqueeze(0), lse[:, rows].unsqueeze(0), go, gl, tag=f"tnd-q kvcache seq {i}")


def test_metadata_is_the_plan_and_the_forward_uses_it():
    """Decode against a ragged contiguous cache: the bytes name the decode kernel's persistent schedule, they
    survive a clone and a round trip through the host, and a forward given them runs exactly that plan."""
    import flash_attn_npu_v3 as fa3
    g = torch.Generator().manual_seed(5)
    b, h, hk, d, s_cache = 24, 32, 8, 128, 4096
    q = U.normal((b, 1, h, d), BF, g)
    kc, vc = U.normal((b, s_cache, hk, d), BF, g), U.normal((b, s_cache, hk, d), BF, g)
    lens = torch.randint(1, s_cache, (b,), generator=g, dtype=torch.int32)
    meta = _meta(fa3, b, 1, s_cache, h, hk, d, lens.cuda(), BF, causal=True)
    pl = _decoded(meta)
    assert pl.kernel == L.KERNEL_DECODE and pl.num_splits > 1 and pl.workspace_bytes > 0
    go, gl = OA.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens, causal=True)
    for m in (meta, meta.clone(), meta.cpu().cuda()):  # nothing rides on the tensor object
        assert not hasattr(m, "_fa_b200_plan")
        out, lse, *_ = fa3.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens.cuda(), causal=True,
                                                   scheduler_metadata=m, num_splits=0, return_softmax_lse=True)
        U.check_rules(out, lse, go, gl, tag="decode + metadata")
    # a plan that asks for 3 splits is followed, whatever the heuristic would have chosen
    meta3 = _meta(fa3, b, 1, s_cache, h, hk, d, lens.cuda(), BF, causal=True, num_splits=3)
    assert _decoded(meta3).num_splits == 3
    n0 = L.load().fa_b200_launch_count()
    out, lse, *_ = fa3.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens.cuda(), causal=True,
                                               scheduler_metadata=meta3, num_splits=3, return_softmax_lse=True)
    assert L.load().fa_b200_launch_count() - n0 == 2  # the split kernel and its merge
    U.check_rules(out, lse, go, gl, tag="decode + 3-split metadata")


def test_metadata_for_another_problem_is_refused():
    import flash_attn_npu_v3 as fa3
    q = torch.zeros((2, 1, 8, 128), dtype=BF, device="cuda")
    kc = torch.zeros((2, 256, 2, 128), dtype=BF, device="cuda")
    lens = torch.full((2,), 100, dtype=torch.int32, device="cuda")
    good = _meta(fa3, 2, 1, 256, 8, 2, 128, lens, BF, causal=True)
    fa3.flash_attn_with_kvcache(q, kc, kc, cache_seqlens=lens, causal=True, scheduler_metadata=good)
    for bad, what in ((_meta(fa3, 3, 1, 256, 8, 2, 128, lens, BF, causal=True), "batch size"),
                      (_meta(fa3, 2, 1, 256, 16, 2, 128, lens, BF, causal=True), "num_heads_q"),
                      (_meta(fa3, 2, 1, 256, 8, 2, 128, lens, FP, causal=True), "dtype"),
                      (_meta(fa3, 2, 1, 256, 8, 2, 128, lens, BF, causal=False), "causal")):
        with pytest.raises(RuntimeError, match=f"different problem: {what}"):
            fa3.flash_attn_with_kvcache(q, kc, kc, cache_seqlens=lens, causal=True, scheduler_metadata=bad)
    with pytest.raises(RuntimeError, match="not made by get_scheduler_metadata"):
        fa3.flash_attn_with_kvcache(q, kc, kc, cache_seqlens=lens, causal=True,
                                    scheduler_metadata=torch.zeros(L.PLAN_BYTES, dtype=torch.uint8, device="cuda"))
    with pytest.raises(RuntimeError, match="uint8 tensor"):
        fa3.flash_attn_with_kvcache(q, kc, kc, cache_seqlens=lens, causal=True,
                                    scheduler_metadata=torch.zeros(8, dtype=torch.uint8, device="cuda"))


def test_flash_attn_combine_through_the_v3_package():
    from flash_attn_npu_v3 import interface as I
    g = torch.Generator().manual_seed(11)
    n, b, s, h, d = 5, 2, 3, 4, 128
    o_parts = torch.randn((n, b, s, h, d), generator=g)
    lse_parts = torch.randn((n, b, s, h), generator=g) * 3
    lse_parts[1, 0] = float("-inf")      # an empty partial
    lse_parts[:, 1, 2, 3] = float("-inf")  # a row every partial of which is empty
    go, gl = OA.merge_partials(o_parts, lse_parts, out_dtype=BF)
    out, lse = I.flash_attn_combine(o_parts.cuda(), lse_parts.cuda(), out_dtype=BF)
    torch.testing.assert_close(out.float().cpu(), go.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse.cpu(), gl, rtol=1e-5, atol=1e-5)
    assert float(lse[1, 2, 3]) == float("inf") and float(out[1, 2, 3].abs().max()) == 0.0


def test_custom_operators_are_registered_for_cuda():
    import flash_attn_npu_v2  # noqa: F401
    import flash_attn_npu_v3  # noqa: F401
    g = torch.Generator().manual_seed(3)
    q, k, v = [U.normal((2, 130, 4, 64), FP, g).cuda() for _ in range(3)]
    out, lse, p, rng = torch.ops.flash_attn_npu_arch22_v2._flash_attn_forward(q, k, v, 0.0, 0.125, True, -1, -1, 0.0, None, False)
    go, gl = OA.flash_attn_func(q.cpu(), k.cpu(), v.cpu(), causal=True)
    U.check_rules(out, lse, go, gl, tag="v2 operator")
    assert p.numel() == 0 and tuple(rng.shape) == (2,)
    out3, lse3, acc, lacc = torch.ops.flash_attn_npu_arch22_v3._flash_attn_forward(q, k, v, softmax_scale=0.125, causal=True)
    assert torch.equal(out3, out) and torch.equal(lse3, lse) and acc.numel() == 0 and lacc.numel() == 0
    with pytest.raises(RuntimeError, match="_flash_attn_forward_inplace"):
        torch.ops.flash_attn_npu_arch22_v3._flash_attn_forward(q, k, v, k, v)
    for name in ("_flash_attn_varlen_forward", "_flash_attn_backward", "_flash_attn_varlen_backward"):
        assert hasattr(torch.ops.flash_attn_npu_arch22_v2, name)
    assert hasattr(torch.ops.flash_attn_npu_arch22_v3, "_flash_attn_backward")


@pytest.mark.parametrize("api", ["v2", "v3"])
def test_flash_attn_func_compiles_as_one_graph(api):
    import flash_attn_npu_v2 as fa2
    import flash_attn_npu_v3 as fa3
    g = torch.Generator().manual_seed(4)
    q, k, v = [U.normal((2, 256, 4, 128), BF, g).cuda() for _ in range(3)]

    def f(q, k, v):
        if api == "v2":
            return fa2.flash_attn_func(q * 1.0, k, v, causal=True) + 0.0
        return fa3.flash_attn_func(q * 1.0, k, v, causal=True) + 0.0

    eager = f(q, k, v)
    compiled = torch.compile(f, fullgraph=True, backend="aot_eager")(q, k, v)
    assert torch.equal(eager, compiled)
    go, _ = OA.flash_attn_func(q.cpu(), k.cpu(), v.cpu(), causal=True)
    torch.testing.assert_close(compiled.float().cpu(), go.float(), rtol=1e-2, atol=1e-2)
    # and with gradients: the backward operator is traced as well
    qg, kg, vg = [t.clone().requires_grad_(True) for t in (q, k, v)]
    torch.compile(f, fullgraph=True, backend="aot_eager")(qg, kg, vg).float().sum().backward()
    qe, ke, ve = [t.clone().requires_grad_(True) for t in (q, k, v)]
    f(qe, ke, ve).float().sum().backward()
    for a, e in ((qg, qe), (kg, ke), (vg, ve)):
        torch.testing.assert_close(a.grad.float(), e.grad.float(), rtol=1e-2, atol=1e-2)
