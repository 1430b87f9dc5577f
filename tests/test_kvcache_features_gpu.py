"""GPU parity for the KV-cache features the reference documents but does not implement natively
(in-place append, rotary, cache_batch_idx, alibi; flash_attn_npu_v2/interface_arch22.py:1452-1537)
and for paged caches with non-identity block tables.  Oracle: oracle/api.py (parity unpinned by
reference tests for these features; the cache update must be bit-exact against the oracle)."""
import pytest
import torch

import parity_util as U
from oracle import api as OA

pytestmark = pytest.mark.gpu
BF, FP = torch.bfloat16, torch.float16


def _run_both(q, kc, vc, k, v, lens, *, cos=None, sin=None, interleaved=False, idx=None, bt=None, causal=True,
              window=(-1, -1), alibi=None, num_splits=0, api="v2"):
    import flash_attn_npu_v2 as fa2
    import flash_attn_npu_v3 as fa3
    kc_o, vc_o = kc.clone(), vc.clone()
    gold_out, gold_lse = OA.flash_attn_with_kvcache(
        q, kc_o, vc_o, k, v, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens, cache_batch_idx=idx,
        block_table=bt, causal=causal, window_size=window, rotary_interleaved=interleaved, alibi_slopes=alibi)
    c = lambda t: None if t is None else t.cuda()
    kc_g, vc_g = kc.cuda(), vc.cuda()
    if api == "v2":
        out, lse = fa2.flash_attn_with_kvcache(
            c(q), kc_g, vc_g, c(k), c(v), rotary_cos=c(cos), rotary_sin=c(sin), cache_seqlens=c(lens),
            cache_batch_idx=c(idx), block_table=c(bt), causal=causal, window_size=window,
            rotary_interleaved=interleaved, alibi_slopes=c(alibi), num_splits=num_splits, return_softmax_lse=True)
    else:
        out, lse, *_ = fa3.flash_attn_with_kvcache(
            c(q), kc_g, vc_g, c(k), c(v), rotary_cos=c(cos), rotary_sin=c(sin), cache_seqlens=c(lens),
            cache_batch_idx=c(idx), page_table=c(bt), causal=causal, window_size=window,
            rotary_interleaved=interleaved, num_splits=num_splits, return_softmax_lse=True)
    torch.cuda.synchronize()
    # bit-exact cache update, untouched rows included
    assert torch.equal(kc_g.cpu().view(torch.int16), kc_o.view(torch.int16)), "k_cache differs"
    assert torch.equal(vc_g.cpu().view(torch.int16), vc_o.view(torch.int16)), "v_cache differs"
    return out, lse, gold_out, gold_lse


@pytest.mark.parametrize("dtype", [BF, FP])
@pytest.mark.parametrize("s_new,s_q", [(1, 1), (3, 3), (5, 2)])
@pytest.mark.parametrize("rotary,interleaved", [(0, False), (64, False), (64, True), (32, False)])
def test_append_rotary_contiguous(dtype, s_new, s_q, rotary, interleaved):
    g = torch.Generator().manual_seed(1000 + s_new * 10 + rotary)
    b, h, hk, d, s_cache = 3, 8, 2, 64, 384
    q = U.normal((b, s_q, h, d), dtype, g)
    kc, vc = U.normal((b, s_cache, hk, d), dtype, g), U.normal((b, s_cache, hk, d), dtype, g)
    k, v = U.normal((b, s_new, hk, d), dtype, g), U.normal((b, s_new, hk, d), dtype, g)
    lens = torch.tensor([0, 129, s_cache - s_new], dtype=torch.int32)
    cos = sin = None
    if rotary:
        cos, sin = U.rotary_tables(s_cache + 8, rotary, dtype)
    out, lse, go, gl = _run_both(q, kc, vc, k, v, lens, cos=cos, sin=sin, interleaved=interleaved, causal=True)
    U.check_rules(out, lse, go, gl, tag="append")


@pytest.mark.parametrize("causal", [False, True])
def test_append_rotary_noncausal_q_position(causal):
    """Non-causal: every q token is rotated at position cache_seqlens (docstring :1462-1467)."""
    g = torch.Generator().manual_seed(7)
    b, h, hk, d, s_cache = 2, 4, 4, 128, 256
    q = U.normal((b, 4, h, d), BF, g)
    kc, vc = U.normal((b, s_cache, hk, d), BF, g), U.normal((b, s_cache, hk, d), BF, g)
    k, v = U.normal((b, 4, hk, d), BF, g), U.normal((b, 4, hk, d), BF, g)
    lens = torch.tensor([100, 17], dtype=torch.int32)
    cos, sin = U.rotary_tables(s_cache, 128, BF)
    out, lse, go, gl = _run_both(q, kc, vc, k, v, lens, cos=cos, sin=sin, causal=causal)
    U.check_rules(out, lse, go, gl, tag="qpos")


@pytest.mark.parametrize("page", [16, 128, 256])
@pytest.mark.parametrize("api", ["v2", "v3"])
def test_paged_permuted_append(page, api):
    g = torch.Generator().manual_seed(page)
    b, h, hk, d, s_q, s_new = 3, 16, 2, 128, 2, 2
    max_blocks = 1024 // page
    nblk = b * max_blocks + 3
    kc, vc = U.normal((nblk, page, hk, d), BF, g), U.normal((nblk, page, hk, d), BF, g)
    bt = torch.randperm(nblk, generator=g)[: b * max_blocks].view(b, max_blocks).to(torch.int32)
    lens = torch.tensor([1, 517, 1024 - s_new], dtype=torch.int32)
    q = U.normal((b, s_q, h, d), BF, g)
    k, v = U.normal((b, s_new, hk, d), BF, g), U.normal((b, s_new, hk, d), BF, g)
    cos, sin = U.rotary_tables(1024, 128, BF)
    out, lse, go, gl = _run_both(q, kc, vc, k, v, lens, cos=cos, sin=sin, bt=bt, causal=True, api=api)
    U.check_rules(out, lse, go, gl, tag="paged")


def test_cache_batch_idx_and_alibi():
    g = torch.Generator().manual_seed(5)
    b, h, hk, d, s_cache = 3, 6, 3, 64, 200
    q = U.normal((b, 2, h, d), FP, g)
    kc, vc = U.normal((5, s_cache, hk, d), FP, g), U.normal((5, s_cache, hk, d), FP, g)
    k, v = U.normal((b, 2, hk, d), FP, g), U.normal((b, 2, hk, d), FP, g)
    lens = torch.tensor([10, 150, 64], dtype=torch.int32)
    idx = torch.tensor([4, 0, 2], dtype=torch.int32)
    slopes = torch.tensor([2.0 ** (-(i + 1)) for i in range(h)], dtype=torch.float32)
    out, lse, go, gl = _run_both(q, kc, vc, k, v, lens, idx=idx, causal=True, alibi=slopes)
    U.check_rules(out, lse, go, gl, tag="idx+alibi")
    slopes2 = torch.rand(b, h, generator=g) * 0.3
    out, lse, go, gl = _run_both(q, kc, vc, None, None, lens, idx=idx, causal=False, alibi=slopes2)
    U.check_rules(out, lse, go, gl, tag="alibi(b,h)")


def test_append_is_replay_idempotent():
    """Same inputs twice -> bit-identical cache and output."""
    import flash_attn_npu_v2 as fa2
    g = torch.Generator().manual_seed(3)
    q = U.normal((2, 1, 8, 128), BF, g).cuda()
    kc, vc = U.normal((2, 300, 2, 128), BF, g).cuda(), U.normal((2, 300, 2, 128), BF, g).cuda()
    k, v = U.normal((2, 1, 2, 128), BF, g).cuda(), U.normal((2, 1, 2, 128), BF, g).cuda()
    lens = torch.tensor([5, 299], dtype=torch.int32).cuda()
    cos, sin = [t.cuda() for t in U.rotary_tables(300, 128, BF)]
    o1 = fa2.flash_attn_with_kvcache(q, kc, vc, k, v, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens, causal=True,
                                     rotary_interleaved=False)
    k1, v1 = kc.clone(), vc.clone()
    o2 = fa2.flash_attn_with_kvcache(q, kc, vc, k, v, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens, causal=True,
                                     rotary_interleaved=False)
    assert torch.equal(o1, o2) and torch.equal(k1, kc) and torch.equal(v1, vc)


@pytest.mark.parametrize("num_splits", [1, 2, 3, 7, 0])
@pytest.mark.parametrize("s_q,h,hk", [(1, 8, 2), (4, 64, 8), (6, 4, 4)])
def test_split_kv_matches_oracle(num_splits, s_q, h, hk):
    g = torch.Generator().manual_seed(num_splits * 31 + s_q)
    b, d, s_cache = 2, 128, 3000
    q = U.normal((b, s_q, h, d), BF, g)
    kc, vc = U.normal((b, s_cache, hk, d), BF, g), U.normal((b, s_cache, hk, d), BF, g)
    lens = torch.tensor([2999, 700], dtype=torch.int32)
    out, lse, go, gl = _run_both(q, kc, vc, None, None, lens, causal=True, num_splits=num_splits)
    U.check_rules(out, lse, go, gl, tag=f"splits={num_splits}")
    out, lse, go, gl = _run_both(q, kc, vc, None, None, lens, causal=True, window=(600, 0), num_splits=num_splits)
    U.check_rules(out, lse, go, gl, tag=f"splits={num_splits} window")


def test_int_cache_seqlens_and_no_seqlens():
    import flash_attn_npu_v2 as fa2
    g = torch.Generator().manual_seed(8)
    q = U.normal((2, 3, 4, 64), FP, g)
    kc, vc = U.normal((2, 130, 4, 64), FP, g), U.normal((2, 130, 4, 64), FP, g)
    go, gl = OA.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=77, causal=True)
    out, lse = fa2.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=77, causal=True,
                                           return_softmax_lse=True)
    U.check_rules(out, lse, go, gl, tag="int seqlens")
    go, gl = OA.flash_attn_with_kvcache(q, kc, vc, causal=False)
    out, lse = fa2.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), return_softmax_lse=True)
    U.check_rules(out, lse, go, gl, tag="no seqlens")


def test_seqlen_q_longer_than_k_dead_rows():
    """s_q > s_k with causal: leading rows see no key -> O = 0, LSE = +inf (README picture :120-126)."""
    import flash_attn_npu_v2 as fa2
    g = torch.Generator().manual_seed(9)
    q, k, v = U.normal((1, 5, 2, 64), BF, g), U.normal((1, 2, 2, 64), BF, g), U.normal((1, 2, 2, 64), BF, g)
    go, gl = OA.flash_attn_func(q, k, v, causal=True)
    out, lse, _ = fa2.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=True, return_attn_probs=True)
    assert torch.isinf(lse[0, :, :3]).all() and (out[0, :3] == 0).all()
    U.check_rules(out, lse, go, gl, tag="dead rows")


def test_errors_raise_runtime_error():
    import flash_attn_npu_v2 as fa2
    q = torch.zeros(1, 1, 3, 64, dtype=BF, device="cuda")
    kc = torch.zeros(1, 8, 2, 64, dtype=BF, device="cuda")
    with pytest.raises(RuntimeError, match="Number of heads"):
        fa2.flash_attn_with_kvcache(q, kc, kc, cache_seqlens=4)
    with pytest.raises(RuntimeError, match="FP16 and BF16"):
        fa2.flash_attn_func(q.float(), q.float(), q.float())
    with pytest.raises(RuntimeError, match="leftpad"):
        fa2.flash_attn_with_kvcache(q[:, :, :2], kc, kc, cache_seqlens=4,
                                    cache_leftpad=torch.zeros(1, dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA"):
        fa2.flash_attn_func(q.cpu(), q.cpu(), q.cpu())


@pytest.mark.parametrize("paged", [False, True])
def test_persistent_decode_ragged(paged):
    """Ragged cache lengths on the persistent decode path (CTAs take equal shares of the KV blocks of the whole
    launch, units cut by a CTA boundary are merged from partials): an empty sequence, very short and full ones,
    append + rotary in place, GQA packing."""
    from flash_b200 import lib as L
    from flash_b200 import ops
    g = torch.Generator().manual_seed(77)
    b, h, hk, d, s_cache, page = 24, 16, 4, 128, 2304, 256
    q = U.normal((b, 1, h, d), BF, g)
    kc, vc = U.normal((b, s_cache, hk, d), BF, g), U.normal((b, s_cache, hk, d), BF, g)
    k, v = U.normal((b, 1, hk, d), BF, g), U.normal((b, 1, hk, d), BF, g)
    lens = torch.randint(1, s_cache - 1, (b,), generator=g, dtype=torch.int32)
    lens[0], lens[1], lens[2], lens[3] = 0, 1, s_cache - 1, 63
    cos, sin = U.rotary_tables(s_cache + 8, 64, BF)
    bt = None
    if paged:
        nblk = b * s_cache // page
        perm = torch.randperm(nblk, generator=g)
        bt = perm.view(b, s_cache // page).to(torch.int32)
        pool_k, pool_v = torch.empty((nblk, page, hk, d), dtype=BF), torch.empty((nblk, page, hk, d), dtype=BF)
        pool_k[perm] = kc.view(nblk, page, hk, d)
        pool_v[perm] = vc.view(nblk, page, hk, d)
        kc, vc = pool_k, pool_v
    out, lse, go, gl = _run_both(q, kc, vc, k, v, lens, cos=cos, sin=sin, bt=bt, causal=True)
    U.check_rules(out, lse, go, gl, tag=f"persistent decode paged={paged}")
    # the plan of this problem is the persistent one: a resident grid and a fixed number of partial slots
    _, _, plan = ops.attention_forward(q.cuda(), kc.cuda(), vc.cuda(), k_new=k.cuda(), v_new=v.cuda(),
                                       seqused_k=lens.cuda(), block_table=None if bt is None else bt.cuda(),
                                       rotary_cos=cos.cuda(), rotary_sin=sin.cuda(), softmax_scale=d ** -0.5,
                                       causal=True, return_plan=True)
    assert plan.kernel == L.KERNEL_DECODE and plan.num_splits == 4 and plan.grid <= 2 * 160
    assert L.load().fa_b200_check_status(torch.cuda.current_stream().cuda_stream) == 0


@pytest.mark.parametrize("page", [0, 128, 256])
@pytest.mark.parametrize("dtype", [BF, FP])
def test_chunked_prefill_against_cache_runs_on_tcgen05(page, dtype):
    """Many query tokens against a KV cache with per-entry lengths (no append), contiguous (page 0) or paged: the
    tcgen05 prefill kernel takes it (keys in use from cache_seqlens, pages from the block table).  Lengths below the
    query count (rows without visible keys), an empty entry, lengths that end inside a block and inside a page."""
    from flash_b200 import lib as L
    from flash_b200 import ops
    g = torch.Generator().manual_seed(500 + page)
    b, s_q, h, hk, d, s_cache = 5, 200, 8, 2, 128, 1280
    q = U.normal((b, s_q, h, d), dtype, g)
    kc, vc = U.normal((b, s_cache, hk, d), dtype, g), U.normal((b, s_cache, hk, d), dtype, g)
    lens = torch.tensor([333, 1280, 77, 0, 1025], dtype=torch.int32)
    bt = None
    if page:
        nblk = b * s_cache // page + 3  # a few pages nobody owns
        perm = torch.randperm(nblk, generator=g)[:b * s_cache // page]
        bt = perm.view(b, s_cache // page).to(torch.int32)
        pool_k, pool_v = U.normal((nblk, page, hk, d), dtype, g), U.normal((nblk, page, hk, d), dtype, g)
        pool_k[perm] = kc.view(-1, page, hk, d)
        pool_v[perm] = vc.view(-1, page, hk, d)
        kc, vc = pool_k, pool_v
    out, lse, go, gl = _run_both(q, kc, vc, None, None, lens, bt=bt, causal=True)
    U.check_rules(out, lse, go, gl, tag=f"chunked prefill page={page}")
    _, _, plan = ops.attention_forward(q.cuda(), kc.cuda(), vc.cuda(), seqused_k=lens.cuda(),
                                       block_table=None if bt is None else bt.cuda(), softmax_scale=d ** -0.5,
                                       causal=True, return_plan=True)
    assert plan.kernel == L.KERNEL_TCGEN05
    if not page:  # the cache rows of the batch entries picked by cache_batch_idx (a cache with more rows than the batch)
        idx = torch.tensor([6, 0, 3, 5, 1], dtype=torch.int32)
        big_k, big_v = U.normal((7, s_cache, hk, d), dtype, g), U.normal((7, s_cache, hk, d), dtype, g)
        out, lse, go, gl = _run_both(q, big_k, big_v, None, None, lens, idx=idx, causal=True)
        U.check_rules(out, lse, go, gl, tag="chunked prefill cache_batch_idx")
        kn, vn = U.normal((b, s_q, hk, d), dtype, g), U.normal((b, s_q, hk, d), dtype, g)
        lens2 = torch.tensor([333, 1000, 77, 0, 1025], dtype=torch.int32)
        out, lse, go, gl = _run_both(q, big_k, big_v, kn, vn, lens2, idx=idx, causal=True)  # + append (bit-exact cache check inside)
        U.check_rules(out, lse, go, gl, tag="chunked prefill cache_batch_idx + append")
        _, _, plan = ops.attention_forward(q.cuda(), big_k.cuda(), big_v.cuda(), seqused_k=lens.cuda(), cache_batch_idx=idx.cuda(),
                                           softmax_scale=d ** -0.5, causal=True, return_plan=True)
        assert plan.kernel == L.KERNEL_TCGEN05
    # a sliding window on top, narrower and wider than every cache length (the rule that turns a window covering all
    # keys into "causal" needs the longest length, which only the device knows: the kernel keeps the window)
    for wl in (300, 5000):
        out, lse, go, gl = _run_both(q, kc, vc, None, None, lens, bt=bt, causal=True, window=(wl, 0))
        U.check_rules(out, lse, go, gl, tag=f"chunked prefill window {wl} page={page}")
    _, _, plan = ops.attention_forward(q.cuda(), kc.cuda(), vc.cuda(), seqused_k=lens.cuda(),
                                       block_table=None if bt is None else bt.cuda(), softmax_scale=d ** -0.5,
                                       causal=True, window_left=300, window_right=0, return_plan=True)
    assert plan.kernel == L.KERNEL_TCGEN05 and plan.is_local == 1


@pytest.mark.parametrize("page", [0, 128, 256])
@pytest.mark.parametrize("rotary,interleaved", [(0, False), (64, False), (128, True)])
def test_chunked_prefill_with_append_runs_on_tcgen05(page, rotary, interleaved):
    """A chunk of new tokens (q, k, v of the same 160 positions) against a cache: the new k (rotated) and v are
    written into the cache bit-exactly, q is rotated at its positions, and the attention runs on the tcgen05
    kernel behind an append / rotary prologue launch."""
    from flash_b200 import lib as L
    from flash_b200 import ops
    g = torch.Generator().manual_seed(900 + page + rotary)
    b, s_q, h, hk, d, s_cache = 4, 160, 8, 2, 128, 1024
    q = U.normal((b, s_q, h, d), BF, g)
    k, v = U.normal((b, s_q, hk, d), BF, g), U.normal((b, s_q, hk, d), BF, g)
    kc, vc = U.normal((b, s_cache, hk, d), BF, g), U.normal((b, s_cache, hk, d), BF, g)
    lens = torch.tensor([0, 100, s_cache - s_q, 511], dtype=torch.int32)
    cos = sin = None
    if rotary:
        cos, sin = U.rotary_tables(s_cache + 8, rotary, BF)
    bt = None
    if page:
        nblk = b * s_cache // page + 2
        perm = torch.randperm(nblk, generator=g)[:b * s_cache // page]
        bt = perm.view(b, s_cache // page).to(torch.int32)
        pool_k, pool_v = U.normal((nblk, page, hk, d), BF, g), U.normal((nblk, page, hk, d), BF, g)
        pool_k[perm] = kc.view(-1, page, hk, d)
        pool_v[perm] = vc.view(-1, page, hk, d)
        kc, vc = pool_k, pool_v
    out, lse, go, gl = _run_both(q, kc, vc, k, v, lens, cos=cos, sin=sin, interleaved=interleaved, bt=bt, causal=True)
    U.check_rules(out, lse, go, gl, tag=f"chunked prefill + append page={page} rotary={rotary}")
    c = lambda t: None if t is None else t.cuda()
    _, _, plan = ops.attention_forward(c(q), c(kc), c(vc), k_new=c(k), v_new=c(v), seqused_k=c(lens), block_table=c(bt),
                                       rotary_cos=c(cos), rotary_sin=c(sin), rotary_interleaved=interleaved,
                                       softmax_scale=d ** -0.5, causal=True, return_plan=True)
    assert plan.kernel == L.KERNEL_TCGEN05 and plan.launches == 2
    assert plan.workspace_bytes == (b * s_q * h * d * 2 if rotary else 0)
