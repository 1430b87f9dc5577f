"""The five benchmark configurations at FULL size on the GPU: seeded synthetic inputs generated on
the device; the CPU oracle checks a sample of (batch, head) slices (the golden needs ~1 s per
slice) and size-independent properties cover the whole output:

* scaling V by 2 scales O by exactly 2 (bf16 doubling is exact) and leaves LSE bit-identical;
* the split-KV result equals the unsplit result within fp32 merge rounding;
* in-place KV append is bit-exact and leaves every other cache row untouched.
"""
import math

import pytest
import torch

import parity_util as U
from oracle import api as OA

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def test_config2_causal_prefill_full():
    import flash_attn_npu_v2 as fa2
    g = _gen(2)
    shape = (4, 4096, 32, 128)
    q, k, v = [(torch.randn(shape, generator=g, device="cuda") / math.sqrt(2)).to(BF) for _ in range(3)]
    out, lse, _ = fa2.flash_attn_func(q, k, v, causal=True, return_attn_probs=True)
    assert lse.shape == (4, 32, 4096) and lse.dtype == torch.float32
    for (b, h) in [(0, 0), (3, 31), (1, 17)]:
        qs, ks, vs = [t[b:b + 1, :, h:h + 1].cpu() for t in (q, k, v)]
        go, gl = OA.flash_attn_func(qs, ks, vs, causal=True)
        plain = U.plain_dtype_attention(qs, ks, vs, 128 ** -0.5, causal=True)
        U.check_rules(out[b:b + 1, :, h:h + 1], lse[b:b + 1, h:h + 1], go, gl, plain_out=plain, tag=f"c2[{b},{h}]")
    out2, lse2, _ = fa2.flash_attn_func(q, k, v * 2, causal=True, return_attn_probs=True)
    assert torch.equal(out2.float(), out.float() * 2) and torch.equal(lse2, lse)


def _rotary(seqlen, dim):
    return [t.cuda() for t in U.rotary_tables(seqlen, dim, BF)]


def test_config3_contiguous_decode_append_rotary_full():
    import flash_attn_npu_v2 as fa2
    g = _gen(3)
    b, s_cache, h, hk, d = 64, 8192, 32, 8, 128
    kc = torch.randn((b, s_cache, hk, d), generator=g, device="cuda").to(BF)
    vc = torch.randn((b, s_cache, hk, d), generator=g, device="cuda").to(BF)
    q = torch.randn((b, 1, h, d), generator=g, device="cuda").to(BF)
    k = torch.randn((b, 1, hk, d), generator=g, device="cuda").to(BF)
    v = torch.randn((b, 1, hk, d), generator=g, device="cuda").to(BF)
    lens = torch.randint(1024, 8192, (b,), generator=g, device="cuda", dtype=torch.int32)
    cos, sin = _rotary(8192, 128)
    sample = [0, 21, 63]
    ref_k = {i: kc[i].cpu() for i in sample}
    ref_v = {i: vc[i].cpu() for i in sample}
    k_before, v_before = kc.clone(), vc.clone()
    out, lse = fa2.flash_attn_with_kvcache(q, kc, vc, k, v, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens,
                                           causal=True, rotary_interleaved=False, return_softmax_lse=True)
    lens_c = lens.cpu()
    for i in sample:
        kci, vci = ref_k[i].unsqueeze(0).clone(), ref_v[i].unsqueeze(0).clone()
        go, gl = OA.flash_attn_with_kvcache(q[i:i + 1].cpu(), kci, vci, k[i:i + 1].cpu(), v[i:i + 1].cpu(),
                                            rotary_cos=cos.cpu(), rotary_sin=sin.cpu(),
                                            cache_seqlens=lens_c[i:i + 1], causal=True, rotary_interleaved=False)
        U.check_rules(out[i:i + 1], lse[i:i + 1], go, gl, tag=f"c3[{i}]")
        assert torch.equal(kc[i].cpu().view(torch.int16), kci[0].view(torch.int16))
        assert torch.equal(vc[i].cpu().view(torch.int16), vci[0].view(torch.int16))
    # every row except the appended one is untouched, in every sequence
    rows = torch.arange(s_cache, device="cuda").view(1, -1)
    untouched = (rows != lens.view(-1, 1).long())
    assert torch.equal(kc[untouched], k_before[untouched]) and torch.equal(vc[untouched], v_before[untouched])
    assert torch.equal(vc[torch.arange(b), lens.long()], v[:, 0])


def test_config4_paged_speculative_decode_full():
    import flash_attn_npu_v2 as fa2
    g = _gen(4)
    b, s_q, h, hk, d, page, nblk = 32, 4, 64, 8, 128, 256, 4096
    kp = torch.randn((nblk, page, hk, d), generator=g, device="cuda").to(BF)
    vp = torch.randn((nblk, page, hk, d), generator=g, device="cuda").to(BF)
    bt = torch.randperm(nblk, generator=g, device="cuda").view(b, 128).to(torch.int32)
    lens = torch.randint(512, 32769, (b,), generator=g, device="cuda", dtype=torch.int32)
    q = torch.randn((b, s_q, h, d), generator=g, device="cuda").to(BF)
    out, lse = fa2.flash_attn_with_kvcache(q, kp, vp, cache_seqlens=lens, block_table=bt, causal=True,
                                           window_size=(4096, 0), return_softmax_lse=True)
    max_k = int(lens.max())
    for i in [0, 13, 31]:
        L = int(lens[i])
        ki = OA.gather_paged(kp.cpu(), bt[i].cpu(), L).unsqueeze(0)
        vi = OA.gather_paged(vp.cpu(), bt[i].cpu(), L).unsqueeze(0)
        # same window normalisation as the batched call: the maximum length over the batch decides
        ic, il, wl, wr = OA.G.normalize_window(s_q, max_k, True, 4096, 0)
        mask = OA.G.build_mask(s_q, L, ic, il, wl, wr)
        go, gl = OA.G.blockwise_attention(q[i].cpu(), ki[0], vi[0], d ** -0.5, mask, BF)
        go, gl = OA.G.patch_dead_rows(go, gl, mask)
        U.check_rules(out[i:i + 1], lse[i:i + 1], go.unsqueeze(0), gl.unsqueeze(0), tag=f"c4[{i}]")
    o1, l1 = fa2.flash_attn_with_kvcache(q, kp, vp, cache_seqlens=lens, block_table=bt, causal=True,
                                         window_size=(4096, 0), num_splits=1, return_softmax_lse=True)
    torch.testing.assert_close(out.float(), o1.float(), rtol=0, atol=2 ** -7)
    torch.testing.assert_close(lse, l1, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n_shards", [1, 2, 8])
def test_config5_sequence_sharded_decode_full(n_shards):
    """The n per-GPU shards are run one after the other on this GPU; the cross-GPU exchange is then
    just the concatenation that the all-gather would produce."""
    from flash_b200 import dist as D
    from flash_b200 import ops
    g = _gen(5)
    b, L, h, hk, d = 8, 131072, 64, 8, 128
    q = torch.randn((b, 1, h, d), generator=g, device="cuda").to(BF)
    kc = torch.randn((b, L, hk, d), generator=g, device="cuda").to(BF)
    vc = torch.randn((b, L, hk, d), generator=g, device="cuda").to(BF)
    bufs = []
    for r in range(n_shards):
        lo, hi = D.kv_shard_range(L, n_shards, r)
        o, l = ops.attention_forward(q, kc[:, lo:hi], vc[:, lo:hi], softmax_scale=d ** -0.5, causal=True,
                                     kv_pos_offset=lo, kv_total=L, partial_out=True)
        assert o.dtype == torch.float32
        bufs.append(D.pack_partial(o, l))
    o_all, lse_all = D.unpack_gathered(torch.cat(bufs), n_shards, (b, 1, h, d), (b, h, 1))
    out, lse = ops.combine(o_all, lse_all, out_dtype=BF)
    lse = lse.permute(0, 2, 1)
    for i in [0, 7]:
        go, gl = OA.flash_attn_with_kvcache(q[i:i + 1].cpu(), kc[i:i + 1].cpu(), vc[i:i + 1].cpu(),
                                            cache_seqlens=L, causal=True)
        U.check_rules(out[i:i + 1], lse[i:i + 1], go, gl, tag=f"c5[{i}] n={n_shards}")
        assert float((lse[i].cpu() - gl[0]).abs().max()) < 1e-4
