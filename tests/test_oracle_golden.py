"""CPU: the oracle restatement reproduces the reference golden outputs stored in
tests/golden/ (produced by the reference's ref_flash_attention + in-test masks and
dead-row patch-up).  This is what pins the oracle."""
import pytest
import torch

import golden_util as GU
from oracle import api as OA
from oracle import golden as OG


def run_oracle(meta, inputs):
    kw = GU.call_kwargs(meta, inputs)
    fn = meta["fn"]
    if fn == "flash_attn_func":
        return OA.flash_attn_func(kw["q"], kw["k"], kw["v"], softmax_scale=kw.get("softmax_scale"),
                                  causal=kw.get("causal", False), window_size=kw.get("window_size", (-1, -1)),
                                  softcap=kw.get("softcap", 0.0))
    if fn == "flash_attn_varlen_func":
        return OA.flash_attn_varlen_func(kw["q"], kw["k"], kw["v"], kw["cu_seqlens_q"], kw["cu_seqlens_k"],
                                         kw["max_seqlen_q"], kw["max_seqlen_k"], softmax_scale=kw["softmax_scale"],
                                         causal=kw["causal"], window_size=kw["window_size"], softcap=kw["softcap"])
    assert fn == "flash_attn_with_kvcache"
    return OA.flash_attn_with_kvcache(kw["q"], kw["k_cache"], kw["v_cache"], cache_seqlens=kw["cache_seqlens"],
                                      block_table=kw.get("block_table"), causal=kw["causal"],
                                      window_size=kw["window_size"], softcap=kw["softcap"])


@pytest.mark.parametrize("name", GU.fixture_names())
def test_oracle_matches_reference_golden(name):
    meta, inputs, expected = GU.load(name)
    out, lse = run_oracle(meta, inputs)
    # Same algorithm, same fp32 chunking: at most one unit in the last place of the 16-bit
    # output (different BLAS batching of the same fp32 sums) and 1e-5 on the fp32 LSE.
    exp = expected["out"].float()
    ulp = 2.0 ** -7 if expected["out"].dtype == torch.bfloat16 else 2.0 ** -10
    assert out.shape == expected["out"].shape
    diff = (out.float() - exp).abs()
    assert bool((diff <= ulp * exp.abs().clamp_min(2.0 ** -14) + 1e-7).all()), float(diff.max())
    assert float((diff > 0).float().mean()) < 0.01
    if "lse" in expected:
        e = expected["lse"]
        assert lse.shape == e.shape
        assert torch.equal(torch.isinf(lse), torch.isinf(e))
        fin = ~torch.isinf(e)
        torch.testing.assert_close(lse[fin], e[fin], rtol=1e-5, atol=1e-5)


def test_blockwise_matches_dense_fp32():
    g = torch.Generator().manual_seed(7)
    q = torch.randn(37, 4, 64, generator=g).to(torch.bfloat16)
    k = torch.randn(700, 2, 64, generator=g).to(torch.bfloat16)
    v = torch.randn(700, 2, 64, generator=g).to(torch.bfloat16)
    mask = OG.build_mask(37, 700, True, False, -1, 0)
    o1, l1 = OG.blockwise_attention(q, k, v, 0.125, mask, torch.bfloat16, round_p=False)
    o2, l2 = OG.dense_softmax_attention(q, k, v, 0.125, mask)
    torch.testing.assert_close(o1.float(), o2.float(), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(l1, l2, rtol=1e-5, atol=1e-5)


def test_window_normalisation_rules():
    # csrc/arch22/flash_attn_npu_v2/flash_api.cpp:483-494
    assert OG.normalize_window(64, 192, False, 32, 64) == (False, True, 32, -1)
    assert OG.normalize_window(1024, 1024, True, 512, 256) == (False, True, 512, 0)
    assert OG.normalize_window(1024, 1024, True, -128, 864) == (True, False, -128, 0)
    assert OG.normalize_window(512, 512, False, 508, -256) == (False, True, 508, -256)
    assert OG.normalize_window(128, 512, True, 511, 0) == (True, False, -1, 0)
    assert OG.normalize_window(4, 100, False, -1, -1) == (False, False, -1, -1)
