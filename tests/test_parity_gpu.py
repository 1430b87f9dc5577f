"""GPU parity tests: the CUDA path, called through the drop-in Python modules (and so through the
C ABI of libfa_b200.so), against (a) the committed reference-golden fixtures and (b) the CPU
oracle on seeded inputs of shapes the reference's own test tables do not have (ragged packed
sequences, the host-buffer pipeline, tile-order chunks; the tables themselves are in
test_reference_tables_gpu.py).

Tolerance: the reference's rule rtol = atol = 1e-2 on O and LSE everywhere; its data_compare
helper and the 2x-error rule additionally on N(0,1) inputs (on U(-5,5) bf16 inputs data_compare
is reported but not asserted: two chunkings of the golden itself disagree under it).
"""
import itertools

import pytest
import torch

import golden_util as GU
import parity_util as U
from oracle import api as OA

pytestmark = pytest.mark.gpu

BF, FP = torch.bfloat16, torch.float16


def _cuda(x):
    return x.cuda() if isinstance(x, torch.Tensor) else x


# ----------------------------------------------------------------------------------------------
# (a) golden fixtures
# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", GU.fixture_names())
def test_fixture(name):
    import flash_attn_npu_v2 as fa2
    meta, inputs, expected = GU.load(name)
    kw = {k: _cuda(v) for k, v in GU.call_kwargs(meta, inputs).items()}
    fn = meta["fn"]
    if fn == "flash_attn_func":
        q, k, v = kw.pop("q"), kw.pop("k"), kw.pop("v")
        kw.pop("dropout_p", None)
        kw["return_attn_probs"] = True
        out, lse, _ = fa2.flash_attn_func(q, k, v, 0.0, **kw)
    elif fn == "flash_attn_varlen_func":
        out, lse, _ = fa2.flash_attn_varlen_func(**kw)
    else:
        q, kc, vc = kw.pop("q"), kw.pop("k_cache"), kw.pop("v_cache")
        kw.pop("k", None), kw.pop("v", None)
        out, lse = fa2.flash_attn_with_kvcache(q, kc, vc, None, None, **kw)
    torch.cuda.synchronize()
    assert out.shape == expected["out"].shape and out.dtype == expected["out"].dtype
    U.check_rules(out, lse, expected["out"], expected.get("lse"), strict_data_compare=False, tag=name)


# ----------------------------------------------------------------------------------------------
# (b) the reference's case tables live in test_reference_tables_gpu.py (all rows); below: shapes they do not have
# ----------------------------------------------------------------------------------------------
def test_varlen_ragged_lengths():
    """Ragged, including an empty sequence (the reference tables only use equal lengths)."""
    import flash_attn_npu_v2 as fa2
    g = torch.Generator().manual_seed(99)
    q_lens, k_lens = [5, 0, 130, 64, 1], [77, 10, 130, 300, 1]
    cq = torch.tensor([0] + list(itertools.accumulate(q_lens)), dtype=torch.int32)
    ck = torch.tensor([0] + list(itertools.accumulate(k_lens)), dtype=torch.int32)
    q = U.normal((sum(q_lens), 6, 128), BF, g)
    k = U.normal((sum(k_lens), 2, 128), BF, g)
    v = U.normal((sum(k_lens), 2, 128), BF, g)
    for causal in (False, True):
        gold_out, gold_lse = OA.flash_attn_varlen_func(q, k, v, cq, ck, max(q_lens), max(k_lens), causal=causal)
        out, lse, _ = fa2.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cq.cuda(), ck.cuda(), max(q_lens),
                                                 max(k_lens), causal=causal, return_attn_probs=True)
        U.check_rules(out, lse, gold_out, gold_lse, tag=f"ragged causal={causal}")


@pytest.mark.parametrize("d,softcap", [(128, 0.0), (64, 0.0), (128, 30.0), (64, 30.0), (256, 0.0), (192, 30.0), (96, 0.0)])
def test_varlen_ragged_lengths_tcgen05(d, softcap):
    """Ragged packed sequences on the tcgen05 kernel (tile widths 64, 128 and 256 columns, head dims in between, with and
    without softcap): tiles that run
    into the next sequence, an empty sequence, queries longer than the keys (rows without a visible key), GQA, a
    sliding window."""
    from flash_b200 import lib as L
    from flash_b200 import ops
    g = torch.Generator().manual_seed(123)
    q_lens, k_lens = [300, 0, 77, 513, 700], [300, 40, 77, 900, 100]
    cq = torch.tensor([0] + list(itertools.accumulate(q_lens)), dtype=torch.int32)
    ck = torch.tensor([0] + list(itertools.accumulate(k_lens)), dtype=torch.int32)
    q = U.normal((sum(q_lens), 4, d), BF, g)
    k = U.normal((sum(k_lens), 2, d), BF, g)
    v = U.normal((sum(k_lens), 2, d), BF, g)
    scale = 1.0 / d ** 0.5
    for causal, window in ((False, (-1, -1)), (True, (-1, -1)), (True, (200, 0))):
        gold_out, gold_lse = OA.flash_attn_varlen_func(q, k, v, cq, ck, max(q_lens), max(k_lens), softmax_scale=scale,
                                                       causal=causal, window_size=window, softcap=softcap)
        out, lse, plan = ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), softmax_scale=scale, causal=causal,
                                               window_left=window[0], window_right=window[1], softcap=softcap,
                                               cu_seqlens_q=cq.cuda(), cu_seqlens_k=ck.cuda(),
                                               max_seqlen_q=max(q_lens), max_seqlen_k=max(k_lens), return_plan=True)
        assert plan.kernel == L.KERNEL_TCGEN05
        assert L.load().fa_b200_check_status(torch.cuda.current_stream().cuda_stream) == 0
        U.check_rules(out, lse, gold_out, gold_lse, tag=f"tcgen05 ragged d={d} softcap={softcap} causal={causal} window={window}")


@pytest.mark.gpu
def test_host_buffer_pipeline_matches_the_device_call():
    """flash_b200.host.HostPrefill (pinned host tensors in and out, batch chunks overlapped on three streams)
    returns bit for bit what one call on device tensors returns, step after step."""
    from flash_b200 import ops
    from flash_b200.host import HostPrefill
    g = torch.Generator().manual_seed(11)
    b, s, h, hk, d = 5, 384, 4, 2, 128
    q = (torch.randn((b, s, h, d), generator=g)).to(torch.bfloat16).pin_memory()
    k = (torch.randn((b, s, hk, d), generator=g)).to(torch.bfloat16).pin_memory()
    v = (torch.randn((b, s, hk, d), generator=g)).to(torch.bfloat16).pin_memory()
    out = torch.empty_like(q).pin_memory()
    lse = torch.empty((b, h, s), dtype=torch.float32).pin_memory()
    pipe = HostPrefill(q.shape, k.shape, torch.bfloat16, chunks=3)
    assert pipe.bounds == [(0, 1), (1, 3), (3, 5)]
    ref_o, ref_l = ops.attention_forward(q.cuda(), k.cuda(), v.cuda(), softmax_scale=d ** -0.5, causal=True)
    for _ in range(3):
        out.zero_()
        pipe(q, k, v, out, lse, softmax_scale=d ** -0.5, causal=True)
        torch.cuda.synchronize()
        assert torch.equal(out, ref_o.cpu()) and torch.equal(lse, ref_l.cpu())
    for _ in range(3):  # steps streamed back to back: the next copies in run under the previous copies out
        pipe(q, k, v, out, lse, after_current_stream=False, softmax_scale=d ** -0.5, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(out, ref_o.cpu()) and torch.equal(lse, ref_l.cpu())
    with pytest.raises(RuntimeError, match="host tensor"):
        pipe(q.cuda(), k, v, out, lse, softmax_scale=d ** -0.5, causal=True)


@pytest.mark.gpu
def test_tile_order_chunks_do_not_change_the_result(monkeypatch):
    """The tcgen05 prefill kernel orders its tiles in chunks of (batch, head) pairs whose K / V stay in L2.  Any chunk
    length (a tuning override here, incl. one that leaves a short last chunk) gives bit-identical O and LSE."""
    from flash_b200 import ops
    g = torch.Generator().manual_seed(21)
    b, s, h, hk, d = 3, 700, 6, 2, 128  # 18 pairs x 3 query tiles
    q, k, v = [U.normal((b, s, n, d), torch.bfloat16, g).cuda() for n in (h, hk, hk)]
    monkeypatch.setenv("FA_B200_TC5_CHUNK", "0")
    ref_o, ref_l = ops.attention_forward(q, k, v, softmax_scale=d ** -0.5, causal=True)
    for chunk in ("1", "4", "5", "18", "100"):
        monkeypatch.setenv("FA_B200_TC5_CHUNK", chunk)
        o, l = ops.attention_forward(q, k, v, softmax_scale=d ** -0.5, causal=True)
        torch.cuda.synchronize()
        assert torch.equal(o, ref_o) and torch.equal(l, ref_l), f"chunk {chunk}"
    # packed varlen input with ragged lengths (an empty sequence among them)
    lens = [300, 0, 700, 129, 512]
    cu = torch.tensor([0] + list(itertools.accumulate(lens)), dtype=torch.int32).cuda()
    tot = sum(lens)
    q, k, v = [U.normal((tot, n, d), torch.bfloat16, g).cuda() for n in (h, hk, hk)]
    kw = dict(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens), softmax_scale=d ** -0.5, causal=True)
    monkeypatch.setenv("FA_B200_TC5_CHUNK", "0")
    ref_o, ref_l = ops.attention_forward(q, k, v, **kw)
    for chunk in ("1", "7", "29"):
        monkeypatch.setenv("FA_B200_TC5_CHUNK", chunk)
        o, l = ops.attention_forward(q, k, v, **kw)
        torch.cuda.synchronize()
        assert torch.equal(o, ref_o) and torch.equal(l, ref_l), f"varlen chunk {chunk}"
