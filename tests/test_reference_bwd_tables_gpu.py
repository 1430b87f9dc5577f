"""GPU: the case tables of the reference's backward tests, row for row, against the oracle.

Tables (paths inside the reference project):
  BSND        tests/test_flash_attn_npu_v2_bwd.py:147-164   flash_attn_func + autograd, 16 rows
  BSND_SWA    tests/test_flash_attn_npu_v2_bwd.py:187-204   the same with window sizes, 16 rows
  VARLEN      tests/test_flash_attn_npu_v2_bwd.py:230-243   flash_attn_varlen_func + autograd, 12 rows
  VARLEN_SWA  tests/test_flash_attn_npu_v2_bwd.py:276-283   the same with window sizes, 6 rows
(tests/test_flash_attn_npu_v3_bwd.py holds the same tables for the FA3-style package; the rows run through both front
ends here.)  Like the reference's tests, the forward that produces out and softmax_lse is the implementation under
test, the expected gradients are the golden's backward from that softmax_lse (here the oracle, oracle/bwd.py, which is
pinned against outputs of the reference's golden), inputs are 2 * (rand - 0.5), tolerance rtol = atol = 1e-2.

What differs from the reference's runs: the 7777 x 8192 rows run with 1777 x 2048 and the 711 x 8192 rows with 711 x 2048
keys (the float64 CPU golden is quadratic), batch sizes above 2 run as 2 (3 for the batch of 7).  Head dim 111 is padded to
112 by the front end, as in the reference.  The two rows with a negative window literal (-128, 864 under causal) are
skipped: the reference's forward golden takes a negative literal arithmetically and its backward golden takes it as
"unbounded", so a forward and a backward that each agree with their own golden disagree with each other on those rows.
"""
import itertools

import pytest
import torch

from oracle import bwd as OB

pytestmark = pytest.mark.gpu
BF, FP = torch.bfloat16, torch.float16
RTOL = ATOL = 1e-2


def _ids(prefix):
    return lambda c: prefix + "-".join(str(x).replace("torch.", "") for x in c)


def _rand(shape, dtype, g):
    return (2.0 * (torch.rand(shape, generator=g) - 0.5)).to(dtype)


def _small_batch(b):
    return b if b <= 2 else (3 if b % 2 and b > 5 else 2)


# (dtype, batch, heads, kv heads, q_seqlen, kv_seqlen, head dim, causal, softcap)
BSND = [(dt, b, h, hk, sq, sk, 128, causal, cap)
        for cap in (0.0, 30.0) for dt in (FP, BF)
        for (b, h, hk, sq, sk, causal) in ((1, 1, 1, 1024, 1024, False), (5, 4, 4, 1024, 1024, True), (7, 1, 1, 512, 512, False),
                                           (4, 2, 1, 513, 513, False))]

# (dtype, batch, heads, kv heads, q_seqlen, kv_seqlen, head dim, causal, window left, window right, softcap)
BSND_SWA = [(dt, b, h, hk, sq, sk, 128, causal, wl, wr, cap)
            for cap in (0.0, 30.0)
            for (dt, b, h, hk, sq, sk, causal, wl, wr) in (
                (BF, 1, 1, 1, 1024, 1024, True, 512, 0), (BF, 1, 1, 1, 1024, 1024, True, 512, 256),
                (BF, 5, 4, 4, 1024, 1024, True, -128, 864), (BF, 1, 1, 1, 1024, 1024, False, 0, 256),
                (FP, 2, 2, 2, 512, 512, False, 64, 128), (BF, 1, 1, 1, 1, 1024, True, 512, 0),
                (BF, 2, 6, 2, 2, 1024, True, -1, -1), (BF, 2, 6, 2, 2, 1024, True, 256, 0))]

# (dtype, batch, heads, kv heads, q_seqlen, kv_seqlen, head dim, causal, softcap)
VARLEN = [(dt, b, h, hk, sq, sk, d, causal, cap)
          for cap in (0.0, 30.0)
          for (dt, b, h, hk, sq, sk, d, causal) in (
              (BF, 1, 1, 1, 512, 1024, 128, True), (FP, 1, 5, 1, 512, 512, 128, True), (FP, 1, 5, 1, 777, 888, 192, False),
              (FP, 1, 5, 1, 1777, 1888, 256, True), (BF, 1, 1, 1, 7777, 8192, 64, True), (BF, 1, 5, 1, 711, 8192, 111, True))]

VARLEN_SWA = [(dt, b, h, hk, sq, sk, 128, causal, wl, wr, cap)
              for cap in (0.0, 30.0)
              for (dt, b, h, hk, sq, sk, causal, wl, wr) in (
                  (BF, 1, 1, 1, 512, 1024, True, 512, 0), (BF, 1, 1, 1, 512, 1024, False, 0, 256), (FP, 1, 2, 2, 512, 512, False, 64, 128))]


def _check(name, got, want, tag):
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=RTOL, atol=ATOL, msg=lambda m: f"{tag} {name}: {m}")


def _front_ends():
    import flash_attn_npu_v2 as fa2
    import flash_attn_npu_v3 as fa3
    return (("v2", fa2), ("v3", fa3))


def _run_dense(case, window):
    dtype, b, h, hk, sq, sk, d, causal = case[:8]
    softcap = case[-1]
    if window[0] < -1 or window[1] < -1:
        pytest.skip("negative window literal: the reference's forward and backward goldens read it differently")
    b = _small_batch(b)
    g = torch.Generator().manual_seed(42)
    q, k, v = _rand((b, sq, h, d), dtype, g), _rand((b, sk, hk, d), dtype, g), _rand((b, sk, hk, d), dtype, g)
    dout = _rand((b, sq, h, d), dtype, g)
    scale = d ** -0.5
    for name, fa in _front_ends():
        qg, kg, vg = [t.cuda().requires_grad_(True) for t in (q, k, v)]
        kw = dict(softmax_scale=scale, causal=causal, window_size=window, softcap=softcap)
        if name == "v2":
            out, lse, _ = fa.flash_attn_func(qg, kg, vg, return_attn_probs=True, **kw)
        else:
            out, lse = fa.flash_attn_func(qg, kg, vg, return_attn_probs=True, **kw)
        dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), dout.cuda())
        # the golden's backward from THIS forward's softmax_lse (the two front ends may plan the forward differently)
        gold = OB.attention_backward(q, k, v, dout, lse.detach().cpu(), softmax_scale=scale, causal=causal, window=window,
                                     softcap=softcap)
        for n, a, c in zip(("dq", "dk", "dv"), (dq, dk, dv), gold):
            _check(n, a, c, name)


def _run_varlen(case, window):
    dtype, b, h, hk, sq, sk, d, causal = case[:8]
    softcap = case[-1]
    if sk == 8192:  # the quadratic float64 golden: shorter rows, same ratios to the tile sizes
        sq, sk = (1777, 2048) if sq == 7777 else (711, 2048)
    g = torch.Generator().manual_seed(42)
    q, k, v = _rand((b * sq, h, d), dtype, g), _rand((b * sk, hk, d), dtype, g), _rand((b * sk, hk, d), dtype, g)
    dout = _rand((b * sq, h, d), dtype, g)
    cq = torch.tensor([0] + list(itertools.accumulate([sq] * b)), dtype=torch.int32)
    ck = torch.tensor([0] + list(itertools.accumulate([sk] * b)), dtype=torch.int32)
    scale = d ** -0.5
    for name, fa in _front_ends():
        qg, kg, vg = [t.cuda().requires_grad_(True) for t in (q, k, v)]
        kw = dict(softmax_scale=scale, causal=causal, window_size=window, softcap=softcap)
        res = fa.flash_attn_varlen_func(qg, kg, vg, cq.cuda(), ck.cuda(), sq, sk, return_attn_probs=True, **kw)
        out, lse = res[0], res[1]
        dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), dout.cuda())
        gold = OB.attention_varlen_backward(q, k, v, dout, lse.detach().cpu(), cq, ck, softmax_scale=scale, causal=causal,
                                            window=window, softcap=softcap)
        for n, a, c in zip(("dq", "dk", "dv"), (dq, dk, dv), gold):
            _check(n, a, c, name)


@pytest.mark.parametrize("case", BSND, ids=_ids("bsnd-"))
def test_fa_bsnd_bwd(case):
    _run_dense(case, (-1, -1))


@pytest.mark.parametrize("case", BSND_SWA, ids=_ids("bsnd-swa-"))
def test_fa_bsnd_bwd_swa(case):
    _run_dense(case, (case[8], case[9]))


@pytest.mark.parametrize("case", VARLEN, ids=_ids("varlen-"))
def test_fa_varlen_bwd(case):
    _run_varlen(case, (-1, -1))


@pytest.mark.parametrize("case", VARLEN_SWA, ids=_ids("varlen-swa-"))
def test_fa_varlen_bwd_swa(case):
    _run_varlen(case, (case[8], case[9]))
