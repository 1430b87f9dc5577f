"""The three acceptance rules applied to GPU outputs (test infrastructure).

1. the reference tests' own rule: assert_close(rtol=1e-2, atol=1e-2) on O and LSE
   (tests/test_flash_attn_npu_v2.py:404-407 of the reference);
2. ``data_compare`` of the reference's tests/precision_compare.py:109-166, restated with numpy:
   relative difference (denominator floor of cal_relative_diff_np :15-21) above 0.005 on at
   most 0.5 % of the elements, and a maximum relative difference below 0.1;
3. the 2x rule: max|out - gold| <= 2 * max|out_plain - gold| where out_plain is a plain
   attention evaluated in the input dtype (a 1e-5 floor keeps the bound non-zero).
"""
import numpy as np
import torch

RTOL = 1e-2
ATOL = 1e-2


def assert_close_rule(out, gold_out, lse=None, gold_lse=None):
    torch.testing.assert_close(out.float().cpu(), gold_out.float().cpu(), rtol=RTOL, atol=ATOL)
    if lse is not None:
        a, b = lse.float().cpu(), gold_lse.float().cpu()
        assert torch.equal(torch.isinf(a), torch.isinf(b)), "dead rows (LSE = +inf) differ"
        assert bool((a[torch.isinf(a)] > 0).all())
        fin = ~torch.isinf(b)
        torch.testing.assert_close(a[fin], b[fin], rtol=RTOL, atol=ATOL)


def relative_diff(real, expect, diff_thd):
    a = np.abs(real - expect)
    b1 = np.maximum(np.abs(real), np.abs(expect))
    b2 = float((1.0 / (1 << 14)) / diff_thd)
    b = np.maximum(b1, b2) + 10e-10
    return np.where(a < diff_thd, a, a / b)


def data_compare(out, gold, diff_thd=0.005, pct_thd=0.005, max_diff_hd=0.1):
    """Returns (result, fulfil_percent, max_error) like the reference helper."""
    real = out.detach().float().cpu().numpy().reshape(-1)
    exp = gold.detach().float().cpu().numpy().reshape(-1)
    if real.size == 0:
        return "success", 100.0, 0.0
    assert real.size == exp.size
    idx = np.where(np.abs(real - exp) > 0)[0]
    rdiff = relative_diff(real[idx], exp[idx], diff_thd)
    err = rdiff[rdiff > diff_thd]
    pct = float(real.size - err.size) / float(real.size) * 100.0
    result = "success" if pct >= (1 - pct_thd) * 100.0 else "failed"
    max_err = float(err.max()) if err.size else 0.0
    if max_err >= max_diff_hd:
        result = "failed"
    return result, pct, max_err


def two_x_rule(out, gold, out_plain, floor=1e-5):
    """Returns (ok, err, bound)."""
    g = gold.float().cpu()
    err = float((out.float().cpu() - g).abs().max())
    base = float((out_plain.float().cpu() - g).abs().max())
    bound = 2.0 * max(base, floor)
    return err <= bound, err, bound
