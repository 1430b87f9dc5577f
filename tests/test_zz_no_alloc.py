"""GPU: the allocation-free entry point ``fa_b200_fwd_noalloc`` against the regular
``fa_b200_fwd``, both called through the C ABI, twice in a row.

Who needs it: a host that is not allowed to allocate device memory while it runs (its memory was
partitioned at start-up, or another component owns the allocator).  The regular entry point wants a
caller-allocated workspace for the split-KV partials; this one keeps them in a fixed array inside
the library.  The two calls in a row check that nothing depends on the array's previous contents.
The file sorts last so that a run stopping at the first failure has already run everything else.
"""
import pytest
import torch

from flash_b200 import lib as L
from flash_b200 import ops
from oracle import api as OA

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _problem(seed, b, s_q, h, hk, d, s_cache):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((b, s_q, h, d), generator=g, device="cuda").to(BF)
    kc = torch.randn((b, s_cache, hk, d), generator=g, device="cuda").to(BF)
    vc = torch.randn((b, s_cache, hk, d), generator=g, device="cuda").to(BF)
    lens = torch.randint(s_cache // 4, s_cache, (b,), generator=g, device="cuda", dtype=torch.int32)
    return q, kc, vc, lens


def test_noalloc_matches_regular_entry_point_twice():
    lib = L.load()
    assert hasattr(lib, "fa_b200_fwd_noalloc")
    # The first call on a device loads the device image that holds the scratch array: a start-up cost by design.
    # From here on the driver's own count of free memory must not move (it sees a cudaMalloc that torch's
    # allocator statistics would miss).
    wq, wk, wv, wl = _problem(9, 1, 1, 8, 8, 128, 512)
    ops.attention_forward_noalloc(wq, wk, wv, torch.empty_like(wq), torch.empty((1, 8, 1), dtype=torch.float32, device="cuda"),
                                  seqused_k=wl, softmax_scale=128 ** -0.5, causal=True)
    torch.cuda.synchronize()
    for call, (seed, b, s_q, h, hk, s_cache) in enumerate([(1, 4, 1, 32, 8, 6000), (2, 2, 4, 64, 8, 9000)]):
        q, kc, vc, lens = _problem(seed, b, s_q, h, hk, 128, s_cache)
        kw = dict(seqused_k=lens, softmax_scale=128 ** -0.5, causal=True)
        ref_out, ref_lse, plan = ops.attention_forward(q, kc, vc, kernel=L.KERNEL_MMA, return_plan=True, **kw)
        assert plan.num_splits > 1 and plan.workspace_bytes > 0  # the path that needs scratch
        out = torch.full_like(q, float("nan"))
        lse = torch.full((b, h, s_q), float("nan"), dtype=torch.float32, device="cuda")
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        ops.attention_forward_noalloc(q, kc, vc, out, lse, **kw)
        assert torch.cuda.memory_allocated() == before  # no torch allocation either
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before  # ... and none behind torch's back
        # same kernels, same split plan: the tolerance of the other parity tests, and in fact equal bits
        torch.testing.assert_close(out.float(), ref_out.float(), rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(lse, ref_lse, rtol=1e-2, atol=1e-2)
        assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse), f"call {call}"
        if call == 0:  # and against the CPU oracle, so that both entry points cannot be wrong together
            go, gl = OA.flash_attn_with_kvcache(q.cpu(), kc.cpu(), vc.cpu(), cache_seqlens=lens.cpu(), causal=True)
            torch.testing.assert_close(out.float().cpu(), go.float(), rtol=1e-2, atol=1e-2)
            torch.testing.assert_close(lse.cpu(), gl, rtol=1e-2, atol=1e-2)


def test_noalloc_refuses_problems_beyond_its_scratch():
    q, kc, vc, lens = _problem(3, 64, 8, 64, 8, 128, 4096)
    out = torch.empty_like(q)
    lse = torch.empty((64, 64, 8), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="scratch"):
        # 16 splits x (64*64*8 rows) x 129 floats = 270 MB of partials: over the 32 MiB limit
        ops.attention_forward_noalloc(q, kc, vc, out, lse, seqused_k=lens, softmax_scale=0.088, causal=True,
                                      num_splits=16)


def test_noalloc_checks_its_tensors_before_any_launch():
    """A short lse, a mis-shaped out or 64-bit cache lengths would turn into out-of-bounds accesses on the device:
    the entry point has to refuse them on the host, like the regular one."""
    q, kc, vc, lens = _problem(4, 2, 1, 16, 8, 128, 1024)
    out = torch.empty_like(q)
    lse = torch.empty((2, 16, 1), dtype=torch.float32, device="cuda")
    kw = dict(softmax_scale=0.088, causal=True)
    n0 = L.load().fa_b200_launch_count()
    with pytest.raises(RuntimeError, match="lse must be"):
        ops.attention_forward_noalloc(q, kc, vc, out, lse[:, :8], seqused_k=lens, **kw)
    with pytest.raises(RuntimeError, match="lse must be"):
        ops.attention_forward_noalloc(q, kc, vc, out, lse.double(), seqused_k=lens, **kw)
    with pytest.raises(RuntimeError, match="out must have"):
        ops.attention_forward_noalloc(q, kc, vc, out[:, :, :8], lse, seqused_k=lens, **kw)
    with pytest.raises(RuntimeError, match="wrong dtype"):
        ops.attention_forward_noalloc(q, kc, vc, out.float(), lse, seqused_k=lens, **kw)
    with pytest.raises(RuntimeError, match="int32"):
        ops.attention_forward_noalloc(q, kc, vc, out, lse, seqused_k=lens.long(), **kw)
    with pytest.raises(RuntimeError, match="same dtype"):
        ops.attention_forward_noalloc(q, kc.half(), vc.half(), out, lse, seqused_k=lens, **kw)
    assert L.load().fa_b200_launch_count() == n0  # nothing reached the GPU
