"""Generate tests/golden/bwd/*.npz by EXECUTING the reference's backward golden (run once, where the
reference checkout is available):

    python tests/golden/make_golden_bwd.py /path/to/reference

The reference's tests/fa_small_op_golden.py is pure PyTorch and is imported as it is.  Its backward golden takes the
forward's out / softmax_lse as inputs; here they come from this repository's CPU oracle of the forward (itself pinned
by the forward fixtures).  Inputs follow the reference's backward tests (tests/test_flash_attn_npu_v2_bwd.py:75-76:
2 * (rand - 0.5), seeded).  Each fixture stores q, k, v, dout, lse and the golden dq, dk, dv.
"""
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import api as OA  # noqa: E402


def to_np(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy(), "bf16"
    return t.numpy(), {torch.float16: "fp16", torch.float32: "fp32", torch.int32: "i32"}[t.dtype]


def rand(shape, dtype, g):
    return (2.0 * (torch.rand(shape, generator=g) - 0.5)).to(dtype)


CASES = [
    # name, dtype, varlen lens (or None), b, s_q, s_k, h, h_k, d, causal, window, softcap
    ("bsnd_causal_gqa_bf16", torch.bfloat16, None, 2, 96, 160, 4, 2, 64, True, (-1, -1), 0.0),
    ("bsnd_full_fp16_d128", torch.float16, None, 1, 130, 70, 2, 2, 128, False, (-1, -1), 0.0),
    ("bsnd_window_bf16", torch.bfloat16, None, 1, 128, 128, 2, 1, 64, False, (40, 10), 0.0),
    ("tnd_causal_ragged_bf16", torch.bfloat16, ([70, 1, 130], [100, 33, 130]), 3, 130, 130, 4, 2, 64, True, (-1, -1), 0.0),
    ("bsnd_softcap_fp16", torch.float16, None, 1, 100, 100, 2, 1, 64, True, (-1, -1), 30.0),
]


def main(ref_root):
    spec = importlib.util.spec_from_file_location("fa_small_op_golden", os.path.join(ref_root, "tests", "fa_small_op_golden.py"))
    G = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(G)
    out_dir = os.path.join(HERE, "bwd")
    os.makedirs(out_dir, exist_ok=True)
    for ci, (name, dtype, lens, b, s_q, s_k, h, h_k, d, causal, window, softcap) in enumerate(CASES):
        g = torch.Generator().manual_seed(42 + ci)
        scale = d ** -0.5
        if lens is None:
            q, k, v = rand((b, s_q, h, d), dtype, g), rand((b, s_k, h_k, d), dtype, g), rand((b, s_k, h_k, d), dtype, g)
            dout = rand((b, s_q, h, d), dtype, g)
            out, lse = OA.flash_attn_func(q, k, v, softmax_scale=scale, causal=causal, window_size=window, softcap=softcap)
            dq, dk, dv = G.golden_bsnd_bwd_from_fwd(q, k, v, dout, out, lse, h, h_k, scale, softcap, 0.0, causal, window[0], window[1])
            extra = {}
        else:
            lq, lk = lens
            cq = torch.tensor([0] + list(np.cumsum(lq)), dtype=torch.int32)
            ck = torch.tensor([0] + list(np.cumsum(lk)), dtype=torch.int32)
            q, k, v = rand((sum(lq), h, d), dtype, g), rand((sum(lk), h_k, d), dtype, g), rand((sum(lk), h_k, d), dtype, g)
            dout = rand((sum(lq), h, d), dtype, g)
            out, lse = OA.flash_attn_varlen_func(q, k, v, cq, ck, max(lq), max(lk), softmax_scale=scale, causal=causal,
                                                 window_size=window, softcap=softcap)
            dq, dk, dv = G.golden_tnd_bwd_from_fwd(q, k, v, dout, out, lse, h, h_k, lq, lk, scale, softcap, 0.0, causal,
                                                   window[0], window[1])
            extra = {"cu_seqlens_q": cq, "cu_seqlens_k": ck}
        arrays, dtypes = {}, {}
        for key, t in dict(q=q, k=k, v=v, dout=dout, out=out, lse=lse, dq=dq, dk=dk, dv=dv, **extra).items():
            arrays[key], dtypes[key] = to_np(t)
        meta = {"dtypes": dtypes, "scale": scale, "causal": causal, "window": list(window), "varlen": lens is not None, "softcap": softcap,
                "source": "tests/fa_small_op_golden.py golden_bsnd_bwd_from_fwd / golden_tnd_bwd_from_fwd"}
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), meta=json.dumps(meta), **arrays)
        print(name, "ok", {k_: tuple(v_.shape) for k_, v_ in arrays.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python " + sys.argv[0] + " /path/to/reference")
    main(sys.argv[1])
