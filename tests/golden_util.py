"""Loader for the committed golden fixtures (tests/golden/*.npz, written by
tests/golden/make_golden.py from the reference's own test code)."""
import glob
import json
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def fixture_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def _to_torch(a, tag):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.view(torch.bfloat16) if tag == "bf16" else t


def load(name):
    """Returns (meta, inputs, expected): tensors as torch CPU tensors in their original dtypes.
    Paged caches are zero-padded back to the number of blocks the reference test allocated."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    inputs, expected = {}, {}
    for key in z.files:
        if key == "meta":
            continue
        t = _to_torch(z[key], meta["dtypes"][key])
        if key.startswith("in_"):
            inputs[key[3:]] = t
        else:
            expected[key[4:]] = t
    sc = meta.get("scalars", {})
    for key in ("k_cache", "v_cache"):
        nb = sc.pop(key + "_num_blocks", None)
        if nb is not None and key in inputs and inputs[key].shape[0] < nb:
            pad = torch.zeros((nb - inputs[key].shape[0],) + tuple(inputs[key].shape[1:]), dtype=inputs[key].dtype)
            inputs[key] = torch.cat([inputs[key], pad])
    return meta, inputs, expected


def call_kwargs(meta, inputs):
    """Keyword arguments for the public API function named by meta['fn']."""
    kw = dict(inputs)
    for k, v in meta.get("scalars", {}).items():
        kw[k] = tuple(v) if isinstance(v, list) else v
    return kw
