"""pytest configuration: registers the ``gpu`` marker and puts the package directory
(which holds the drop-in ``flash_attn_npu_v2`` / ``flash_attn_npu_v3`` modules) and the
repository root (for ``oracle``) on ``sys.path``."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-attention-npu_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
