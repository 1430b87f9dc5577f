"""Drop-in ``flash_attn_npu_v2`` backed by the B200 (sm_100a) library.

Mirrors flash_attn_npu_v2/__init__.py of the reference (:1-23): same version string and
exports.  The reference gates on the NPU device name; here the gate is a CUDA device of
compute capability 10.x, checked lazily at the first call so that the module imports on a
machine without a GPU (the native library itself still has to be present).
"""
__version__ = "0.1.1"

from flash_b200 import lib as _lib

_lib.load()  # no fallback: fail at import when libfa_b200.so is missing

from .interface import (  # noqa: E402
    flash_attn_func,
    flash_attn_kvpacked_func,
    flash_attn_qkvpacked_func,
    flash_attn_varlen_func,
    flash_attn_varlen_kvpacked_func,
    flash_attn_varlen_qkvpacked_func,
    flash_attn_with_kvcache,
)

__all__ = [
    "flash_attn_func",
    "flash_attn_kvpacked_func",
    "flash_attn_qkvpacked_func",
    "flash_attn_varlen_func",
    "flash_attn_varlen_kvpacked_func",
    "flash_attn_varlen_qkvpacked_func",
    "flash_attn_with_kvcache",
]
