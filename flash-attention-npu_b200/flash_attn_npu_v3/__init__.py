"""Drop-in ``flash_attn_npu_v3`` backed by the B200 (sm_100a) library.

Mirrors flash_attn_npu_v3/__init__.py of the reference (:1-28): same version string and the
arch22 export list (the arch35 variant of the reference exports only flash_attn_with_kvcache,
with the same signature; one B200 backend serves both).
"""
__version__ = "0.1.1"

from flash_b200 import lib as _lib

_lib.load()  # no fallback: fail at import when libfa_b200.so is missing

from .interface import (  # noqa: E402
    flash_attn_func,
    flash_attn_varlen_func,
    flash_attn_with_kvcache,
    get_scheduler_metadata,
)

__all__ = ["flash_attn_func", "flash_attn_varlen_func", "flash_attn_with_kvcache", "get_scheduler_metadata"]
