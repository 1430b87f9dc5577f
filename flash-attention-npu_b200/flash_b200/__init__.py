"""B200 backend of the flash_attn_npu_v2 / flash_attn_npu_v3 drop-in modules.

``ops.attention_forward`` / ``ops.combine`` wrap the C ABI of libfa_b200.so;
``dist`` holds the multi-GPU helpers (sharding, cross-GPU merge of partials).
"""
from . import lib, ops  # noqa: F401

__all__ = ["lib", "ops"]
