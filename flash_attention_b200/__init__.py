"""B200-native exact attention with the public API of FlashAttention v2.3.3.

    from flash_attention_b200 import flash_attn_func, flash_attn_with_kvcache, ...

The compute path is libfa_b200.so (hand-written sm_100a CUDA, C ABI in include/fa_b200.h) reached
through the drop-in extension module `flash_attn_2_cuda` of this repository.
"""
__version__ = "0.1.0"

from flash_attention_b200.flash_attn_interface import (  # noqa: E402,F401
    flash_attn_func,
    flash_attn_kvpacked_func,
    flash_attn_qkvpacked_func,
    flash_attn_varlen_func,
    flash_attn_varlen_kvpacked_func,
    flash_attn_varlen_qkvpacked_func,
    flash_attn_with_kvcache,
)
