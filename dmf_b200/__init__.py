"""B200-native (sm_100a) attention kernels behind Decoupled MeanFlow's flash_attn_func.

    from dmf_b200 import flash_attn_func            # (B, L, H, D) in / out, forward-AD aware
    from dmf_b200.dropin import install             # makes the reference's imports resolve here
"""

from .flash_attn_jvp import FlashAttnFunc, flash_attn_func, flash_attn_qkvpacked_func  # noqa: F401

__all__ = ["flash_attn_func", "flash_attn_qkvpacked_func", "FlashAttnFunc"]
