"""B200-native drop-in for ``flag_attn.flash_attention``."""
from .flash import (FlashAttentionFunction, check_device_status, flash_attention,  # noqa: F401
                    flash_attention_split_kv)
from .paged import paged_attention  # noqa: F401
from .piecewise import piecewise_attention  # noqa: F401

__all__ = ["flash_attention", "flash_attention_split_kv", "paged_attention", "piecewise_attention",
           "FlashAttentionFunction",
           "check_device_status"]
__version__ = "0.2.0"
