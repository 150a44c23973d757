"""The RTN part of the reference's gradual-quantization package (bitween/gradual/): the
per-block RTN loop and a cache for its repeated (bits, group_size) trials."""
from .base_wrapper import BaseBlockWrapper, RTNWrapper, quantize_block
from .rtn_cache import RTNCache, default_cache

__all__ = ["BaseBlockWrapper", "RTNWrapper", "quantize_block", "RTNCache", "default_cache"]
