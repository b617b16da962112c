"""Same module path as the reference's op registration
(train/acctransformer/flash_attention/ops/flash_attention/flash_attention_impl.py:96-154)."""
from acctransformer_b200.flash_attention.ops.flash_attention.flash_attention_impl import (get_flash_attention,
                                                                                           get_flash_attention_grad)

__all__ = ["get_flash_attention", "get_flash_attention_grad"]
