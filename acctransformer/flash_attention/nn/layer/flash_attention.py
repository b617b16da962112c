"""Same module path as the reference's cell (train/acctransformer/flash_attention/nn/layer/flash_attention.py:31-207)."""
from acctransformer_b200.flash_attention.nn.layer.flash_attention import HEAD_DIM_MAX_LIMIT, FlashAttention

__all__ = ['FlashAttention']
