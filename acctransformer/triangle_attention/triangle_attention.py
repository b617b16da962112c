"""Same module path as the reference's layer (train/acctransformer/triangle_attention/triangle_attention.py:28-165)."""
from acctransformer_b200.triangle_attention.triangle_attention import TriangleAttention

__all__ = ["TriangleAttention"]
