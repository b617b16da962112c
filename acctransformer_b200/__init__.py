"""B200-native attention hot path of acctransformer: FlashAttention2 forward/backward,
TriangleAttention and the inference prefill/decode op behind the reference's Python signatures,
running hand-written sm_100a CUDA through the C ABI in ``include/acct_b200.h``."""

__all__ = ["FlashAttention", "TriangleAttention", "get_flash_attention", "get_flash_attention_grad",
           "FlashAttentionTik", "flash_attention_tik", "flash_attention_decode"]


def __getattr__(name):
    if name == "FlashAttention":
        from .flash_attention.nn.layer.flash_attention import FlashAttention
        return FlashAttention
    if name == "TriangleAttention":
        from .triangle_attention.triangle_attention import TriangleAttention
        return TriangleAttention
    if name in ("get_flash_attention", "get_flash_attention_grad"):
        from .flash_attention.ops.flash_attention import flash_attention_impl as m
        return getattr(m, name)
    if name in ("FlashAttentionTik", "flash_attention_tik", "flash_attention_decode"):
        from .infer import flash_attention as m
        return getattr(m, name)
    raise AttributeError(name)
