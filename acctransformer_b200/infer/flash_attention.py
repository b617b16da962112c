"""The inference attention op and its decode companion.

``FlashAttentionTik`` mirrors the reference's custom op ``FlashAttentionTik(q, k, v) -> y``
(infer/flash_attention/tik/op_proto/flash_attention_tik.h:22-27; kernel entry
infer/flash_attention/tik/tbe/impl/flash_attention_tik.py:8-16): ``y = softmax(q k^T) v`` on fp16
rank-3 ``[B*N, S, D]`` or rank-4 ``[B, N, S, D]`` inputs, y shaped like q, no scale and no mask.
``scale``, ``causal`` and ``seq_lens`` are additions (all off by default).  Shape errors raise
``ValueError`` where the reference's InferShape returns GRAPH_FAILED
(op_proto/flash_attention_tik.cpp:160-193).

``flash_attention_decode`` is the q_len = 1 step over a KV cache with per-sequence valid lengths;
the reference has no such path.
"""
from __future__ import annotations

import torch

from .. import ops as _ops

__all__ = ["FlashAttentionTik", "flash_attention_tik", "flash_attention_decode", "DecodeWorkspace"]

DecodeWorkspace = _ops.DecodeWorkspace


def flash_attention_tik(q, k, v, *, scale=1.0, causal=False, seq_lens=None):
    if q.dim() not in (3, 4):
        raise ValueError("the dim of q should be 3 or 4")
    if k.dim() != q.dim() or v.dim() != q.dim():
        raise ValueError("q, k, v must have the same rank")
    if tuple(k.shape) != tuple(v.shape):
        raise ValueError("k and v must have the same shape")
    if q.shape[:-2] != k.shape[:-2] or q.shape[-1] != k.shape[-1]:
        raise ValueError("q and k must agree on batch, heads and head_dim")
    return _ops.infer_prefill(q, k, v, causal=causal, scale=scale, seq_lens=seq_lens)


class FlashAttentionTik(torch.nn.Module):
    """Module form, as the reference's ONNX test model wraps the op
    (tests/infer/flash_attention/tik/model.py:18-53)."""

    def __init__(self, scale=1.0, causal=False):
        super().__init__()
        self.scale, self.causal = scale, causal

    def forward(self, q, k, v, seq_lens=None):
        return flash_attention_tik(q, k, v, scale=self.scale, causal=self.causal, seq_lens=seq_lens)


def flash_attention_decode(q, k_cache, v_cache, seq_lens=None, *, scale=None, num_splits=0, workspace=None,
                           out=None):
    """y[b,n,0,:] = softmax(scale * q[b,n,0,:] K[b,n,:len_b]^T) V[b,n,:len_b]; scale defaults to D^-1/2."""
    return _ops.infer_decode(q, k_cache, v_cache, seq_lens, scale=scale, num_splits=num_splits,
                             workspace=workspace, out=out)
