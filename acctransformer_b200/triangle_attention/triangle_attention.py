"""``TriangleAttention`` layer with the reference's constructor and call signature.

Mirrors train/acctransformer/triangle_attention/triangle_attention.py:28-165:
``TriangleAttention(block_size=512, dropout_rate=0., dp=1, mp=1)`` and
``layer(query, key, value, attention_mask) -> output`` where, for each group of ``block_size``
query rows ending at row ``q_end``, the output is ``softmax(Q K[0:q_end]^T + (-10000) * mask) V[0:q_end]``
(:105-165).  No 1/sqrt(d) is applied inside (the caller pre-scales).

The reference slices q/k/v/mask per row group and runs BatchMatMul / Softmax / Concat on the
lower-left trapezoid.  Here one kernel launch covers the whole sequence: the kernel is told the row
group size (``tri_block``), skips every 128x128 tile that lies wholly past a row group's ``q_end``,
excludes single keys past ``q_end`` inside straddling tiles, and still reads and applies the mask
tensor inside the tiles it computes, so arbitrary masks keep the reference's meaning.  If ``attention_mask`` is
exactly the strict upper triangle (checked once per tensor on the GPU, ``detect_causal_mask``; or declared with
``assume_causal=True``) it is not read at all and the triangle is generated in-kernel.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from ..flash_attention.nn.layer.flash_attention import _draw_dropout_key
from ..flash_attention.ops.flash_attention.flash_attention_impl import _FlashAttentionFunction

__all__ = ["TriangleAttention"]


class TriangleAttention(torch.nn.Module):
    def __init__(self, block_size=512, dropout_rate=0., dp=1, mp=1, assume_causal=False):
        super().__init__()
        if block_size <= 0:
            raise ValueError(f"block size must be positive integer, but got {block_size}")
        if dropout_rate < 0. or dropout_rate >= 1.:
            raise ValueError(f"dropout rate must be between 0 and 1, but got {dropout_rate}")
        if dp <= 0:
            raise ValueError(f"data parallel must be positive integer, but got {dp}")
        if mp <= 0:
            raise ValueError(f"model parallel must be positive integer, but got {mp}")
        self.block_size = block_size
        self.dropout_rate = dropout_rate
        self.enable_dropout = dropout_rate > 0.
        self.keep_prob = 1.0 - dropout_rate
        self.dp, self.mp = dp, mp
        self.assume_causal = assume_causal
        # attention_mask is inspected once per tensor (not per step): if it is exactly the causal mask the kernels
        # generate the triangle themselves, read no mask and skip the tiles above the diagonal
        self.detect_causal_mask = True
        self.generator = None
        self.dropout_in_kernel = True   # dropout decided inside the kernels from (seed, step); False: a mask tensor

    def tiles_skipped_fraction(self, seq_length):
        """Fraction of the 128x128 score tiles the kernel never touches for this sequence length."""
        nt = (seq_length + 127) // 128
        done = 0
        for i in range(nt):
            last_row = min(i * 128 + 127, seq_length - 1)
            q_end = min(seq_length, (last_row // self.block_size + 1) * self.block_size)
            if self.assume_causal:
                q_end = min(q_end, last_row + 1)
            done += (q_end + 127) // 128
        return 1.0 - done / float(nt * nt)

    def construct(self, query, key, value, attention_mask):
        bsz, head_num, seq_length, _ = query.shape
        drop_mask, seed, offset = None, None, 0
        if self.enable_dropout and self.training:
            if self.dropout_in_kernel:
                seed, offset = _draw_dropout_key(self.generator)
            else:
                drop_mask = (torch.rand((bsz, head_num, seq_length, key.shape[2]), device=query.device,
                                        generator=self.generator) < self.keep_prob).to(torch.uint8)
        # tri_block: a query row in group g sees keys [0, (g+1)*block_size) only, as in the reference's slices;
        # inside that range the mask tensor decides (or the in-kernel triangle when assume_causal).
        # (under the in-kernel triangle the group bound excludes nothing more, so it is not passed)
        causal = self.assume_causal or (self.detect_causal_mask and attention_mask is not None
                                        and attention_mask.is_cuda and not torch.cuda.is_current_stream_capturing()
                                        and _ops.mask_is_causal(attention_mask))
        cfg = dict(prev_block_num=65536, next_block_num=65536, scale=1.0, causal=causal,
                   keep_prob=self.keep_prob, tri_block=0 if causal else self.block_size,
                   dropout_seed=seed, dropout_offset=offset)
        mask = None if causal else attention_mask
        out, _ = _FlashAttentionFunction.apply(query, key, value, mask, drop_mask, None, cfg)
        return out

    forward = construct
