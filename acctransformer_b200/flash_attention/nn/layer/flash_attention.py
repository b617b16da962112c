"""``FlashAttention`` layer with the reference's constructor and call signature.

Mirrors train/acctransformer/flash_attention/nn/layer/flash_attention.py:31-207 on torch CUDA
tensors: ``FlashAttention(head_dim, dropout_rate, prev_block_num, next_block_num,
tiling_stgy_name, dp, mp, have_attention_mask_batch, alibi)`` and
``layer(query, key, value, attn_mask=None, alibi_mask=None) -> output``.

Differences that do not change results beyond rounding:

* The reference multiplies q and k by fp16(head_dim^-1/4) in two separate elementwise kernels
  (:117,188-189); here the product head_dim^-1/2 is folded into the kernel's exponent constant.
* The reference materialises an fp16 ``[B,N,S,S]`` tensor of {0, 1/keep_prob} with
  DropoutGenMask / DropoutDoMask (:198-203); here a uint8 keep mask of the same shape is drawn
  with torch's CUDA generator and ``keep_prob`` is passed as a scalar.
* ``alibi=True`` is accepted (the reference raises, :107-108): ``alibi_mask`` ``[B,N,1,S_k]`` is
  added to every score row as the op contract declares (ops/flash_attention/attention.py:347-355).
* Dropout follows ``torch.nn.Module`` practice and is applied in training mode only (``layer.train()``);
  the reference cell applies its DropoutGenMask whenever ``dropout_rate > 0`` (:198-203) and leaves it to
  the caller to build the cell with rate 0 for evaluation.
* ``dp`` / ``mp`` / ``shard()`` are recorded and otherwise ignored: every (batch, head) slice is
  independent, so a data/model-parallel caller just passes its local slice.
"""
from __future__ import annotations

import math

import torch

from .... import ops as _ops
from ...ops.flash_attention.flash_attention_impl import _is_tile_mask, get_flash_attention

__all__ = ['FlashAttention']
HEAD_DIM_MAX_LIMIT = 256


def _draw_dropout_key(generator=None):
    """(seed, offset) of one forward call's in-kernel dropout, drawn from ``generator`` (default: torch's CPU
    generator).  Both values come from the generator's state and from nothing else, so whatever replays that state
    replays the mask: ``torch.utils.checkpoint`` restores the RNG state before it recomputes a forward, and the
    recomputed call then drops the same positions as the original one.  (A counter kept on the layer would not be
    restored and the recomputed forward would disagree with the loss that was computed.)  With a CPU generator the
    draw involves no device synchronisation."""
    dev = generator.device if generator is not None else "cpu"
    pair = torch.randint(0, 2 ** 31, (3,), generator=generator, device=dev).tolist()
    return (pair[0] << 31) | pair[1], pair[2]


class FlashAttention(torch.nn.Module):
    def __init__(self,
                 head_dim,
                 dropout_rate=0.0,
                 prev_block_num=65536,
                 next_block_num=65536,
                 tiling_stgy_name="sparse",
                 dp=1,
                 mp=1,
                 have_attention_mask_batch=True,
                 alibi=False
                 ):
        super().__init__()
        if head_dim > HEAD_DIM_MAX_LIMIT:
            raise ValueError("head_dim too large, reduce head_dim and try again.")
        self.head_dim = head_dim
        self.scale_factor = 1.0 / math.sqrt(math.sqrt(head_dim))      # what the reference applies to q and k
        self.flash_attention = get_flash_attention(
            prev_block_num=prev_block_num,
            next_block_num=next_block_num,
            tiling_stgy_name=tiling_stgy_name,
            scale=1.0 / math.sqrt(head_dim),
        )
        self.dropout_rate = dropout_rate
        self.enable_dropout = self.dropout_rate > 0.0
        self.keep_prob = 1.0 - dropout_rate
        self.have_attention_mask_batch = have_attention_mask_batch
        self.alibi = alibi
        self.dp, self.mp = dp, mp
        self.in_strategy = None
        self.generator = None      # optional torch.Generator for reproducible dropout
        # The reference draws a [B,N,S,S] mask tensor per step (DropoutGenMask, reference :124-130,198-203) and keeps
        # it for the backward.  Here the kernels decide dropout from (seed, offset) on the fly; set
        # dropout_in_kernel = False to get the mask as a tensor instead (same statistics, 1 byte per score).
        self.dropout_in_kernel = True
        # The reference refuses key / value tensors with fewer heads than the query ("change themselves to be same by
        # tile", reference :193-196).  Set allow_grouped_kv = True to pass such tensors as they are (grouped-query /
        # multi-query attention: query head n reads key/value head n // (N // N_kv); no tiled copy is made).
        self.allow_grouped_kv = False
        # A full attn_mask is inspected once per tensor (not per step): if it is exactly the causal mask, the kernels
        # generate the triangle themselves, read no mask and skip the tiles above the diagonal.
        self.detect_causal_mask = True

    def shard(self, in_strategy=None, out_strategy=None):
        """Records the split strategy (reference :132-177).  Nothing else to do: the op needs no
        exchange between (batch, head) slices."""
        if in_strategy is None:
            in_strategy = ((1, 1, 1, 1), (1, 1, 1, 1), (1, 1, 1, 1))
        self.in_strategy = in_strategy
        self.dp, self.mp = in_strategy[0][0], in_strategy[0][1]
        self.flash_attention.shard(in_strategy)

    def construct(self, q, k, v, attn_mask=None, alibi_mask=None):
        """FlashAttention forward
        :param q:           [bsz, head_num, seq_len, head_dim]
        :param k:           [bsz, head_num, seq_len, head_dim]
        :param v:           [bsz, head_num, seq_len, head_dim]
        :param attn_mask:   [1 or bsz, seq_len, seq_len], or the [1, 128, 128] causal tile when the layer
                            was built with have_attention_mask_batch=False
        :param alibi_mask:  [bsz, head_num, 1, seq_len], if not None
        :return: o          [bsz, head_num, seq_len, head_dim]
        """
        bsz, head_num, seq_len, _ = q.shape
        k_head_num, v_head_num = k.shape[1], v.shape[1]
        grouped = (self.allow_grouped_kv and k_head_num == v_head_num and k_head_num > 0
                   and head_num % k_head_num == 0)
        if (head_num != k_head_num or head_num != v_head_num) and not grouped:
            raise ValueError(
                "the head_num of query, key and value must be the same, "
                "If different head_num are used, users need to change themselves to be same by tile.")
        if alibi_mask is not None and not self.alibi:
            raise ValueError("alibi_mask given but the layer was built with alibi=False")
        drop_mask, seed, offset = None, None, 0
        if self.enable_dropout and self.training:
            if self.dropout_in_kernel:
                seed, offset = _draw_dropout_key(self.generator)
            else:
                drop_mask = (torch.rand((bsz, head_num, seq_len, k.shape[2]), device=q.device,
                                        generator=self.generator) < self.keep_prob).to(torch.uint8)
        implicit = False
        # (the check reads the mask on the GPU and synchronises once per mask tensor: it is skipped while a CUDA graph
        # is being captured, where the mask then simply stays a tensor)
        if (self.detect_causal_mask and attn_mask is not None and attn_mask.is_cuda
                and not torch.cuda.is_current_stream_capturing()):
            if not _is_tile_mask(attn_mask):
                implicit = _ops.mask_is_causal(attn_mask)
            elif self.flash_attention.next_block_num == 0 or max(seq_len, k.shape[2]) <= 128:
                # the 128x128 tile form acts on the diagonal tiles only; with no tile above the diagonal in the band
                # (next_block_num = 0), a tile that is exactly the strict upper triangle IS the causal mask
                implicit = _ops.mask_is_causal(attn_mask.reshape(1, 128, 128))
        o, _ = self.flash_attention(q, k, v, attn_mask, drop_mask, alibi_mask, keep_prob=self.keep_prob,
                                    dropout_seed=seed, dropout_offset=offset, implicit_causal=implicit)
        return o

    forward = construct
