"""The FlashAttention forward / grad primitives, backed by ``libacct_b200.so``.

Mirrors the reference's op registration module
(train/acctransformer/flash_attention/ops/flash_attention/flash_attention_impl.py:96-154):

* ``get_flash_attention(prev_block_num, next_block_num, tiling_stgy_name)`` returns the forward
  primitive ``fa(query, key, value, attn_mask=None, dropout_mask=None, alibi_mask=None)
  -> (output, rowsum)``; ``output`` has q's dtype and shape, ``rowsum`` is the fp32
  log-sum-exp ``[B, N, S_q]`` (:132-140).  No scaling happens inside the primitive.
* ``get_flash_attention_grad(...)`` returns the grad primitive
  ``fa_grad(query, key, value, output, do, rowsum, attn_mask, dropout_mask, alibi_mask)
  -> (dq, dk, dv)`` in fp32 (:99-105).
* The forward primitive is differentiable: its backward calls the grad primitive and casts
  dq/dk/dv to the input dtype, like the reference's ``bprop`` (:117-124).

The tensors are torch CUDA tensors in ``[B, N, S, D]`` layout.  An ``attn_mask`` whose shape is
``(128, 128)`` or ``(1, 128, 128)`` is the causal-tile form and is applied to diagonal 128x128
tiles only (ops/flash_attention/attention.py:279-285); any other mask is ``[1 or B, S_q, S_k]``.
``dropout_mask`` is either the reference's 16-bit ``{0, 1/keep_prob}`` tensor or a uint8 ``{0,1}``
tensor together with ``keep_prob``.  ``tiling_stgy_name`` is accepted for compatibility; tile
sizes are fixed inside the CUDA kernels.
"""
from __future__ import annotations

import torch

from .... import ops as _ops

__all__ = ["get_flash_attention", "get_flash_attention_grad"]


def _mask_tiles(attn_mask, enabled=True):
    """Per-tile summary of a full attn_mask (made once per mask tensor, see ops.mask_tile_classes), with which the
    kernels read only the 128x128 tiles of the mask that are neither all 0 nor all 1; None for no mask / the tile form."""
    if not enabled or attn_mask is None or _is_tile_mask(attn_mask) or not attn_mask.is_cuda:
        return None
    return _ops.mask_tile_classes(attn_mask)


def _is_tile_mask(attn_mask):
    if attn_mask is None:
        return False
    shp = tuple(attn_mask.shape)
    return shp == (128, 128) or shp == (1, 128, 128)


def get_flash_attention_grad(prev_block_num=65536, next_block_num=65536, tiling_stgy_name='sparse',
                             scale=1.0, causal=False, deterministic=False):
    """Returns the grad primitive (fp32 dq, dk, dv).  ``deterministic`` makes dq bit-reproducible from run to
    run (the reference's tests require that of its gradients, tests/train/flash_attention/st/test_sharding.py:91-115)
    at some cost in speed; dk and dv always are."""

    def fa_grad(query, key, value, output, do, rowsum, attn_mask=None, dropout_mask=None, alibi_mask=None,
                keep_prob=1.0, grads_fp32=True, dropout_seed=None, dropout_offset=0):
        return _ops.fa_backward(query, key, value, output, rowsum, do, attn_mask,
                                mask_tile128=_is_tile_mask(attn_mask), causal=causal,
                                dropout_mask=dropout_mask, keep_prob=keep_prob, alibi=alibi_mask,
                                prev_block_num=prev_block_num, next_block_num=next_block_num, scale=scale,
                                grads_fp32=grads_fp32, deterministic=deterministic,
                                dropout_seed=dropout_seed, dropout_offset=dropout_offset,
                                mask_tiles=_mask_tiles(attn_mask))

    fa_grad.prev_block_num = prev_block_num
    fa_grad.next_block_num = next_block_num
    fa_grad.tiling_stgy_name = tiling_stgy_name
    return fa_grad


class _FlashAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, attn_mask, dropout_mask, alibi_mask, cfg):
        ctx.mask_tiles = _mask_tiles(attn_mask, cfg.get("classify_mask_tiles", True))
        output, rowsum = _ops.fa_forward(
            query, key, value, attn_mask, mask_tile128=_is_tile_mask(attn_mask), causal=cfg["causal"],
            dropout_mask=dropout_mask, keep_prob=cfg["keep_prob"], alibi=alibi_mask,
            prev_block_num=cfg["prev_block_num"], next_block_num=cfg["next_block_num"], scale=cfg["scale"],
            tri_block=cfg.get("tri_block", 0), dropout_seed=cfg.get("dropout_seed"),
            dropout_offset=cfg.get("dropout_offset", 0), mask_tiles=ctx.mask_tiles)
        ctx.save_for_backward(query, key, value, output, rowsum,
                              *(t for t in (attn_mask, dropout_mask, alibi_mask) if t is not None))
        ctx.present = (attn_mask is not None, dropout_mask is not None, alibi_mask is not None)
        ctx.cfg = cfg
        ctx.mark_non_differentiable(rowsum)
        return output, rowsum

    @staticmethod
    def backward(ctx, d_output, _d_rowsum):
        saved = list(ctx.saved_tensors)
        query, key, value, output, rowsum = saved[:5]
        rest = saved[5:]
        opt = []
        for present in ctx.present:
            opt.append(rest.pop(0) if present else None)
        attn_mask, dropout_mask, alibi_mask = opt
        cfg = ctx.cfg
        dq, dk, dv = _ops.fa_backward(
            query, key, value, output, rowsum, d_output.contiguous(), attn_mask,
            mask_tile128=_is_tile_mask(attn_mask), causal=cfg["causal"], dropout_mask=dropout_mask,
            keep_prob=cfg["keep_prob"], alibi=alibi_mask, prev_block_num=cfg["prev_block_num"],
            next_block_num=cfg["next_block_num"], scale=cfg["scale"], grads_fp32=False,
            tri_block=cfg.get("tri_block", 0), deterministic=cfg.get("deterministic", False),
            dropout_seed=cfg.get("dropout_seed"), dropout_offset=cfg.get("dropout_offset", 0),
            mask_tiles=ctx.mask_tiles)
        return dq, dk, dv, None, None, None, None


def get_flash_attention(prev_block_num=65536, next_block_num=65536, tiling_stgy_name='sparse',
                        scale=1.0, causal=False, deterministic=False):
    """Returns the forward primitive.  ``scale`` (default 1: the raw primitive) and ``causal``
    (an in-kernel triangle that needs no mask tensor) are this library's additions."""

    def fa_forward(query, key, value, attn_mask=None, dropout_mask=None, alibi_mask=None, keep_prob=1.0,
                   dropout_seed=None, dropout_offset=0, implicit_causal=False):
        # dropout_seed / dropout_offset: dropout decided inside the kernels (no mask tensor); the backward that
        # autograd runs later reuses the same two values
        # implicit_causal: the caller has established that attn_mask is exactly the causal mask; the kernels then
        # generate the triangle and the tensor is not read
        if implicit_causal:
            attn_mask = None
        cfg = dict(prev_block_num=prev_block_num, next_block_num=next_block_num, scale=scale,
                   causal=causal or implicit_causal, keep_prob=keep_prob, deterministic=deterministic,
                   dropout_seed=dropout_seed, dropout_offset=dropout_offset)
        return _FlashAttentionFunction.apply(query, key, value, attn_mask, dropout_mask, alibi_mask, cfg)

    fa_forward.prev_block_num = prev_block_num
    fa_forward.next_block_num = next_block_num
    fa_forward.tiling_stgy_name = tiling_stgy_name
    fa_forward.prim_attrs = {}

    def add_prim_attr(name, value):
        fa_forward.prim_attrs[name] = value

    fa_forward.add_prim_attr = add_prim_attr
    fa_forward.shard = lambda strategy: fa_forward.prim_attrs.__setitem__("in_strategy", strategy)
    return fa_forward
