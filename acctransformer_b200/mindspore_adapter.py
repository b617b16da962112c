"""MindSpore side of the boundary: the two FlashAttention primitives and the cell, registered as
``ops.Custom(func_type="aot")`` operators that call ``libacct_b200.so``.

This is the module a MindSpore-on-GPU user puts where the reference has
train/acctransformer/flash_attention/ops/flash_attention/flash_attention_impl.py:96-154 (the
``Custom(func_type="tbe")`` registration of the forward and grad primitives and the ``bprop`` that
ties them together) and train/acctransformer/flash_attention/nn/layer/flash_attention.py:31-207
(the cell and its ``shard()``).  The shape / dtype inference functions, the attribute handling
and the strategy tables below are plain Python and are tested without MindSpore; only
``get_flash_attention`` / ``get_flash_attention_grad`` / ``FlashAttention`` need ``mindspore``
itself and raise ``ImportError`` without it (MindSpore is not part of this library's
requirements, and no MindSpore graph has run these operators here).

How the pieces of the reference map:

* out_shape / out_dtype of the forward: ``(q_shape, [B, N, S_q])`` and ``(q_dtype, float32)``
  (flash_attention_impl.py:132-140).
* out_shape / out_dtype of the grad primitive: the three fp32 gradients (:99-105) PLUS a 1-D
  uint8 workspace as a fourth output, so that the framework's allocator provides the scratch
  memory the kernel needs (the reference's outputs are "atomic add" buffers zero-filled by its
  runtime, flash_attention_bwd.py:55-57; the library zero-fills its own accumulator).
* ``bprop`` (:117-124): calls the grad primitive, casts dq/dk/dv to the input dtype and returns
  zeros for the three optional inputs.
* primitive attributes (:146-152): MindSpore's AOT calling convention carries no attributes, so
  every distinct (prev_block_num, next_block_num, keep_prob, scale, causal) tuple is given a
  numbered slot in the library (``acct_ms_fa_attrs_slot``) and the primitive is bound to that
  slot's entry points ``acct_ms_fa_fwd_s<k>`` / ``acct_ms_fa_grad_s<k>``.  Two layers with
  different band widths or dropout rates in one graph therefore keep their own values.
"""
from __future__ import annotations

import ctypes as C
import math

from . import _lib

__all__ = ["get_flash_attention", "get_flash_attention_grad", "FlashAttention", "forward_out_shape",
           "forward_out_dtype", "grad_out_shape", "grad_out_dtype", "bwd_workspace_bytes", "attrs_slot",
           "aot_func", "shard_attrs"]

MAX_SLOTS = 32


# ---------------------------------------------------------------------------------------------
# plain-Python parts (no MindSpore needed)
# ---------------------------------------------------------------------------------------------
def forward_out_shape(q_shape, k_shape, v_shape, attn_mask_shape=None, dropout_mask_shape=None, alibi_mask_shape=None):
    """(output, rowsum) shapes: flash_attention_impl.py:132-136."""
    batch, head_num, seq_len, _ = q_shape
    return tuple(q_shape), (batch, head_num, seq_len)


def forward_out_dtype(q_dtype, k_dtype, v_dtype, attn_mask_dtype=None, dropout_mask_dtype=None, alibi_mask_dtype=None,
                      float32="float32"):
    """(output, rowsum) dtypes: flash_attention_impl.py:138-140."""
    return q_dtype, float32


def bwd_workspace_bytes(q_shape, grads_fp32=True):
    """Bytes of the backward's scratch for q of this shape, as the library itself states them."""
    a = _lib.FaArgs()
    a.B, a.N, a.S_q, a.D = (int(x) for x in q_shape)
    a.S_k = a.S_q
    a.flags = _lib.FLAG_GRAD_F32 if grads_fp32 else 0
    return int(_lib.load().acct_fa_bwd_workspace_bytes(C.byref(a)))


def grad_out_shape(q_shape, k_shape, v_shape, o_shape, do_shape, l_shape, attn_mask_shape=None,
                   dropout_mask_shape=None, alibi_mask_shape=None):
    """(dq, dk, dv, workspace) shapes: the reference's three (flash_attention_impl.py:99-101) and the scratch."""
    return tuple(q_shape), tuple(k_shape), tuple(v_shape), (bwd_workspace_bytes(q_shape),)


def grad_out_dtype(q_dtype, k_dtype, v_dtype, o_dtype, do_dtype, l_dtype, attn_mask_dtype=None, dropout_mask_dtype=None,
                   alibi_mask_dtype=None, float32="float32", uint8="uint8"):
    """fp32 gradients as in the reference (flash_attention_impl.py:103-105); the workspace is bytes."""
    return float32, float32, float32, uint8


HAS_ATTN_MASK, HAS_DROPOUT_MASK, HAS_ALIBI_MASK = 1, 2, 4     # ACCT_MS_HAS_* of include/acct_b200.h


def attrs_slot(prev_block_num=65536, next_block_num=65536, keep_prob=1.0, scale=1.0, causal=False, optional_inputs=None):
    """Number of the library's attribute slot that holds these values (an identical tuple gets the slot it already
    has).  Raises when all slots are taken by other tuples.

    ``optional_inputs``: which of attn_mask / dropout_mask / alibi_mask the primitive will pass (a sum of ``HAS_*``);
    the library then takes exactly those, by position, and checks each one's shape.  ``None``: the library tells the
    optional inputs apart by their shapes (it cannot tell an alibi_mask from a dropout_mask when S_q = 1)."""
    lib = _lib.load()
    lib.acct_ms_fa_attrs_slot_ex.argtypes = [C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int]
    lib.acct_ms_fa_attrs_slot_ex.restype = C.c_int
    declared = -1 if optional_inputs is None else int(optional_inputs)
    if not -1 <= declared <= 7:
        raise ValueError(f"optional_inputs = {optional_inputs}: a sum of HAS_ATTN_MASK, HAS_DROPOUT_MASK, HAS_ALIBI_MASK")
    slot = lib.acct_ms_fa_attrs_slot_ex(int(min(prev_block_num, 65536)), int(min(next_block_num, 65536)), float(keep_prob),
                                        float(scale), 1 if causal else 0, declared)
    if slot < 0:
        raise RuntimeError(f"all {MAX_SLOTS} attribute slots of libacct_b200.so are in use by other attribute tuples")
    return slot


def aot_func(kind, slot):
    """The ``func`` string of ops.Custom for entry point ``kind`` ("fwd" or "grad") bound to ``slot``."""
    if kind not in ("fwd", "grad"):
        raise ValueError(kind)
    return f"{_lib.LIB_PATH}:acct_ms_fa_{kind}_s{int(slot)}"


def shard_attrs(in_strategy=None, have_attention_mask_batch=True, enable_dropout=False, alibi=False):
    """The primitive attributes the reference cell's ``shard()`` sets (nn/layer/flash_attention.py:132-177), as a
    dict: device matrix [dp, mp, 1, 1] taken from the strategy of q, one tensor map per input (q, k, v on all four
    axes; the mask on the batch axis only, or on none when it has no batch; dropout and alibi masks like q), the
    maps of the two outputs, and the count of absent optional inputs."""
    if in_strategy is None:
        in_strategy = ((1, 1, 1, 1), (1, 1, 1, 1), (1, 1, 1, 1))
    dp, mp = in_strategy[0][0], in_strategy[0][1]
    full = [3, 2, 1, 0]
    maps = [list(full), list(full), list(full), [3, 1, 0] if have_attention_mask_batch else [-1, 1, 0]]
    absent = 2
    for present in (enable_dropout, alibi):
        if present:
            absent -= 1
            maps.append(list(full))
    return {"in_strategy": tuple(tuple(s) for s in in_strategy), "dev_matrix_shape": [dp, mp, 1, 1],
            "inputs_tensor_map": maps, "outputs_tensor_map": [list(full), [3, 2, 1]], "as_loss_divisor": 0,
            "empty_mirror_ops": absent}


# ---------------------------------------------------------------------------------------------
# MindSpore parts
# ---------------------------------------------------------------------------------------------
def _ms():
    try:
        import mindspore
    except ImportError as e:      # pragma: no cover - MindSpore is an optional host framework
        raise ImportError("acctransformer_b200.mindspore_adapter needs the mindspore package for this call") from e
    return mindspore


def get_flash_attention_grad(prev_block_num=65536, next_block_num=65536, tiling_stgy_name='sparse', keep_prob=1.0,
                             scale=1.0, causal=False, optional_inputs=None):
    """Returns the ``bprop`` function of the forward primitive, built around the grad primitive
    (flash_attention_impl.py:96-126)."""
    ms = _ms()
    from mindspore import ops
    from mindspore.common import dtype as mstype
    from mindspore.ops import Custom
    slot = attrs_slot(prev_block_num, next_block_num, keep_prob, scale, causal, optional_inputs)

    def out_dtype(*dtypes):
        return mstype.float32, mstype.float32, mstype.float32, mstype.uint8

    fa_grad = Custom(aot_func("grad", slot), out_shape=grad_out_shape, out_dtype=out_dtype, func_type="aot")
    fa_grad.add_prim_attr("prev_block_num", prev_block_num)
    fa_grad.add_prim_attr("next_block_num", next_block_num)
    fa_grad.add_prim_attr("tiling_stgy_name", tiling_stgy_name)
    fa_grad.init_prim_io_names(
        inputs=["query", "key", "value", "output", "do", "rowsum", "attn_mask", "dropout_mask", "alibi_mask"],
        outputs=["dq", "dk", "dv", "workspace"])
    zeros_like = ops.ZerosLike()

    def bprop(query, key, value, attn_mask, dropout_mask, alibi_mask, outs, douts):
        output, rowsum = outs
        dout, _ = douts
        dq, dk, dv, _ = fa_grad(query, key, value, output, dout, rowsum, attn_mask, dropout_mask, alibi_mask)
        dt = query.dtype
        return (ops.cast(dq, dt), ops.cast(dk, dt), ops.cast(dv, dt), zeros_like(attn_mask), zeros_like(dropout_mask),
                zeros_like(alibi_mask))

    del ms
    return bprop


def get_flash_attention(prev_block_num=65536, next_block_num=65536, tiling_stgy_name='sparse', keep_prob=1.0, scale=1.0,
                        causal=False, optional_inputs=None):
    """Returns the forward primitive ``fa(query, key, value, attn_mask, dropout_mask, alibi_mask) -> (output, rowsum)``
    with its ``bprop`` attached (flash_attention_impl.py:129-154).  ``optional_inputs`` (a sum of ``HAS_*``) declares
    which of the three optional inputs the caller will pass; see ``attrs_slot``."""
    _ms()
    from mindspore.common import dtype as mstype
    from mindspore.ops import Custom
    slot = attrs_slot(prev_block_num, next_block_num, keep_prob, scale, causal, optional_inputs)

    def out_dtype(q_dtype, *rest):
        return q_dtype, mstype.float32

    bprop = get_flash_attention_grad(prev_block_num, next_block_num, tiling_stgy_name, keep_prob, scale, causal,
                                     optional_inputs)
    fa_forward = Custom(aot_func("fwd", slot), out_shape=forward_out_shape, out_dtype=out_dtype, func_type="aot",
                        bprop=bprop)
    fa_forward.add_prim_attr("prev_block_num", prev_block_num)
    fa_forward.add_prim_attr("next_block_num", next_block_num)
    fa_forward.add_prim_attr("tiling_stgy_name", tiling_stgy_name)
    fa_forward.init_prim_io_names(inputs=["query", "key", "value", "attn_mask", "dropout_mask", "alibi_mask"],
                                  outputs=["output", "rowsum"])
    return fa_forward


def FlashAttention(head_dim, dropout_rate=0.0, prev_block_num=65536, next_block_num=65536, tiling_stgy_name="sparse",
                   dp=1, mp=1, have_attention_mask_batch=True, alibi=False):
    """Builds the MindSpore cell with the reference's constructor (nn/layer/flash_attention.py:70-130).  The two
    fp16 multiplies of q and k by head_dim^-1/4 are folded into the primitive's ``scale`` attribute; the dropout
    mask is generated with the same MindSpore operators as in the reference (:198-203) and handed to the primitive
    as its 16-bit {0, 1/keep} tensor."""
    ms = _ms()
    from mindspore import Tensor, nn, ops
    from mindspore.common import dtype as mstype
    if head_dim > 256:
        raise ValueError("head_dim too large, reduce head_dim and try again.")

    class _FlashAttention(nn.Cell):
        def __init__(self):
            super().__init__()
            self.flash_attention = get_flash_attention(prev_block_num, next_block_num, tiling_stgy_name,
                                                       scale=1.0 / math.sqrt(head_dim))
            self.flash_attention.add_prim_attr("primitive_target", "GPU")
            self.enable_dropout = dropout_rate > 0.0
            self.have_attention_mask_batch = have_attention_mask_batch
            self.alibi = alibi
            if self.enable_dropout:
                self.keep_prob = Tensor(1 - dropout_rate, dtype=mstype.float16)
                self.fill_v2 = ops.FillV2().shard(((dp, mp, 1, 1), ()))
                self.tensor_one = Tensor(1.0, mstype.float16)
                self.drop_gen_mask = ops.DropoutGenMask()
                self.do_dropout = ops.DropoutDoMask().shard(((dp, mp, 1, 1),))
                self.depend = ops.Depend()

        def shard(self, in_strategy=None, out_strategy=None):
            attrs = shard_attrs(in_strategy, self.have_attention_mask_batch, self.enable_dropout, self.alibi)
            self.flash_attention.shard(attrs.pop("in_strategy"))
            for name, value in attrs.items():
                self.flash_attention.add_prim_attr(name, value)

        def construct(self, q, k, v, attn_mask=None, alibi_mask=None):
            bsz, head_num, seq_len, _ = q.shape
            if head_num != k.shape[1] or head_num != v.shape[1]:
                raise ValueError(
                    "the head_num of query, key and value must be the same, "
                    "If different head_num are used, users need to change themselves to be same by tile.")
            drop_mask = None
            if self.enable_dropout:
                bits = self.drop_gen_mask((bsz, head_num, seq_len, seq_len), self.keep_prob)
                ones = self.fill_v2(Tensor((bsz, head_num, seq_len, seq_len), mstype.int32), self.tensor_one)
                ones = self.depend(ones, q)
                drop_mask = self.do_dropout(ones, bits, self.keep_prob)
            o, _ = self.flash_attention(q, k, v, attn_mask, drop_mask, alibi_mask)
            return o

    del ms
    return _FlashAttention()
