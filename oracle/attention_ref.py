"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain NumPy, the *standard-attention* functions that the
reference's own tests use as ground truth.  It is the checker that the CUDA path
is compared against; it is never the thing that is shipped or measured.  Only the
test-suite, the smoke check and the ``cpu_baseline`` / ``--impl reference`` legs
of the benchmark may import it.

What each function follows (paths are relative to the reference project):

* ``sa_fwd``        tests/train/flash_attention/st/common.py:110-132
                    (``np_impl_sa_fwd``: S=QK^T, ``S += -10000*mask`` broadcast over
                    heads, softmax, ``P *= drop_mask``, ``O = P V``) and
                    tests/train/flash_attention/st/test_fa_grad_precision.py:35-36
                    (``L = row_max + log(row_sum)``).
* ``sa_grad``       tests/train/flash_attention/st/common.py:147-175
                    (``np_impl_sa_grad``, the "fa grad of softmax" branch) with the
                    un-dropped P inside dS, as the reference kernel does at
                    train/acctransformer/flash_attention/ops/flash_attention/flash_attention_bwd.py:161-181,359-406.
* ``band_mask``     train/acctransformer/flash_attention/ops/flash_attention/flash_attention_fwd.py:444-445
                    (tile (i,j) is computed iff ``j - next <= i <= j + prev``).
* alibi             train/acctransformer/flash_attention/ops/flash_attention/attention.py:347-355
                    (bias ``[B,N,1,S_k]`` added to every row of S).
* cell scaling      train/acctransformer/flash_attention/nn/layer/flash_attention.py:117,188-189
                    (q and k each multiplied by fp16(d^-1/4)).
* ``triangle_fwd``  train/acctransformer/triangle_attention/triangle_attention.py:105-165.
* ``infer_fwd``     tests/infer/flash_attention/tik/data_gen.py:32-34.
* ``data_compare``  tests/train/flash_attention/st/common.py:178-192.

Two arithmetic modes exist:

* ``faithful=False`` (default): every intermediate is kept in ``dtype`` (float32 or
  float64).  This is the mode parity tolerances are stated against.
* ``faithful=True``: reproduces the reference functions' own rounding sequence
  (fp16 matmuls, fp16 P, fp16 D).  It exists so that the restatement can be pinned
  bit-for-bit against outputs of the reference functions themselves (the golden
  files under tests/golden/ were produced by running those functions).

Parity status: pinned for forward, backward and the inference golden by those
fixtures.  Alibi, ``prev_block_num``, dropout-in-backward, ``seq_lens`` and decode
have no test or vector in the reference, so for those the oracle is "parity
unpinned" (it follows the contract the reference declares, see above).
"""
from __future__ import annotations

import numpy as np

MASK_FILL_VALUE = -10000.0   # .../ops/flash_attention/constants.py:31
BAND_BLOCK = 128             # .../ops/flash_attention/constants.py:19


def band_mask(s_q, s_k, prev_block_num, next_block_num, block=BAND_BLOCK):
    """Boolean [s_q, s_k] array, True where the 128-tile holding (row, col) is computed."""
    qi = (np.arange(s_q) // block)[:, None]
    kj = (np.arange(s_k) // block)[None, :]
    return (kj - next_block_num <= qi) & (qi <= kj + prev_block_num)


def _scores(q, k, attn_mask, alibi, scale, prev_block_num, next_block_num, causal,
            seq_lens, dtype):
    """Return (S, excluded) where excluded marks entries that do not exist at all
    (outside the block band / causal triangle / valid length) as opposed to entries
    an explicit mask pushes down by -10000."""
    b, n, s_q, d = q.shape
    s_k = k.shape[2]
    s = np.matmul(q.astype(dtype), np.swapaxes(k.astype(dtype), -1, -2))
    if scale != 1.0:
        s = s * dtype(scale)
    if alibi is not None:
        s = s + alibi.astype(dtype).reshape(b, n, 1, s_k)
    if attn_mask is not None:
        m = attn_mask.astype(dtype)
        if m.ndim == 2:
            m = m[None]
        s = s + (dtype(MASK_FILL_VALUE) * m)[:, None, :, :]
    excluded = np.zeros((1, 1, s_q, s_k), dtype=bool)
    if prev_block_num is not None or next_block_num is not None:
        p = 65536 if prev_block_num is None else prev_block_num
        nx = 65536 if next_block_num is None else next_block_num
        excluded = excluded | ~band_mask(s_q, s_k, p, nx)[None, None]
    if causal:
        excluded = excluded | (np.arange(s_k)[None, :] > np.arange(s_q)[:, None])[None, None]
    if seq_lens is not None:
        lens = np.asarray(seq_lens).reshape(b, 1, 1, 1)
        excluded = excluded | (np.arange(s_k).reshape(1, 1, 1, s_k) >= lens)
    return s, excluded


def expand_tile_mask(tile, s_q, s_k, block=BAND_BLOCK):
    """The 128x128 mask form (have_attention_mask_batch=False) applies its tile only
    on diagonal tiles: flash_attention_fwd.py:352-361.  Expanded here to [1,s_q,s_k]."""
    tile = np.asarray(tile).reshape(block, block)
    out = np.zeros((1, s_q, s_k), dtype=tile.dtype)
    for i in range(0, min(s_q, s_k), block):
        h = min(block, s_q - i)
        w = min(block, s_k - i)
        out[0, i:i + h, i:i + w] = tile[:h, :w]
    return out


def sa_fwd(q, k, v, attn_mask=None, drop_mask=None, keep_prob=1.0, alibi=None, scale=1.0,
           prev_block_num=None, next_block_num=None, causal=False, seq_lens=None,
           dtype=np.float32, return_p=False):
    """Standard attention forward.  Returns (O, L[, P]) in ``dtype``.

    drop_mask is either a {0,1} uint8/bool array [B,N,S_q,S_k] (P is multiplied by
    mask/keep_prob) or a float array that already holds {0, 1/keep_prob}."""
    dtype = np.dtype(dtype).type
    s, excluded = _scores(q, k, attn_mask, alibi, scale, prev_block_num, next_block_num,
                          causal, seq_lens, dtype)
    s = np.where(excluded, dtype(-np.inf), s)
    row_max = np.max(s, axis=-1, keepdims=True)
    e = np.exp(s - row_max)
    row_sum = np.sum(e, axis=-1, keepdims=True)
    p = e / row_sum
    lse = (row_max + np.log(row_sum))[..., 0]
    pd = p
    if drop_mask is not None:
        pd = p * _drop_factor(drop_mask, keep_prob, dtype)
    o = np.matmul(pd, v.astype(dtype))
    if return_p:
        return o, lse, p
    return o, lse


def _drop_factor(drop_mask, keep_prob, dtype):
    dm = np.asarray(drop_mask)
    if dm.dtype == np.uint8 or dm.dtype == np.bool_:
        return dm.astype(dtype) * dtype(1.0 / keep_prob)
    return dm.astype(dtype)


def sa_grad(q, k, v, do, attn_mask=None, drop_mask=None, keep_prob=1.0, alibi=None, scale=1.0,
            prev_block_num=None, next_block_num=None, causal=False, seq_lens=None,
            dtype=np.float32):
    """Standard attention backward.  Returns (dQ, dK, dV) in ``dtype``.

    dV = (P*M)^T dO ; dP = (dO V^T)*M ; D = rowsum(dO*O) ; dS = P*(dP - D) ;
    dQ = scale * dS K ; dK = scale * dS^T Q."""
    dtype = np.dtype(dtype).type
    o, _, p = sa_fwd(q, k, v, attn_mask, drop_mask, keep_prob, alibi, scale, prev_block_num,
                     next_block_num, causal, seq_lens, dtype, return_p=True)
    do = do.astype(dtype)
    fac = None if drop_mask is None else _drop_factor(drop_mask, keep_prob, dtype)
    pd = p if fac is None else p * fac
    dv = np.matmul(np.swapaxes(pd, -1, -2), do)
    dp = np.matmul(do, np.swapaxes(v.astype(dtype), -1, -2))
    if fac is not None:
        dp = dp * fac
    dsum = np.sum(do * o, axis=-1, keepdims=True)
    ds = p * (dp - dsum)
    if scale != 1.0:
        ds = ds * dtype(scale)
    dq = np.matmul(ds, k.astype(dtype))
    dk = np.matmul(np.swapaxes(ds, -1, -2), q.astype(dtype))
    return dq, dk, dv


# --------------------------------------------------------------------------------------
# Rounding-faithful restatements, used only to pin this file against the reference's own
# functions (see tests/golden/make_golden.py).
# --------------------------------------------------------------------------------------

def sa_fwd_faithful(q, k, v, attn_mask=None, drop_mask=None):
    """Same rounding sequence as np_impl_sa_fwd (st/common.py:110-132): fp16 matmul,
    fp16 mask add and max, fp32 exp/sum/divide, fp16 P, fp16 PV.
    Returns (O fp16, (E fp32, P fp16, row_sum fp32, row_max fp16))."""
    sim = np.matmul(q, np.transpose(k, (0, 1, 3, 2)))
    if attn_mask is not None:
        sim = sim + np.expand_dims(-10000.0 * attn_mask, 1)
    row_max = np.max(sim, axis=-1, keepdims=True)
    sim = (sim - row_max).astype(np.float32)
    e = np.exp(sim)
    row_sum = np.sum(e, axis=-1, keepdims=True)
    p = (e / row_sum).astype(np.float16)
    if drop_mask is not None:
        p = p * drop_mask
    o = np.matmul(p, v)
    return o, (e, p, row_sum, row_max)


def sa_grad_faithful(q, k, v, p, o, do, drop_mask=None):
    """Same rounding sequence as np_impl_sa_grad (st/common.py:147-175)."""
    dv = np.matmul(np.transpose(p, (0, 1, 3, 2)), do)
    dp = np.matmul(do, np.transpose(v, (0, 1, 3, 2)))
    if drop_mask is not None:
        dp = dp * drop_mask
    dsum = np.sum((do * o).astype(np.float32), axis=-1, keepdims=True).astype(np.float16)
    ds = p * (dp - dsum)
    dq = np.matmul(ds, k)
    dk = np.matmul(np.transpose(ds, (0, 1, 3, 2)), q)
    return dq, dk, dv


def cell_scale(x, head_dim):
    """The cell's prologue: x * fp16(head_dim^-1/4) in fp16
    (nn/layer/flash_attention.py:117,188-189)."""
    f = np.float16(1.0 / np.sqrt(np.sqrt(head_dim)))
    return (x.astype(np.float16) * f).astype(np.float16)


def triangle_fwd(q, k, v, attention_mask, block_size=512, dtype=np.float32):
    """TriangleAttention.construct (triangle_attention.py:137-165): for each group of
    ``block_size`` query rows, softmax over keys [0, q_end) of S + (-10000)*mask, then PV;
    row groups are concatenated.  No scaling inside."""
    dtype = np.dtype(dtype).type
    s_len = q.shape[2]
    groups, tail = divmod(s_len, block_size)
    bounds = [(i * block_size, (i + 1) * block_size) for i in range(groups)]
    if tail > 0:
        bounds.append((groups * block_size, s_len))
    outs = []
    for q_begin, q_end in bounds:
        cq = q[:, :, q_begin:q_end].astype(dtype)
        ck = k[:, :, 0:q_end].astype(dtype)
        cv = v[:, :, 0:q_end].astype(dtype)
        cm = attention_mask[:, q_begin:q_end, 0:q_end].astype(dtype)
        sim = np.matmul(cq, np.swapaxes(ck, -1, -2)) + (cm * dtype(MASK_FILL_VALUE))[:, None]
        sim = sim - sim.max(axis=-1, keepdims=True)
        e = np.exp(sim)
        outs.append(np.matmul(e / e.sum(axis=-1, keepdims=True), cv))
    return np.concatenate(outs, axis=2)


def infer_fwd(q, k, v, scale=1.0, causal=False, seq_lens=None, dtype=np.float32):
    """Inference op golden (data_gen.py:32-34): softmax(Q K^T) V in fp32, no scale and no
    mask in the reference; ``scale``/``causal``/``seq_lens`` are this library's extensions.
    Accepts rank-3 [B*N,S,D] or rank-4 [B,N,S,D] like the op (flash_attention_fwd.py:58-69)."""
    rank3 = q.ndim == 3
    if rank3:
        q, k, v = q[None], k[None], v[None]
    o, _ = sa_fwd(q, k, v, scale=scale, causal=causal, seq_lens=seq_lens, dtype=dtype)
    return o[0] if rank3 else o


def decode_ref(q, k_cache, v_cache, seq_lens, scale, dtype=np.float32):
    """One-token attention over a KV cache: y[b,h,0,:] = softmax(scale * q K[:len_b]^T) V[:len_b].
    No reference code exists for this (the inference op has no decode path); it is the
    q_len=1 case of ``infer_fwd`` with per-sequence valid lengths."""
    return infer_fwd(q, k_cache, v_cache, scale=scale, seq_lens=seq_lens, dtype=dtype)


def alibi_slopes(n_heads):
    """Per-head slopes 2^(-8(h+1)/N)."""
    return np.array([2.0 ** (-8.0 * (h + 1) / n_heads) for h in range(n_heads)], dtype=np.float64)


def alibi_bias(batch, n_heads, s_k, dtype=np.float16):
    """[B,N,1,S_k] row-broadcast bias slope_h * key_position, in the declared layout
    (nn/layer/flash_attention.py:185)."""
    sl = alibi_slopes(n_heads).reshape(1, n_heads, 1, 1)
    pos = np.arange(s_k, dtype=np.float64).reshape(1, 1, 1, s_k)
    return np.broadcast_to(sl * pos, (batch, n_heads, 1, s_k)).astype(dtype)


def data_compare(ground_truth, predict, rtol=0.001, rtol_pct_thd=0.001, atol=0.001, max_rtol=0.1):
    """The reference tests' two-threshold criterion (st/common.py:178-192): "Pass" iff at most
    rtol_pct_thd of the elements are off by more than rtol*|gt|+atol and none by more than
    max_rtol*|gt|+atol.  Returns (result, proportion_1, proportion_2)."""
    gt = np.asarray(ground_truth, dtype=np.float64)
    pr = np.asarray(predict, dtype=np.float64)
    diff = np.abs(pr - gt)
    total = gt.size
    p1 = np.sum(diff > rtol * np.abs(gt) + atol) / total
    p2 = np.sum(diff > max_rtol * np.abs(gt) + atol) / total
    ok = not (p1 > rtol_pct_thd or p2 > 0)
    return ("Pass" if ok else "Failed"), float(p1), float(p2)


# ----------------------------------------------------------------------------------------------
# In-kernel dropout: the mask as a function of the position
# ----------------------------------------------------------------------------------------------
# No counterpart in the reference, whose cell draws the mask with MindSpore's DropoutGenMask
# (nn/layer/flash_attention.py:124-130,198-203) and keeps the tensor for the backward.  The
# generator is Philox4x32-10 (Salmon, Moraes, Dror, Shaw, "Parallel random numbers: as easy as
# 1, 2, 3", SC'11), restated here from the paper; it is pinned by the known-answer vectors the
# authors publish with their Random123 library (tests/test_dropout_philox.py).
_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(ctr, key):
    """ctr: four uint32 arrays (broadcastable), key: two uint32 scalars.  Returns four uint32 arrays."""
    c = [np.asarray(x, dtype=np.uint64) for x in ctr]
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    lo32 = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(_PHILOX_M0) * c[0]
        p1 = np.uint64(_PHILOX_M1) * c[2]
        c = [(p1 >> np.uint64(32)) ^ c[1] ^ k0, p1 & lo32, (p0 >> np.uint64(32)) ^ c[3] ^ k1, p0 & lo32]
        k0 = (k0 + np.uint64(_PHILOX_W0)) & lo32
        k1 = (k1 + np.uint64(_PHILOX_W1)) & lo32
    return [x.astype(np.uint32) for x in c]


def dropout_threshold(keep_prob):
    """round(keep_prob * 256) clamped to [1, 256] (float32 arithmetic, ties away from zero like lroundf)."""
    t = int(np.floor(np.float32(keep_prob) * np.float32(256.0) + np.float32(0.5)))
    return min(256, max(1, t))


def dropout_mask_philox(B, N, S_q, S_k, keep_prob, seed, offset=0, units=None):
    """uint8 {0,1} mask [B,N,S_q,S_k]: position (b,n,q,k) is kept iff byte (k & 15) of
    Philox(counter = (q, k >> 4, b*N + n, offset), key = (seed low, seed high)) is below the threshold.
    ``units``: a list of unit numbers b*N + n; the result is then [len(units), 1, S_q, S_k] for those units only."""
    groups = (S_k + 15) // 16
    q = np.arange(S_q, dtype=np.uint32).reshape(1, S_q, 1)
    g = np.arange(groups, dtype=np.uint32).reshape(1, 1, groups)
    if units is not None:
        u = np.asarray(units, dtype=np.uint32).reshape(-1, 1, 1)
        B, N = u.shape[0], 1
    else:
        u = np.arange(B * N, dtype=np.uint32).reshape(B * N, 1, 1)
    shape = (B * N, S_q, groups)
    words = philox4x32_10([np.broadcast_to(q, shape), np.broadcast_to(g, shape), np.broadcast_to(u, shape),
                           np.full(shape, offset & 0xFFFFFFFF, dtype=np.uint32)],
                          (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    by = np.stack([(w >> np.uint32(8 * i)) & np.uint32(0xFF) for w in words for i in range(4)], axis=-1)  # [..., 16]
    keep = (by < dropout_threshold(keep_prob)).astype(np.uint8).reshape(B * N, S_q, groups * 16)[:, :, :S_k]
    return np.ascontiguousarray(keep.reshape(B, N, S_q, S_k))


# ----------------------------------------------------------------------------------------------
# Grouped-query attention (fewer key/value heads than query heads)
# ----------------------------------------------------------------------------------------------
# The reference has no such path: its cell asks the user to tile K and V up to the query's head
# count (nn/layer/flash_attention.py:193-196).  These helpers ARE that tiling, around the
# functions above, so the grouped path is checked against the reference's own prescription.
def expand_kv_heads(x, n_q_heads):
    """[B,N_kv,S,D] -> [B,N,S,D]: query head n uses key/value head n // (N // N_kv)."""
    group = n_q_heads // x.shape[1]
    return np.repeat(x, group, axis=1)


def reduce_kv_heads(g, n_kv_heads):
    """Gradient of expand_kv_heads: sums the heads of each group.  [B,N,S,D] -> [B,N_kv,S,D]."""
    B, N, S, D = g.shape
    return g.reshape(B, n_kv_heads, N // n_kv_heads, S, D).sum(axis=2)


def gqa_fwd(q, k, v, **kw):
    return sa_fwd(q, expand_kv_heads(k, q.shape[1]), expand_kv_heads(v, q.shape[1]), **kw)


def gqa_grad(q, k, v, do, **kw):
    dq, dk, dv = sa_grad(q, expand_kv_heads(k, q.shape[1]), expand_kv_heads(v, q.shape[1]), do, **kw)
    return dq, reduce_kv_heads(dk, k.shape[1]), reduce_kv_heads(dv, v.shape[1])
