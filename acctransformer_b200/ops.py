"""Torch-tensor front end of the C ABI: fills the argument structs from CUDA tensors and launches
on torch's current stream.  torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
import math
import weakref

import torch

from . import _lib
from ._lib import (ACCT_BF16, ACCT_F16, ACCT_U8, BAND_UNBOUNDED, FLAG_DETERMINISTIC, FLAG_DROPOUT_PHILOX, FLAG_GRAD_F32, MASK_FULL, MASK_NONE,
                   MASK_TILE128, DecodeArgs, FaArgs, FaBwdIO, InferArgs, check, load)

_DTYPES = {torch.float16: ACCT_F16, torch.bfloat16: ACCT_BF16, torch.uint8: ACCT_U8, torch.bool: ACCT_U8}


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(name, t):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")


def _dtype_code(t, what):
    if t.dtype not in _DTYPES:
        raise ValueError(f"{what}: unsupported dtype {t.dtype}")
    return _DTYPES[t.dtype]


def _strides3(t):
    if t.stride(-1) != 1:
        raise ValueError("head_dim must be contiguous")
    return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def _fill_fa_args(q, k, v, o, lse, attn_mask, mask_tile128, causal, dropout_mask, keep_prob, alibi,
                  alibi_slopes, prev_block_num, next_block_num, scale, seq_lens, flags=0, tri_block=0,
                  dropout_seed=None, dropout_offset=0, mask_tiles=None):
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda(name, t)
        if t.dim() != 4:
            raise ValueError(f"{name} must be [B, N, S, D]")
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share dtype float16 or bfloat16")
    B, N, S_q, D = q.shape
    S_k, N_kv = k.shape[2], k.shape[1]
    if k.shape != (B, N_kv, S_k, D) or v.shape != (B, N_kv, S_k, D) or N_kv < 1 or N % N_kv != 0:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)} "
                         "(k and v may have fewer heads than q if their head count divides q's)")
    a = FaArgs()
    a.N_kv = N_kv
    a.dtype = _DTYPES[q.dtype]
    a.B, a.N, a.S_q, a.S_k, a.D = B, N, S_q, S_k, D
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.q_stride, a.k_stride, a.v_stride, a.o_stride = _strides3(q), _strides3(k), _strides3(v), _strides3(o)
    keep = []
    a.mask_kind = MASK_NONE
    if attn_mask is not None:
        _require_cuda("attn_mask", attn_mask)
        m = attn_mask.contiguous()
        keep.append(m)
        a.mask_dtype = _dtype_code(m, "attn_mask")
        if mask_tile128:
            if m.numel() != 128 * 128:
                raise ValueError("the tile form of attn_mask must hold 128x128 elements")
            a.mask_kind, a.mask_batch = MASK_TILE128, 1
        else:
            if m.dim() == 2:
                m = m.unsqueeze(0)
            if m.dim() != 3 or m.shape[1] != S_q or m.shape[2] != S_k or m.shape[0] not in (1, B):
                raise ValueError(f"attn_mask must be [1 or B, S_q, S_k], got {tuple(attn_mask.shape)}")
            a.mask_kind, a.mask_batch = MASK_FULL, m.shape[0]
        a.attn_mask = m.data_ptr()
    if mask_tiles is not None:
        if a.mask_kind != MASK_FULL:
            raise ValueError("mask_tiles goes with a full attn_mask tensor")
        _require_cuda("mask_tiles", mask_tiles)
        want = (a.mask_batch, -(-S_q // 128), -(-S_k // 128))
        if mask_tiles.dtype != torch.uint8 or tuple(mask_tiles.shape) != want or not mask_tiles.is_contiguous():
            raise ValueError(f"mask_tiles must be a contiguous uint8 tensor {want}, as mask_tile_classes() returns it")
        keep.append(mask_tiles)
        a.mask_tiles = mask_tiles.data_ptr()
    a.causal = 1 if causal else 0
    a.keep_prob = float(keep_prob)
    if dropout_mask is not None:
        _require_cuda("dropout_mask", dropout_mask)
        dm = dropout_mask.contiguous()
        keep.append(dm)
        if tuple(dm.shape) != (B, N, S_q, S_k):
            raise ValueError("dropout_mask must be [B, N, S_q, S_k]")
        a.dropout_mask = dm.data_ptr()
        a.dropout_dtype = _dtype_code(dm, "dropout_mask")
    if alibi is not None:
        _require_cuda("alibi", alibi)
        al = alibi.contiguous()
        keep.append(al)
        if tuple(al.shape) != (B, N, 1, S_k) or al.dtype != q.dtype:
            raise ValueError("alibi must be [B, N, 1, S_k] in the dtype of q")
        a.alibi = al.data_ptr()
    if alibi_slopes is not None:
        _require_cuda("alibi_slopes", alibi_slopes)
        sl = alibi_slopes.to(torch.float32).contiguous()
        keep.append(sl)
        if sl.numel() != N:
            raise ValueError("alibi_slopes must hold N values")
        a.alibi_slopes = sl.data_ptr()
    a.prev_block_num = min(int(prev_block_num), BAND_UNBOUNDED)
    a.next_block_num = min(int(next_block_num), BAND_UNBOUNDED)
    a.scale = float(scale)
    if seq_lens is not None:
        _require_cuda("seq_lens", seq_lens)
        sl = seq_lens.to(torch.int32).contiguous()
        keep.append(sl)
        a.seq_lens = sl.data_ptr()
    if dropout_seed is not None:
        if dropout_mask is not None:
            raise ValueError("give either dropout_mask (tensor form) or dropout_seed (in-kernel form), not both")
        flags |= FLAG_DROPOUT_PHILOX
        a.dropout_seed = int(dropout_seed) & 0xFFFFFFFFFFFFFFFF
        a.dropout_offset = int(dropout_offset)
    a.flags = flags
    a.tri_block = int(tri_block)
    return a, keep


def fa_forward(q, k, v, attn_mask=None, *, mask_tile128=False, causal=False, dropout_mask=None,
               keep_prob=1.0, alibi=None, alibi_slopes=None, prev_block_num=BAND_UNBOUNDED,
               next_block_num=BAND_UNBOUNDED, scale=1.0, seq_lens=None, need_lse=True, tri_block=0,
               dropout_seed=None, dropout_offset=0, mask_tiles=None, out=None, lse_out=None):
    """Forward primitive: returns (output [B,N,S_q,D] in q's dtype, lse [B,N,S_q] fp32 or None).

    ``mask_tiles`` (optional, from ``mask_tile_classes(attn_mask)``) lets the kernel skip reading the 128x128 tiles
    of a full ``attn_mask`` that are all 0 or all 1; results are the same as without it.

    Dropout comes either as a tensor (``dropout_mask`` + ``keep_prob``) or is decided inside the kernel from
    ``dropout_seed`` / ``dropout_offset`` + ``keep_prob`` (no [B,N,S_q,S_k] tensor exists then; the backward must
    be given the same three values).

    ``out`` / ``lse_out``: tensors to write into instead of new ones (a caller that steps in a loop and wants no
    allocation in it)."""
    lib = load()
    o = out if out is not None else torch.empty(q.shape, dtype=q.dtype, device=q.device)
    if o.shape != q.shape or o.dtype != q.dtype or not o.is_cuda:
        raise ValueError("out must be a CUDA tensor shaped and typed like q")
    lse = None
    if need_lse:
        lse = lse_out if lse_out is not None else torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
        if tuple(lse.shape) != tuple(q.shape[:3]) or lse.dtype != torch.float32 or not lse.is_contiguous():
            raise ValueError("lse_out must be a contiguous float32 tensor [B, N, S_q]")
    a, keep = _fill_fa_args(q, k, v, o, lse, attn_mask, mask_tile128, causal, dropout_mask, keep_prob, alibi,
                            alibi_slopes, prev_block_num, next_block_num, scale, seq_lens, tri_block=tri_block,
                            dropout_seed=dropout_seed, dropout_offset=dropout_offset, mask_tiles=mask_tiles)
    with torch.cuda.device(q.device):
        check(lib.acct_fa_fwd(C.byref(a), _stream()))
    del keep
    return o, lse


def fa_backward(q, k, v, o, lse, d_o, attn_mask=None, *, mask_tile128=False, causal=False,
                dropout_mask=None, keep_prob=1.0, alibi=None, alibi_slopes=None,
                prev_block_num=BAND_UNBOUNDED, next_block_num=BAND_UNBOUNDED, scale=1.0, seq_lens=None,
                grads_fp32=False, tri_block=0, deterministic=False, dropout_seed=None, dropout_offset=0,
                kernel_events=None, mask_tiles=None, out=None, workspace=None):
    """Grad primitive: returns (dq, dk, dv), fp32 when ``grads_fp32`` (what the reference primitive
    returns) else in q's dtype (what its bprop hands back after the cast).

    ``out`` = (dq, dk, dv) to write into and ``workspace`` = a uint8 CUDA tensor of at least
    ``acct_fa_bwd_workspace_bytes`` bytes (see ``fa_backward_workspace_bytes``), for callers that want no allocation
    inside their step loop."""
    lib = load()
    _require_cuda("o", o)
    _require_cuda("d_o", d_o)
    _require_cuda("lse", lse)
    if d_o.stride() != o.stride():
        d_o = d_o.contiguous()
        o = o.contiguous()
    gdt = torch.float32 if grads_fp32 else q.dtype
    if out is not None:
        dq, dk, dv = out
        for t, like in ((dq, q), (dk, k), (dv, v)):
            if t.shape != like.shape or t.dtype != gdt or not t.is_contiguous() or not t.is_cuda:
                raise ValueError("out must be contiguous CUDA tensors (dq, dk, dv) shaped like q, k, v in the gradient dtype")
    else:
        dq = torch.empty(q.shape, dtype=gdt, device=q.device)
        dk = torch.empty(k.shape, dtype=gdt, device=q.device)
        dv = torch.empty(v.shape, dtype=gdt, device=q.device)
    lse = lse.contiguous()
    a, keep = _fill_fa_args(q, k, v, o, lse, attn_mask, mask_tile128, causal, dropout_mask, keep_prob, alibi,
                            alibi_slopes, prev_block_num, next_block_num, scale, seq_lens,
                            flags=(FLAG_GRAD_F32 if grads_fp32 else 0) | (FLAG_DETERMINISTIC if deterministic else 0),
                            tri_block=tri_block, dropout_seed=dropout_seed, dropout_offset=dropout_offset,
                            mask_tiles=mask_tiles)
    nbytes = lib.acct_fa_bwd_workspace_bytes(C.byref(a))
    if workspace is not None:
        if workspace.dtype != torch.uint8 or not workspace.is_cuda or workspace.numel() < nbytes or workspace.data_ptr() % 256:
            raise ValueError(f"workspace must be a 256-byte aligned uint8 CUDA tensor of at least {nbytes} bytes")
        ws = workspace
    else:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    g = FaBwdIO()
    g.d_o, g.dq, g.dk, g.dv = d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    g.workspace, g.workspace_bytes = ws.data_ptr(), nbytes
    if kernel_events is not None:     # (start, stop) torch.cuda.Event pair recorded around the main kernel only
        for ev in kernel_events:
            if not ev.cuda_event:     # torch creates the underlying event lazily: force it
                ev.record()
        g.ev_kernel_start, g.ev_kernel_stop = kernel_events[0].cuda_event, kernel_events[1].cuda_event
    with torch.cuda.device(q.device):
        check(lib.acct_fa_bwd(C.byref(a), C.byref(g), _stream()))
    del keep
    return dq, dk, dv


def fa_backward_workspace_bytes(q, k, grads_fp32=False):
    """Bytes of scratch ``fa_backward`` needs for inputs shaped like q [B,N,S_q,D] and k [B,N_kv,S_k,D]."""
    a = FaArgs()
    a.B, a.N, a.S_q, a.D = q.shape
    a.S_k = k.shape[2]
    a.flags = FLAG_GRAD_F32 if grads_fp32 else 0
    return int(load().acct_fa_bwd_workspace_bytes(C.byref(a)))


_causal_cache = {}     # id(tensor) -> (weak reference to that tensor, its version counter, answer)
_tiles_cache = {}      # the same for mask_tile_classes()


def _recall(cache, t):
    hit = cache.get(id(t))
    if hit is not None and hit[0]() is t and hit[1] == t._version:
        return hit
    return None


def _remember(cache, t, answer):
    if len(cache) > 64:
        for k_ in [k_ for k_, v_ in cache.items() if v_[0]() is None]:
            del cache[k_]
        if len(cache) > 64:
            cache.clear()
    cache[id(t)] = (weakref.ref(t), t._version, answer)


def mask_tile_classes(attn_mask):
    """uint8 tensor [Bm, ceil(S_q/128), ceil(S_k/128)] for the ``mask_tiles`` argument of fa_forward / fa_backward:
    0 where the 128x128 tile of ``attn_mask`` ([S_q,S_k] or [Bm,S_q,S_k]) is all 0, 2 where it is all 1, else 1.
    One pass over the mask on the GPU, no synchronisation.  Remembered per tensor object and version counter, like
    mask_is_causal(): a mask that is built once and used by many layers and steps is summarised once."""
    if attn_mask is None or attn_mask.dim() not in (2, 3) or attn_mask.dtype not in _DTYPES:
        raise ValueError("attn_mask must be a [S_q,S_k] or [Bm,S_q,S_k] tensor of float16, bfloat16 or uint8")
    _require_cuda("attn_mask", attn_mask)
    hit = _recall(_tiles_cache, attn_mask)
    if hit is not None:
        return hit[2]
    m = attn_mask.contiguous()
    if m.dim() == 2:
        m = m.unsqueeze(0)
    lib = load()
    tiles = torch.empty((m.shape[0], -(-m.shape[1] // 128), -(-m.shape[2] // 128)), dtype=torch.uint8, device=m.device)
    assert tiles.numel() == lib.acct_mask_tiles_bytes(m.shape[0], m.shape[1], m.shape[2])
    with torch.cuda.device(m.device):
        check(lib.acct_mask_classify_tiles(m.data_ptr(), _dtype_code(m, "attn_mask"), m.shape[0], m.shape[1], m.shape[2],
                                           tiles.data_ptr(), _stream()))
    _remember(_tiles_cache, attn_mask, tiles)
    return tiles


def mask_is_causal(attn_mask):
    """True iff ``attn_mask`` ([S_q,S_k] or [Bm,S_q,S_k]) is exactly the causal mask (1 where key > query, else 0).
    Reads the tensor once on the GPU and synchronises.  The answer is remembered for the tensor OBJECT (held by weak
    reference, so a new tensor that happens to reuse the address of a freed one is inspected afresh) and its version
    counter (so in-place edits are noticed): a mask that is built once and reused is inspected once."""
    if attn_mask is None or attn_mask.dim() not in (2, 3) or attn_mask.dtype not in _DTYPES:
        return False
    _require_cuda("attn_mask", attn_mask)
    hit = _recall(_causal_cache, attn_mask)
    if hit is not None:
        return hit[2]
    m = attn_mask.contiguous()
    if m.dim() == 2:
        m = m.unsqueeze(0)
    out = C.c_int32(0)
    with torch.cuda.device(m.device):
        check(load().acct_mask_is_causal(m.data_ptr(), _dtype_code(m, "attn_mask"), m.shape[0], m.shape[1], m.shape[2],
                                         C.byref(out), _stream()))
    _remember(_causal_cache, attn_mask, bool(out.value))
    return bool(out.value)


def dropout_mask(B, N, S_q, S_k, keep_prob, dropout_seed, dropout_offset=0, device="cuda"):
    """The uint8 {0,1} mask [B,N,S_q,S_k] that in-kernel dropout with these values uses (for checks, or for a caller
    that wants the tensor form)."""
    lib = load()
    dev = torch.device(device)
    mask = torch.empty((B, N, S_q, S_k), dtype=torch.uint8, device=dev)
    a = FaArgs()
    a.B, a.N, a.S_q, a.S_k = B, N, S_q, S_k
    a.keep_prob = float(keep_prob)
    a.dropout_seed = int(dropout_seed) & 0xFFFFFFFFFFFFFFFF
    a.dropout_offset = int(dropout_offset)
    with torch.cuda.device(dev):
        check(lib.acct_dropout_mask(C.byref(a), mask.data_ptr(), _stream()))
    return mask


def infer_prefill(q, k, v, *, causal=False, scale=1.0, seq_lens=None):
    """The inference op y = softmax(scale * q k^T) v on rank-3 [B*N,S,D] or rank-4 [B,N,S,D] input."""
    lib = load()
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda(name, t)
    rank = q.dim()
    if rank not in (3, 4):
        raise ValueError("q must have rank 3 or 4")
    if k.dim() != rank or v.dim() != rank or k.shape != v.shape:
        raise ValueError("k and v must have q's rank and one shape")
    q4, k4, v4 = (t.contiguous() if rank == 4 else t.contiguous().unsqueeze(0) for t in (q, k, v))
    if q4.shape[0] != k4.shape[0] or q4.shape[3] != k4.shape[3] or q4.shape[1] % k4.shape[1] != 0:
        raise ValueError("q and k must agree on batch and head_dim, and k's head count must divide q's")
    y = torch.empty_like(q4)
    a = InferArgs()
    a.dtype = _DTYPES[q.dtype] if q.dtype in (torch.float16, torch.bfloat16) else -1
    a.rank = rank
    a.B, a.N, a.S_q, a.D = q4.shape[0], q4.shape[1], q4.shape[2], q4.shape[3]
    a.S_k = k4.shape[2]
    a.N_kv = k4.shape[1]
    a.q, a.k, a.v, a.y = q4.data_ptr(), k4.data_ptr(), v4.data_ptr(), y.data_ptr()
    a.causal = 1 if causal else 0
    a.scale = float(scale)
    sl = None
    if seq_lens is not None:
        sl = seq_lens.to(torch.int32).contiguous()
        a.seq_lens = sl.data_ptr()
    with torch.cuda.device(q.device):
        check(lib.acct_infer_prefill(C.byref(a), _stream()))
    return y if rank == 4 else y.squeeze(0)


class DecodeWorkspace:
    """Caller-owned scratch for ``infer_decode`` (partial results of the key splits)."""

    def __init__(self, B, N, D, device, num_splits=0):
        a = DecodeArgs()
        a.B, a.N, a.D, a.num_splits = B, N, D, num_splits
        self.nbytes = load().acct_infer_decode_workspace_bytes(C.byref(a))
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)


def infer_decode(q, k_cache, v_cache, seq_lens=None, *, scale=None, num_splits=0, workspace=None, out=None,
                 block_table=None):
    """y[b,n,0,:] = softmax(scale * q K[:len_b]^T) V[:len_b] for q [B,N,1,D], caches [B,N_kv,S_max,D]
    (N_kv = N, or N / N_kv in {2, 4, 8}: grouped-query attention, the heads of a group share one pass over the cache).

    With ``block_table`` ([B, max_pages] int32) the caches are page pools [num_pages, N_kv, page_size, D] and key
    position s of sequence b is row s % page_size of page block_table[b, s // page_size]."""
    lib = load()
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache)):
        _require_cuda(name, t)
    B, N, one, D = q.shape
    if one != 1:
        raise ValueError("decode takes one query token: q must be [B, N, 1, D]")
    N_kv = k_cache.shape[1]
    paged = block_table is not None
    if (k_cache.shape != v_cache.shape or (not paged and k_cache.shape[0] != B) or k_cache.shape[3] != D or N_kv < 1
            or N % N_kv != 0):
        raise ValueError("k_cache and v_cache must be [B, N_kv, S_max, D] (or page pools [pages, N_kv, page_size, D]) "
                         "with N_kv dividing q's head count")
    if k_cache.stride() != v_cache.stride():
        raise ValueError("k_cache and v_cache must share strides")
    q = q.contiguous()
    y = out if out is not None else torch.empty_like(q)
    if workspace is None:
        workspace = DecodeWorkspace(B, N, D, q.device, num_splits)
    a = DecodeArgs()
    a.dtype = _DTYPES.get(q.dtype, -1)
    a.B, a.N, a.D = B, N, D
    a.N_kv = N_kv
    bt = None
    if paged:
        _require_cuda("block_table", block_table)
        bt = block_table.to(torch.int32).contiguous()
        if bt.dim() != 2 or bt.shape[0] != B:
            raise ValueError("block_table must be [B, max_pages]")
        a.block_table = bt.data_ptr()
        a.page_size, a.max_pages = k_cache.shape[2], bt.shape[1]
        a.S_max = a.page_size * a.max_pages
    else:
        a.S_max = k_cache.shape[2]
    a.q, a.k_cache, a.v_cache, a.y = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), y.data_ptr()
    a.kv_stride = _strides3(k_cache)
    sl = None
    if seq_lens is not None:
        sl = seq_lens.to(torch.int32).contiguous()
        a.seq_lens = sl.data_ptr()
    a.scale = float(scale if scale is not None else 1.0 / math.sqrt(D))
    a.num_splits = num_splits
    a.workspace, a.workspace_bytes = workspace.buf.data_ptr(), workspace.nbytes
    with torch.cuda.device(q.device):
        check(lib.acct_infer_decode(C.byref(a), _stream()))
    del bt, sl
    return y
