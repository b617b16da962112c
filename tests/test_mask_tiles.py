"""Per-tile summary of an attn_mask tensor (acct_mask_classify_tiles / acct_fa_args.mask_tiles).

With the summary the kernels read only the 128x128 tiles of the mask that are neither all 0 nor all 1; the results
must be those of reading every tile.  The masks here are the kinds a caller builds that are NOT the causal mask
(which the cells recognise and replace by the in-kernel triangle): documents packed into one sequence, a padded
batch, a prefix that every query sees.  The reference reads such a mask tile by tile for every head
(train/acctransformer/flash_attention/ops/flash_attention/flash_attention_fwd.py:352-361,
flash_attention_bwd.py:359-372).
"""
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref as ref

pytestmark = pytest.mark.gpu

O_TOL = 2e-3
G_TOL = 1e-2


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib
    _lib.load()
    return torch.device("cuda", 0)


def _ops():
    from acctransformer_b200 import ops
    return ops


def _np(t):
    return t.detach().float().cpu().numpy()


def _document_mask(s_q, s_k, bounds):
    """1 = masked.  Query i sees key j iff both lie in the same document and j <= i."""
    doc_q = np.searchsorted(bounds, np.arange(s_q), side="right")
    doc_k = np.searchsorted(bounds, np.arange(s_k), side="right")
    visible = (doc_q[:, None] == doc_k[None, :]) & (np.arange(s_k)[None, :] <= np.arange(s_q)[:, None])
    return (~visible).astype(np.float32)


def _classes_np(mask):
    """Brute-force classes of a [Bm, S_q, S_k] mask."""
    bm, s_q, s_k = mask.shape
    tq, tk = -(-s_q // 128), -(-s_k // 128)
    out = np.empty((bm, tq, tk), np.uint8)
    for b in range(bm):
        for i in range(tq):
            for j in range(tk):
                t = mask[b, i * 128:(i + 1) * 128, j * 128:(j + 1) * 128]
                out[b, i, j] = 0 if not t.any() else (2 if (t == 1).all() else 1)
    return out


@pytest.mark.parametrize("dtype", [torch.uint8, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 384, 384), (3, 333, 451), (2, 128, 1000)])
def test_classes_against_brute_force(dev, dtype, shape):
    rs = np.random.RandomState(5)
    bm, s_q, s_k = shape
    mask = np.zeros(shape, np.float32)
    tq, tk = -(-s_q // 128), -(-s_k // 128)
    kinds = rs.randint(0, 4, (bm, tq, tk))
    for b in range(bm):
        for i in range(tq):
            for j in range(tk):
                blk = mask[b, i * 128:(i + 1) * 128, j * 128:(j + 1) * 128]
                if kinds[b, i, j] == 1:
                    blk[...] = 1.0
                elif kinds[b, i, j] == 2:
                    blk[...] = (rs.random_sample(blk.shape) < 0.5)
                elif kinds[b, i, j] == 3:                  # a single element differs from an otherwise uniform tile
                    base = float(rs.randint(0, 2))
                    blk[...] = base
                    blk[rs.randint(blk.shape[0]), rs.randint(blk.shape[1])] = 1.0 - base
    m = torch.tensor(mask).to(dtype).to(dev)
    got = _ops().mask_tile_classes(m).cpu().numpy()
    assert got.shape == (bm, tq, tk)
    np.testing.assert_array_equal(got, _classes_np(mask))


def test_a_value_other_than_zero_or_one_makes_the_tile_mixed(dev):
    mask = torch.zeros(1, 256, 256, dtype=torch.float16, device=dev)
    mask[0, :128, 128:] = 1.0
    mask[0, 128:, :128] = 0.5          # uniform, but neither 0 nor 1: must be read
    got = _ops().mask_tile_classes(mask).cpu().numpy()
    np.testing.assert_array_equal(got[0], [[0, 2], [1, 0]])


def test_summary_is_remembered_per_tensor_and_version(dev):
    ops = _ops()
    mask = torch.zeros(1, 256, 256, dtype=torch.uint8, device=dev)
    t1 = ops.mask_tile_classes(mask)
    assert ops.mask_tile_classes(mask) is t1
    mask[0, 0, 200] = 1                 # in-place edit bumps the version counter
    t2 = ops.mask_tile_classes(mask)
    assert t2 is not t1
    np.testing.assert_array_equal(t2.cpu().numpy()[0], [[0, 1], [0, 0]])


@pytest.mark.parametrize("case", ["documents", "padded_batch", "prefix_gqa"])
def test_forward_backward_with_summary_match_oracle_and_full_read(dev, case):
    ops = _ops()
    rs = np.random.RandomState(17)
    if case == "documents":
        B, N, N_kv, S_q, S_k, D = 1, 2, 2, 1024, 1024, 64
        mask = _document_mask(S_q, S_k, np.array([200, 512, 900]))[None]
    elif case == "padded_batch":
        B, N, N_kv, S_q, S_k, D = 2, 2, 2, 300, 700, 128
        mask = np.zeros((B, S_q, S_k), np.float32)
        mask[0, :, 450:] = 1.0          # keys past each sequence's length are masked
        mask[1, :, 128:] = 1.0
    else:
        B, N, N_kv, S_q, S_k, D = 1, 4, 2, 512, 512, 128
        causal = np.triu(np.ones((S_q, S_k), np.float32), 1)
        causal[:, :160] = 0.0           # every query sees the first 160 keys
        mask = causal[None]
    want_classes = _classes_np(mask)
    assert {0, 1, 2} <= set(want_classes.ravel().tolist())
    q = torch.tensor(rs.randn(B, N, S_q, D).astype(np.float32)).half()
    k = torch.tensor(rs.randn(B, N_kv, S_k, D).astype(np.float32)).half()
    v = torch.tensor(rs.randn(B, N_kv, S_k, D).astype(np.float32)).half()
    do = torch.tensor(rs.randn(B, N, S_q, D).astype(np.float32)).half()
    scale = 1.0 / math.sqrt(D)
    m_dev = torch.tensor(mask).half().to(dev)
    tiles = ops.mask_tile_classes(m_dev)
    np.testing.assert_array_equal(tiles.cpu().numpy(), want_classes)

    args = [t.to(dev) for t in (q, k, v)]
    o1, l1 = ops.fa_forward(*args, m_dev, scale=scale, mask_tiles=tiles)
    o0, l0 = ops.fa_forward(*args, m_dev, scale=scale)
    g1 = ops.fa_backward(*args, o1, l1, do.to(dev), m_dev, scale=scale, mask_tiles=tiles)
    g0 = ops.fa_backward(*args, o0, l0, do.to(dev), m_dev, scale=scale)
    from acctransformer_b200 import _lib
    torch.cuda.synchronize()
    _lib.device_status()

    o_ref, l_ref = ref.gqa_fwd(q.numpy(), k.numpy(), v.numpy(), attn_mask=mask, scale=scale)
    g_ref = ref.gqa_grad(q.numpy(), k.numpy(), v.numpy(), do.numpy(), attn_mask=mask, scale=scale)
    assert float(np.max(np.abs(_np(o1) - o_ref))) <= O_TOL
    assert float(np.max(np.abs(_np(l1) - l_ref))) <= O_TOL
    for got, full, want, name in zip(g1, g0, g_ref, ("dq", "dk", "dv")):
        rel = float(np.max(np.abs(_np(got) - want)) / np.max(np.abs(want)))
        assert rel <= G_TOL, f"{name}: relative error {rel}"
        # skipping the all-0 / all-1 tiles changes rounding at most (the masked scores get the same -10000)
        assert float(np.max(np.abs(_np(got) - _np(full)))) <= 2e-3 * max(1.0, float(np.max(np.abs(want)))), name
    assert float(np.max(np.abs(_np(o1) - _np(o0)))) <= 1e-3


def test_cell_uses_the_summary_for_a_mask_that_is_not_causal(dev):
    from acctransformer_b200.flash_attention.nn.layer.flash_attention import FlashAttention
    ops = _ops()
    rs = np.random.RandomState(23)
    B, N, S, D = 1, 2, 512, 64
    mask = _document_mask(S, S, np.array([130, 300]))[None]
    q, k, v = (torch.tensor(rs.randn(B, N, S, D).astype(np.float32)).half().to(dev).requires_grad_(True) for _ in range(3))
    m_dev = torch.tensor(mask).half().to(dev)
    cell = FlashAttention(head_dim=D)
    o = cell(q, k, v, m_dev)
    assert ops._recall(ops._tiles_cache, m_dev) is not None        # the cell summarised the mask
    o.sum().backward()
    scale = 1.0 / math.sqrt(D)          # what the cell's two multiplications by head_dim^-1/4 amount to
    o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), attn_mask=mask, scale=scale)
    assert float(np.max(np.abs(_np(o) - o_ref))) <= O_TOL
    g_ref = ref.sa_grad(_np(q), _np(k), _np(v), np.ones_like(o_ref), attn_mask=mask, scale=scale)
    rel = float(np.max(np.abs(_np(v.grad) - g_ref[2])) / np.max(np.abs(g_ref[2])))
    assert rel <= G_TOL
