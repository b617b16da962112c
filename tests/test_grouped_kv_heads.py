"""Grouped-query / multi-query attention: key and value tensors with fewer heads than the query.
The reference asks its users to tile K and V up to the query's head count (nn/layer/flash_attention.py:193-196);
the oracle does exactly that tiling, the kernels read the shared heads in place."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref as ref


def test_oracle_head_tiling_and_its_gradient():
    rs = np.random.RandomState(0)
    x = rs.randn(2, 2, 5, 4).astype(np.float32)
    e = ref.expand_kv_heads(x, 6)
    assert e.shape == (2, 6, 5, 4)
    for n in range(6):
        assert (e[:, n] == x[:, n // 3]).all()
    g = rs.randn(2, 6, 5, 4).astype(np.float32)
    r = ref.reduce_kv_heads(g, 2)
    assert np.allclose(r[:, 1], g[:, 3] + g[:, 4] + g[:, 5])
    # <expand(x), g> == <x, reduce(g)>  (adjointness)
    assert np.isclose((e * g).sum(), (x * r).sum(), rtol=1e-5)


def test_cell_refuses_fewer_kv_heads_unless_told():
    from acctransformer_b200.flash_attention.nn.layer.flash_attention import FlashAttention
    cell = FlashAttention(head_dim=64)
    q = torch.zeros(1, 4, 128, 64, dtype=torch.float16)
    k = torch.zeros(1, 2, 128, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="head_num of query, key and value must be the same"):
        cell(q, k, k)
    cell.allow_grouped_kv = True
    k3 = torch.zeros(1, 3, 128, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="head_num of query, key and value must be the same"):
        cell(q, k3, k3)          # 3 does not divide 4


def _np(t):
    return t.detach().float().cpu().numpy()


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib
    _lib.load()
    return torch.device("cuda", 0)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype, B, N, N_kv, S_q, S_k, D, kw", [
    (torch.float16, 2, 4, 2, 384, 384, 64, dict(causal=True)),
    (torch.float16, 1, 8, 1, 256, 520, 128, dict()),                       # multi-query, ragged keys
    (torch.bfloat16, 1, 6, 2, 300, 300, 128, dict(causal=True)),
    (torch.float16, 1, 4, 2, 640, 640, 128, dict(prev_block_num=1, next_block_num=2)),
])
def test_forward_and_backward_with_fewer_kv_heads(dev, dtype, B, N, N_kv, S_q, S_k, D, kw):
    from acctransformer_b200 import ops, _lib
    rs = np.random.RandomState(3)
    mk = lambda n, s: torch.tensor(rs.randn(B, n, s, D).astype(np.float32) * 0.8).to(dtype).to(dev)
    q, k, v, do = mk(N, S_q), mk(N_kv, S_k), mk(N_kv, S_k), mk(N, S_q)
    scale = 1.0 / math.sqrt(D)
    alibi_np = np.ascontiguousarray(ref.alibi_bias(B, N, S_k))
    alibi = torch.tensor(alibi_np).to(dtype).to(dev)
    o, lse = ops.fa_forward(q, k, v, scale=scale, alibi=alibi, **kw)
    dq, dk, dv = ops.fa_backward(q, k, v, o, lse, do, scale=scale, alibi=alibi, **kw)
    torch.cuda.synchronize()
    _lib.device_status()
    assert dk.shape == k.shape and dv.shape == v.shape
    al32 = _np(alibi)
    o_ref, l_ref = ref.gqa_fwd(_np(q), _np(k), _np(v), scale=scale, alibi=al32, **kw)
    tol = 2e-3 if dtype == torch.float16 else 8e-3
    assert np.max(np.abs(_np(o) - o_ref)) <= tol
    assert np.max(np.abs(_np(lse) - l_ref)) <= 2e-3
    g_ref = ref.gqa_grad(_np(q), _np(k), _np(v), _np(do), scale=scale, alibi=al32, **kw)
    for got, want, name in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
        err = np.max(np.abs(_np(got) - want)) / np.max(np.abs(want))
        assert err <= (1e-2 if dtype == torch.float16 else 2e-2), (name, err)
    # the same as tiling K and V by hand, which is what the reference tells its users to do
    group = N // N_kv
    kt, vt = k.repeat_interleave(group, dim=1), v.repeat_interleave(group, dim=1)
    o_t, lse_t = ops.fa_forward(q, kt, vt, scale=scale, alibi=alibi, **kw)
    assert torch.equal(o, o_t) and torch.equal(lse, lse_t)


@pytest.mark.gpu
def test_prefill_and_decode_with_fewer_kv_heads(dev):
    from acctransformer_b200 import ops
    rs = np.random.RandomState(4)
    B, N, D, S = 3, 8, 128, 700
    for N_kv in (8, 4, 2, 1):
        q = torch.tensor(rs.randn(B, N, 1, D).astype(np.float32)).half().to(dev)
        kc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).half().to(dev)
        vc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).half().to(dev)
        lens = torch.tensor([700, 1, 333], dtype=torch.int32, device=dev)
        y = ops.infer_decode(q, kc, vc, lens)
        scale = 1.0 / math.sqrt(D)
        y_ref = ref.decode_ref(_np(q), ref.expand_kv_heads(_np(kc), N), ref.expand_kv_heads(_np(vc), N),
                               lens.cpu().numpy(), scale)
        assert np.max(np.abs(_np(y) - y_ref)) <= 2e-3, N_kv
    # prefill, causal
    qp = torch.tensor(rs.randn(1, 8, 256, 64).astype(np.float32)).half().to(dev)
    kp = torch.tensor(rs.randn(1, 2, 256, 64).astype(np.float32)).half().to(dev)
    vp = torch.tensor(rs.randn(1, 2, 256, 64).astype(np.float32)).half().to(dev)
    yp = ops.infer_prefill(qp, kp, vp, causal=True, scale=0.125)
    yp_ref = ref.infer_fwd(_np(qp), ref.expand_kv_heads(_np(kp), 8), ref.expand_kv_heads(_np(vp), 8), scale=0.125,
                           causal=True)
    assert np.max(np.abs(_np(yp) - yp_ref)) <= 2e-3
    # above head_dim 128 the groups are 2, 4 or 8 heads; 3 is refused there
    with pytest.raises(Exception):
        ops.infer_decode(torch.zeros(1, 6, 1, 160, dtype=torch.float16, device=dev),
                         torch.zeros(1, 2, 64, 160, dtype=torch.float16, device=dev),
                         torch.zeros(1, 2, 64, 160, dtype=torch.float16, device=dev))


@pytest.mark.gpu
@pytest.mark.parametrize("D, N, N_kv, dtype, S", [(128, 32, 4, torch.float16, 5000), (128, 12, 4, torch.float16, 333),
                                                   (128, 16, 1, torch.bfloat16, 2100), (64, 10, 2, torch.float16, 1000),
                                                   (40, 6, 2, torch.float16, 777), (80, 14, 1, torch.float16, 4097),
                                                   (128, 4, 2, torch.float16, 16)])
def test_decode_with_the_group_on_tensor_cores(dev, D, N, N_kv, dtype, S):
    """Groups of 2 to 16 query heads per cache head at head_dim <= 128 (3, 5, 7, 14 and 16 included), ragged lengths
    that end inside a 16-row tile, a length of 1, every split count, head_dim that is not a multiple of 16."""
    from acctransformer_b200 import ops
    rs = np.random.RandomState(18)
    B = 3
    q = torch.tensor(rs.randn(B, N, 1, D).astype(np.float32)).to(dtype).to(dev)
    kc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).to(dtype).to(dev)
    vc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).to(dtype).to(dev)
    lens = torch.tensor([S, 1, max(1, S // 3 + 5)], dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(D)
    y_ref = ref.decode_ref(_np(q), ref.expand_kv_heads(_np(kc), N), ref.expand_kv_heads(_np(vc), N), lens.cpu().numpy(), scale)
    tol = 2e-3 if dtype == torch.float16 else 8e-3
    for splits in (0, 1, 5):
        y = ops.infer_decode(q, kc, vc, lens, scale=scale, num_splits=splits)
        torch.cuda.synchronize()
        assert np.max(np.abs(_np(y) - y_ref)) <= tol, splits


@pytest.mark.gpu
@pytest.mark.parametrize("D, N, N_kv, dtype", [(64, 8, 1, torch.float16), (64, 8, 2, torch.bfloat16), (256, 8, 1, torch.float16),
                                               (256, 16, 4, torch.float16), (80, 8, 2, torch.float16)])
def test_decode_group_sizes_at_other_head_dims(dev, D, N, N_kv, dtype):
    """Groups of 4 and 8 query heads share their score reduction across the lanes of a cache row; the number of lanes
    per row depends on head_dim (8, 16 or 32), so every width is checked."""
    from acctransformer_b200 import ops
    rs = np.random.RandomState(8)
    B, S = 2, 1500
    q = torch.tensor(rs.randn(B, N, 1, D).astype(np.float32)).to(dtype).to(dev)
    kc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).to(dtype).to(dev)
    vc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).to(dtype).to(dev)
    lens = torch.tensor([1500, 77], dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(D)
    y = ops.infer_decode(q, kc, vc, lens, scale=scale)
    y_ref = ref.decode_ref(_np(q), ref.expand_kv_heads(_np(kc), N), ref.expand_kv_heads(_np(vc), N), lens.cpu().numpy(), scale)
    tol = 2e-3 if dtype == torch.float16 else 8e-3
    assert np.max(np.abs(_np(y) - y_ref)) <= tol


@pytest.mark.gpu
@pytest.mark.parametrize("N_kv, page", [(8, 16), (2, 64), (1, 256)])
def test_decode_over_a_paged_cache(dev, N_kv, page):
    """Paged caches give the same bits as the contiguous cache they were cut from."""
    from acctransformer_b200 import ops
    rs = np.random.RandomState(6)
    B, N, D = 4, 8, 128
    lens_list = [1000, 17, 512, 1]
    max_pages = (max(lens_list) + page - 1) // page
    S = max_pages * page
    q = torch.tensor(rs.randn(B, N, 1, D).astype(np.float32)).half().to(dev)
    kc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).half().to(dev)
    vc = torch.tensor(rs.randn(B, N_kv, S, D).astype(np.float32)).half().to(dev)
    lens = torch.tensor(lens_list, dtype=torch.int32, device=dev)
    y_flat = ops.infer_decode(q, kc, vc, lens, num_splits=4)
    # scatter the pages of every sequence over a shuffled pool (with some unused pages in between)
    n_pool = B * max_pages + 5
    perm = rs.permutation(n_pool)[:B * max_pages].reshape(B, max_pages)
    kp = torch.zeros(n_pool, N_kv, page, D, dtype=torch.float16, device=dev)
    vp = torch.full((n_pool, N_kv, page, D), float("nan"), dtype=torch.float16, device=dev)
    for b in range(B):
        for pg in range(max_pages):
            kp[perm[b, pg]] = kc[b, :, pg * page:(pg + 1) * page]
            vp[perm[b, pg]] = vc[b, :, pg * page:(pg + 1) * page]
    table = torch.tensor(perm.astype(np.int32), device=dev)
    y_paged = ops.infer_decode(q, kp, vp, lens, num_splits=4, block_table=table)
    assert torch.equal(y_paged, y_flat)
    scale = 1.0 / math.sqrt(D)
    y_ref = ref.decode_ref(_np(q), ref.expand_kv_heads(_np(kc), N), ref.expand_kv_heads(_np(vc), N), np.array(lens_list), scale)
    assert np.max(np.abs(_np(y_paged) - y_ref)) <= 2e-3


@pytest.mark.gpu
def test_grouped_heads_with_in_kernel_dropout_and_mask_tensor(dev):
    """Everything that is indexed per QUERY head (dropout stream, alibi row) or per batch (mask) keeps its meaning when
    the key/value heads are shared."""
    from acctransformer_b200 import ops, _lib
    rs = np.random.RandomState(8)
    B, N, N_kv, S, D = 2, 4, 2, 320, 64
    mk = lambda n: torch.tensor(rs.randn(B, n, S, D).astype(np.float32) * 0.8).half().to(dev)
    q, k, v, do = mk(N), mk(N_kv), mk(N_kv), mk(N)
    mask_np = (rs.rand(B, S, S) < 0.2).astype(np.float16)
    mask = torch.tensor(mask_np).to(dev)
    keep, seed, offset = 0.75, 4242, 11
    scale = 1.0 / math.sqrt(D)
    o, lse = ops.fa_forward(q, k, v, mask, scale=scale, keep_prob=keep, dropout_seed=seed, dropout_offset=offset)
    dq, dk, dv = ops.fa_backward(q, k, v, o, lse, do, mask, scale=scale, keep_prob=keep, dropout_seed=seed,
                                 dropout_offset=offset)
    torch.cuda.synchronize()
    _lib.device_status()
    m_ref = ref.dropout_mask_philox(B, N, S, S, keep, seed, offset)
    keep_eff = ref.dropout_threshold(keep) / 256.0
    o_ref, l_ref = ref.gqa_fwd(_np(q), _np(k), _np(v), attn_mask=mask_np.astype(np.float32), drop_mask=m_ref,
                               keep_prob=keep_eff, scale=scale)
    assert np.max(np.abs(_np(o) - o_ref)) <= 2e-3
    assert np.max(np.abs(_np(lse) - l_ref)) <= 2e-3
    g_ref = ref.gqa_grad(_np(q), _np(k), _np(v), _np(do), attn_mask=mask_np.astype(np.float32), drop_mask=m_ref,
                         keep_prob=keep_eff, scale=scale)
    for got, want, name in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
        err = np.max(np.abs(_np(got) - want)) / np.max(np.abs(want))
        assert err <= 1e-2, (name, err)
