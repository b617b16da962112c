"""In-kernel dropout: the generator, the mask as a function of the position, and the equivalence of the in-kernel
form with the tensor form given the same mask."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref as ref


# ------------------------------------------------------------------------------------------ CPU
def test_philox_known_answers():
    # known-answer vectors published with the Random123 library (philox4x32, 10 rounds)
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        got = tuple(int(x) for x in ref.philox4x32_10(ctr, key))
        assert got == want


def test_threshold_and_keep_fraction():
    assert ref.dropout_threshold(1.0) == 256
    assert ref.dropout_threshold(0.9) == 230
    assert ref.dropout_threshold(0.5) == 128
    assert ref.dropout_threshold(1e-6) == 1
    m = ref.dropout_mask_philox(2, 3, 64, 200, 0.9, seed=1234, offset=7)
    assert m.shape == (2, 3, 64, 200) and m.dtype == np.uint8 and set(np.unique(m)) <= {0, 1}
    frac = m.mean()
    assert abs(frac - 230 / 256) < 0.01
    # another offset or seed gives another mask; the same values give the same mask
    assert (ref.dropout_mask_philox(2, 3, 64, 200, 0.9, 1234, 8) != m).any()
    assert (ref.dropout_mask_philox(2, 3, 64, 200, 0.9, 1235, 7) != m).any()
    assert (ref.dropout_mask_philox(2, 3, 64, 200, 0.9, 1234, 7) == m).all()
    # rows and units are independent streams: no two rows of a unit are equal
    assert len({r.tobytes() for r in m[0, 0]}) == 64


# ------------------------------------------------------------------------------------------ GPU
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
@pytest.mark.parametrize("shape, keep, seed, offset", [((1, 2, 256, 256), 0.9, 42, 0), ((2, 3, 200, 333), 0.75, 2**40 + 5, 17),
                                                       ((1, 1, 130, 17), 0.5, 7, 2**32 - 1),
                                                       ((1, 1, 64, 48), 1.0, 3, 0), ((1, 2, 40, 70), 0.002, 9, 1)])
def test_materialised_mask_equals_the_oracle(dev, shape, keep, seed, offset):
    from acctransformer_b200 import ops
    B, N, S_q, S_k = shape
    got = ops.dropout_mask(B, N, S_q, S_k, keep, seed, offset, device=dev).cpu().numpy()
    want = ref.dropout_mask_philox(B, N, S_q, S_k, keep, seed, offset)
    assert (got == want).all()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype, B, N, S_q, S_k, D, kw", [
    (torch.float16, 1, 2, 384, 384, 64, dict(causal=True)),
    (torch.bfloat16, 2, 2, 300, 517, 128, dict()),
    (torch.float16, 1, 2, 640, 640, 128, dict(prev_block_num=1, next_block_num=1)),
])
def test_in_kernel_dropout_equals_tensor_form_and_oracle(dev, dtype, B, N, S_q, S_k, D, kw):
    from acctransformer_b200 import ops, _lib
    rs = np.random.RandomState(5)
    q, k, v, do = (torch.tensor(rs.randn(B, N, S, D).astype(np.float32) * 0.7).to(dtype).to(dev)
                   for S in (S_q, S_k, S_k, S_q))
    keep, seed, offset = 0.8, 987654321, 3
    scale = 1.0 / math.sqrt(D)
    t_eff = ref.dropout_threshold(keep) / 256.0      # the keep probability actually applied
    mask = ops.dropout_mask(B, N, S_q, S_k, keep, seed, offset, device=dev)

    o1, l1 = ops.fa_forward(q, k, v, scale=scale, keep_prob=keep, dropout_seed=seed, dropout_offset=offset, **kw)
    o2, l2 = ops.fa_forward(q, k, v, scale=scale, keep_prob=t_eff, dropout_mask=mask, **kw)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)

    g1 = ops.fa_backward(q, k, v, o1, l1, do, scale=scale, keep_prob=keep, dropout_seed=seed, dropout_offset=offset,
                         deterministic=True, **kw)
    g2 = ops.fa_backward(q, k, v, o2, l2, do, scale=scale, keep_prob=t_eff, dropout_mask=mask, deterministic=True, **kw)
    torch.cuda.synchronize()
    _lib.device_status()
    for a_, b_ in zip(g1, g2):
        assert torch.equal(a_, b_)

    # against the oracle, with the oracle's own evaluation of the generator
    m_ref = ref.dropout_mask_philox(B, N, S_q, S_k, keep, seed, offset)
    okw = dict(kw)
    o_ref, l_ref = ref.sa_fwd(_np(q), _np(k), _np(v), drop_mask=m_ref, keep_prob=t_eff, scale=scale, **okw)
    tol = 2e-3 if dtype == torch.float16 else 8e-3
    assert np.max(np.abs(_np(o1) - o_ref)) <= tol
    assert np.max(np.abs(_np(l1) - l_ref)) <= 2e-3
    g_ref = ref.sa_grad(_np(q), _np(k), _np(v), _np(do), drop_mask=m_ref, keep_prob=t_eff, scale=scale, **okw)
    for got, want, name in zip(g1, g_ref, ("dq", "dk", "dv")):
        err = np.max(np.abs(_np(got) - want)) / np.max(np.abs(want))
        assert err <= (1e-2 if dtype == torch.float16 else 2e-2), (name, err)


@pytest.mark.gpu
def test_cell_uses_in_kernel_dropout_and_its_backward_sees_the_same_mask(dev):
    from acctransformer_b200 import ops
    from acctransformer_b200.flash_attention.nn.layer.flash_attention import FlashAttention
    B, N, S, D = 1, 2, 256, 64
    rs = np.random.RandomState(9)
    q, k, v = (torch.tensor(rs.randn(B, N, S, D).astype(np.float32)).half().to(dev).requires_grad_(True) for _ in range(3))
    do = torch.tensor(rs.randn(B, N, S, D).astype(np.float32)).half().to(dev)
    cell = FlashAttention(head_dim=D, dropout_rate=0.25)
    from acctransformer_b200.flash_attention.nn.layer.flash_attention import _draw_dropout_key
    cell.generator = torch.Generator().manual_seed(123)
    seed, offset = _draw_dropout_key(torch.Generator().manual_seed(123))     # what the cell will draw
    cell.train()
    o = cell(q, k, v)
    o.backward(do)
    keep_eff = ref.dropout_threshold(0.75) / 256.0
    m_ref = ref.dropout_mask_philox(B, N, S, S, 0.75, seed, offset)
    scale = 1.0 / math.sqrt(D)
    o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), drop_mask=m_ref, keep_prob=keep_eff, scale=scale)
    assert np.max(np.abs(_np(o) - o_ref)) <= 2e-3
    g_ref = ref.sa_grad(_np(q), _np(k), _np(v), _np(do), drop_mask=m_ref, keep_prob=keep_eff, scale=scale)
    for got, want, name in zip((q.grad, k.grad, v.grad), g_ref, ("dq", "dk", "dv")):
        err = np.max(np.abs(_np(got) - want)) / np.max(np.abs(want))
        assert err <= 1e-2, (name, err)
    # the next step draws another mask; evaluation mode drops nothing
    o2 = cell(q, k, v)
    assert not torch.equal(o2, o)
    # a forward that is recomputed after the generator's state has been put back (what torch.utils.checkpoint
    # does before it re-runs a forward) drops the same positions again
    state = cell.generator.get_state()
    o4 = cell(q, k, v)
    cell.generator.set_state(state)
    assert torch.equal(cell(q, k, v), o4)
    cell.eval()
    o3 = cell(q, k, v)
    o_plain, _ = ref.sa_fwd(_np(q), _np(k), _np(v), scale=scale)
    assert np.max(np.abs(_np(o3) - o_plain)) <= 2e-3
