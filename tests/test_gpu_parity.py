"""Parity of the CUDA path (called through the C ABI) with the CPU oracle on the same seeded inputs.

Tolerances (stated by the benchmark definition, versus an fp32 reference):
  O and L:      max |x - x_ref| <= 2e-3            (fp16; bf16 outputs carry an 8-bit significand, see BF16_O_TOL)
  dQ, dK, dV:   max |g - g_ref| / max |g_ref| <= 1e-2
The reference's own two-threshold criterion (tests/train/flash_attention/st/common.py:178-192) is
checked as well wherever the reference tests use it.
"""
import math
import os

import numpy as np
import pytest
import torch

from oracle import attention_ref as ref

pytestmark = pytest.mark.gpu

O_TOL = 2e-3
BF16_O_TOL = 8e-3      # half a bf16 ulp at |O| < 2
G_TOL = 1e-2


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib
    _lib.load()     # raises if the CUDA library is missing: no silent fallback
    return torch.device("cuda", 0)


def _ops():
    from acctransformer_b200 import ops
    return ops


def _status():
    from acctransformer_b200 import _lib
    torch.cuda.synchronize()
    _lib.device_status()


def _np(t):
    return t.detach().float().cpu().numpy()


def _rand(shape, seed, dtype=torch.float16, std=1.0, dist="randn"):
    rs = np.random.RandomState(seed)
    x = rs.randn(*shape) if dist == "randn" else rs.random_sample(shape)
    return torch.tensor((x * std).astype(np.float32)).to(dtype)


def _check_o(o, o_ref, tol=O_TOL):
    err = float(np.max(np.abs(_np(o) - o_ref)))
    assert err <= tol, f"max|O - O_ref| = {err}"


def _check_g(g, g_ref, name):
    rel = float(np.max(np.abs(_np(g) - g_ref)) / np.max(np.abs(g_ref)))
    assert rel <= G_TOL, f"{name}: relative error {rel}"


def _to_np16(t):
    return t.float().numpy().astype(np.float32) if t.dtype == torch.bfloat16 else t.numpy()


# ---------------------------------------------------------------------------------------------
# golden fixtures produced by the reference's own NumPy functions
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["fa_cfg1_randn_triu", "fa_st_128x80_uniform_triu", "fa_st_128x80_randn_triu",
                                  "fa_st_1x2x256x128_uniform_nomask"])
def test_raw_primitive_against_reference_goldens(dev, golden_dir, name):
    from acctransformer_b200 import get_flash_attention, get_flash_attention_grad
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    q, k, v, do = (torch.tensor(g[x]).to(dev) for x in ("q", "k", "v", "do"))
    s = q.shape[2]
    masked = str(g["mask_kind"]) == "triu"
    mask = torch.triu(torch.ones(1, s, s, dtype=torch.float16, device=dev), diagonal=1) if masked else None
    # the reference tests run the raw primitive (no scaling) with next_block_num=0 under the triu mask
    fa = get_flash_attention(next_block_num=0 if masked else 65536)
    o, lse = fa(q, k, v, mask)
    fa_grad = get_flash_attention_grad(next_block_num=0 if masked else 65536)
    dq, dk, dv = fa_grad(q, k, v, o, do, lse, mask)
    _status()
    assert dq.dtype == torch.float32       # the primitive returns fp32 gradients
    npmask = _np(mask) if masked else None
    o_ref, l_ref = ref.sa_fwd(g["q"], g["k"], g["v"], npmask)
    _check_o(o, o_ref)
    assert float(np.max(np.abs(_np(lse) - l_ref))) <= O_TOL
    gq, gk, gv = ref.sa_grad(g["q"], g["k"], g["v"], g["do"], npmask)
    for a, b, n in ((dq, gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
        _check_g(a, b, n)
    # and against the reference functions' own fp16 outputs, by the reference tests' criteria
    if str(g["dist"]) == "uniform":
        _, p1, p2 = ref.data_compare(g["o"].astype(np.float32), _np(o))
        assert p2 == 0 and p1 < 1e-2
    for a, b in ((dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        rel = float(np.max(np.abs(_np(a) - b.astype(np.float32))) / np.max(np.abs(b.astype(np.float32))))
        assert rel <= G_TOL


@pytest.mark.parametrize("name", ["infer_1x2x256x384x64", "infer_1x1x512x512x40"])
def test_infer_op_against_reference_golden(dev, golden_dir, name):
    from acctransformer_b200 import flash_attention_tik
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    q, k, v = (torch.tensor(g[x]).to(dev) for x in ("query", "key", "value"))
    y = flash_attention_tik(q, k, v)
    _status()
    gold = g["golden"].astype(np.float32)
    _check_o(y, ref.infer_fwd(g["query"], g["key"], g["value"]))
    assert np.allclose(_np(y), gold, rtol=0.05, atol=2e-3)        # tests/infer/.../compare.py:53 uses rtol 0.05
    b, n, s, d = q.shape
    y3 = flash_attention_tik(q.reshape(b * n, s, d), k.reshape(b * n, -1, d), v.reshape(b * n, -1, d))
    assert torch.equal(y3.reshape(y.shape), y)


# ---------------------------------------------------------------------------------------------
# the benchmark configurations (sub-sampled in batch/heads where the oracle is O(S^2) per unit)
# ---------------------------------------------------------------------------------------------
def test_config1_cell_with_full_causal_mask_tensor(dev):
    from acctransformer_b200 import FlashAttention
    B, N, S, D = 1, 2, 256, 64
    q, k, v = (_rand((B, N, S, D), 1 + i) for i in range(3))
    mask = torch.triu(torch.ones(1, S, S, dtype=torch.float16), diagonal=1)
    layer = FlashAttention(head_dim=D)
    o = layer(q.to(dev), k.to(dev), v.to(dev), mask.to(dev))
    _status()
    o_ref, _ = ref.sa_fwd(q.numpy(), k.numpy(), v.numpy(), mask.numpy(), scale=1.0 / math.sqrt(D))
    _check_o(o, o_ref)
    # the cell as the reference computes it: q and k each scaled by fp16(d^-1/4) in fp16, raw primitive
    o_cell, _ = ref.sa_fwd(ref.cell_scale(q.numpy(), D), ref.cell_scale(k.numpy(), D), v.numpy(), mask.numpy())
    _check_o(o, o_cell, tol=4e-3)


def test_config2_causal_plus_alibi_forward_backward(dev):
    ops = _ops()
    B, N, S, D = 2, 16, 2048, 128      # config 2 with the batch cut from 4 to 2 (units are independent)
    q, k, v, do = (_rand((B, N, S, D), 20 + i) for i in range(4))
    alibi = torch.tensor(ref.alibi_bias(B, N, S))
    scale = 1.0 / math.sqrt(D)
    kw = dict(causal=True, alibi=alibi.to(dev), scale=scale)
    o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev), **kw)
    dq, dk, dv = ops.fa_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, do.to(dev), **kw)
    _status()
    for b in range(B):     # oracle per batch entry to bound its memory
        sl = slice(b, b + 1)
        okw = dict(causal=True, alibi=alibi[sl].numpy(), scale=scale)
        o_ref, l_ref = ref.sa_fwd(q[sl].numpy(), k[sl].numpy(), v[sl].numpy(), **okw)
        _check_o(o[sl], o_ref)
        assert float(np.max(np.abs(_np(lse[sl]) - l_ref))) <= O_TOL
        gq, gk, gv = ref.sa_grad(q[sl].numpy(), k[sl].numpy(), v[sl].numpy(), do[sl].numpy(), **okw)
        for a, r, n in ((dq, gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
            _check_g(a[sl], r, n)
    # slopes given instead of a bias tensor: the bias slope_h * j is then formed in fp32 inside the kernel
    slopes = torch.tensor(ref.alibi_slopes(N), dtype=torch.float32, device=dev)
    o2, _ = ops.fa_forward(q[:1].to(dev), k[:1].to(dev), v[:1].to(dev), causal=True, alibi_slopes=slopes, scale=scale)
    _status()
    o2_ref, _ = ref.sa_fwd(q[:1].numpy(), k[:1].numpy(), v[:1].numpy(), causal=True, scale=scale,
                           alibi=ref.alibi_bias(1, N, S, np.float32))
    _check_o(o2, o2_ref)


def test_config3_bf16_band_dropout_one_unit_full_length(dev):
    ops = _ops()
    B, N, S, D = 1, 1, 8192, 128
    q, k, v, do = (_rand((B, N, S, D), 30 + i, torch.bfloat16, std=0.5) for i in range(4))
    rs = np.random.RandomState(33)
    drop = torch.tensor((rs.random_sample((B, N, S, S)) < 0.9).astype(np.uint8))
    kw = dict(dropout_mask=drop.to(dev), keep_prob=0.9, prev_block_num=4, next_block_num=4, scale=1.0 / math.sqrt(D))
    o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev), **kw)
    dq, dk, dv = ops.fa_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, do.to(dev), **kw)
    _status()
    okw = dict(drop_mask=drop.numpy(), keep_prob=0.9, prev_block_num=4, next_block_num=4, scale=1.0 / math.sqrt(D))
    qn, kn, vn, don = (_to_np16(t) for t in (q, k, v, do))
    o_ref, l_ref = ref.sa_fwd(qn, kn, vn, **okw)
    assert float(np.max(np.abs(o_ref))) < 0.5       # keeps bf16 output rounding under the 2e-3 budget
    _check_o(o, o_ref)
    assert float(np.max(np.abs(_np(lse) - l_ref))) <= O_TOL
    gq, gk, gv = ref.sa_grad(qn, kn, vn, don, **okw)
    for a, r, n in ((dq, gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
        _check_g(a, r, n)


@pytest.mark.parametrize("S, block, assume_causal", [(4096, 512, False), (4608, 1024, False), (1000, 300, False),
                                                      (4096, 512, True)])
def test_config4_triangle_attention_forward_backward(dev, S, block, assume_causal):
    from acctransformer_b200 import TriangleAttention
    B, N, D = 1, 2, 128
    q, k, v, do = (_rand((B, N, S, D), 40 + i) for i in range(4))
    q = (q.float() / math.sqrt(D)).to(torch.float16)          # the caller pre-scales q (no scaling inside)
    mask = torch.triu(torch.ones(B, S, S, dtype=torch.float16), diagonal=1)
    layer = TriangleAttention(block_size=block, assume_causal=assume_causal)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    o = layer(qd, kd, vd, mask.to(dev))
    o.backward(do.to(dev))
    _status()
    o_ref = ref.triangle_fwd(q.numpy(), k.numpy(), v.numpy(), mask.numpy(), block_size=block)
    _check_o(o, o_ref)
    gq, gk, gv = ref.sa_grad(q.numpy(), k.numpy(), v.numpy(), do.numpy(), mask.numpy())
    for a, r, n in ((qd.grad, gq, "dq"), (kd.grad, gk, "dk"), (vd.grad, gv, "dv")):
        _check_g(a, r, n)


def test_triangle_attention_with_a_non_causal_mask_keeps_group_bounds(dev):
    # an all-zero mask: rows see every key up to the end of their own row group and nothing beyond
    from acctransformer_b200 import TriangleAttention
    B, N, S, D, block = 1, 1, 640, 64, 256
    q, k, v = (_rand((B, N, S, D), 50 + i, std=0.3) for i in range(3))
    mask = torch.zeros(B, S, S, dtype=torch.float16)
    o = TriangleAttention(block_size=block)(q.to(dev), k.to(dev), v.to(dev), mask.to(dev))
    _status()
    _check_o(o, ref.triangle_fwd(q.numpy(), k.numpy(), v.numpy(), mask.numpy(), block_size=block))


def test_config5_prefill_causal_and_decode(dev):
    from acctransformer_b200 import flash_attention_decode, flash_attention_tik
    B, N, S, D = 1, 2, 4096, 128
    q, k, v = (_rand((B, N, S, D), 60 + i) for i in range(3))
    scale = 1.0 / math.sqrt(D)
    y = flash_attention_tik(q.to(dev), k.to(dev), v.to(dev), scale=scale, causal=True)
    _status()
    _check_o(y, ref.infer_fwd(q.numpy(), k.numpy(), v.numpy(), scale=scale, causal=True))
    # decode over a 16384-long cache with per-sequence valid lengths
    B, N, S = 4, 3, 16384
    qd = _rand((B, N, 1, D), 70)
    kc, vc = _rand((B, N, S, D), 71), _rand((B, N, S, D), 72)
    lens = torch.tensor([1024, 16384, 7777, 1], dtype=torch.int32)
    for splits in (0, 1, 7):
        yd = flash_attention_decode(qd.to(dev), kc.to(dev), vc.to(dev), lens.to(dev), scale=scale, num_splits=splits)
        _status()
        _check_o(yd, ref.decode_ref(qd.numpy(), kc.numpy(), vc.numpy(), lens.numpy(), scale))


@pytest.mark.parametrize("D, S_q, S_k, causal", [(160, 512, 512, False), (160, 300, 700, False), (256, 384, 384, True),
                                                    (192, 1024, 1024, True)])
def test_forward_head_dims_above_128(dev, D, S_q, S_k, causal):
    # the inference op's envelope includes head_dim 160 (infer/flash_attention/tik/tbe/impl/flash_attention_fwd.py:34-40),
    # the cell's goes up to 256 (nn/layer/flash_attention.py:26)
    from acctransformer_b200 import flash_attention_tik
    B, N = 1, 2
    q = _rand((B, N, S_q, D), 140, std=0.5)
    k, v = _rand((B, N, S_k, D), 141, std=0.5), _rand((B, N, S_k, D), 142, std=0.5)
    y = flash_attention_tik(q.to(dev), k.to(dev), v.to(dev), scale=1.0 / math.sqrt(D), causal=causal)
    _status()
    _check_o(y, ref.infer_fwd(q.numpy(), k.numpy(), v.numpy(), scale=1.0 / math.sqrt(D), causal=causal))
    ops = _ops()
    o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev), causal=causal, scale=1.0 / math.sqrt(D))
    _status()
    _, l_ref = ref.sa_fwd(q.numpy(), k.numpy(), v.numpy(), causal=causal, scale=1.0 / math.sqrt(D))
    assert float(np.max(np.abs(_np(lse) - l_ref))) <= O_TOL
    # and the backward at these widths (two CTAs per K/V tile, one per half of head_dim)
    do = _rand((B, N, S_q, D), 143, std=0.5)
    grads = ops.fa_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, do.to(dev), causal=causal, scale=1.0 / math.sqrt(D))
    _status()
    g_ref = ref.sa_grad(q.numpy(), k.numpy(), v.numpy(), do.numpy(), causal=causal, scale=1.0 / math.sqrt(D))
    for g, want, name in zip(grads, g_ref, ("dq", "dk", "dv")):
        _check_g(g, want, name)


@pytest.mark.parametrize("D, what, backward", [(64, "alibi", True), (64, "mask", True), (64, "slopes+dropout", True),
                                               (128, "alibi", True), (128, "mask+philox", True), (128, "slopes", True),
                                               (160, "mask", True), (160, "alibi+dropout", True), (256, "slopes", True),
                                               (192, "mask+philox", True)])
def test_every_kernel_variant_of_every_width(dev, D, what, backward):
    """The kernels are compiled per head_dim width (64 / 128 / 256) and per combination of mask, alibi and dropout
    kind; head_dim 128 has every combination, the other widths fold mask and alibi into one variant.  One case per
    family, ragged lengths, forward and backward against the oracle."""
    ops = _ops()
    B, N, S_q, S_k = 2, 2, 200, 333
    scale = 1.0 / math.sqrt(D)
    q, k, v, do = (_rand((B, N, S, D), 150 + i, std=0.6) for i, S in enumerate((S_q, S_k, S_k, S_q)))
    kw, okw = dict(scale=scale), dict(scale=scale)
    mask = None
    if "mask" in what:
        m = (np.random.RandomState(3).random_sample((B, S_q, S_k)) < 0.3).astype(np.float32)
        m[:, :, 0] = 0.0                                   # every row keeps a key
        mask = torch.tensor(m).half().to(dev)
        okw["attn_mask"] = m
    if "alibi" in what:
        al = ref.alibi_bias(B, N, S_k, np.float32)
        kw["alibi"] = torch.tensor(al).half().to(dev)
        okw["alibi"] = _np(kw["alibi"])
    if "slopes" in what:
        sl = np.asarray(ref.alibi_slopes(N), np.float32)
        kw["alibi_slopes"] = torch.tensor(sl, device=dev)
        okw["alibi"] = (sl[None, :, None, None] * np.arange(S_k, dtype=np.float32)[None, None, None, :]).repeat(B, 0)
    if "dropout" in what:
        dm = (np.random.RandomState(4).random_sample((B, N, S_q, S_k)) < 0.8).astype(np.uint8)
        kw.update(dropout_mask=torch.tensor(dm).to(dev), keep_prob=0.8)
        okw.update(drop_mask=dm, keep_prob=0.8)
    if "philox" in what:
        kw.update(keep_prob=0.75, dropout_seed=77, dropout_offset=5)
        okw.update(drop_mask=ref.dropout_mask_philox(B, N, S_q, S_k, 0.75, 77, 5), keep_prob=ref.dropout_threshold(0.75) / 256.0)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    o, lse = ops.fa_forward(qd, kd, vd, mask, **kw)
    _status()
    o_ref, l_ref = ref.sa_fwd(q.numpy(), k.numpy(), v.numpy(), **okw)
    _check_o(o, o_ref)
    assert float(np.max(np.abs(_np(lse) - l_ref))) <= O_TOL
    if backward:
        grads = ops.fa_backward(qd, kd, vd, o, lse, do.to(dev), mask, **kw)
        _status()
        g_ref = ref.sa_grad(q.numpy(), k.numpy(), v.numpy(), do.numpy(), **okw)
        for g, want, name in zip(grads, g_ref, ("dq", "dk", "dv")):
            _check_g(g, want, name)


# ---------------------------------------------------------------------------------------------
# edge cases taken from the reference tests' shape lists, and ragged / mixed-option cases
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("q_shape, kv_shape", [((1, 1, 256, 128), (1, 1, 128 * 1024, 128)),
                                               ((1, 1, 128 * 1024, 128), (1, 1, 256, 128)),
                                               ((4, 8, 128, 80), (4, 8, 128, 80)),
                                               ((1, 1, 200, 40), (1, 1, 333, 40))])
def test_cross_lengths_without_mask(dev, q_shape, kv_shape):
    # tests/train/flash_attention/st/test_fa_fwd_precision.py:69-94 (uniform inputs, no mask, raw primitive)
    ops = _ops()
    q = _rand(q_shape, 80, dist="uniform")
    k, v = _rand(kv_shape, 81, dist="uniform"), _rand(kv_shape, 82, dist="uniform")
    o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev))
    _status()
    o_ref, l_ref = ref.sa_fwd(q.numpy(), k.numpy(), v.numpy())
    _check_o(o, o_ref)
    res, p1, p2 = ref.data_compare(o_ref, _np(o))
    assert res == "Pass", (p1, p2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_everything_at_once_ragged(dev, dtype):
    ops = _ops()
    B, N, Sq, Sk, D = 2, 3, 333, 451, 80
    std = 0.5 if dtype == torch.bfloat16 else 1.0
    q, do = _rand((B, N, Sq, D), 90, dtype, std), _rand((B, N, Sq, D), 93, dtype, std)
    k, v = _rand((B, N, Sk, D), 91, dtype, std), _rand((B, N, Sk, D), 92, dtype, std)
    rs = np.random.RandomState(94)
    mask = torch.tensor((rs.random_sample((B, Sq, Sk)) < 0.2).astype(np.float16))
    drop = torch.tensor((rs.random_sample((B, N, Sq, Sk)) < 0.8).astype(np.uint8))
    alibi = torch.tensor(ref.alibi_bias(B, N, Sk, np.float32)).to(dtype)
    kw = dict(dropout_mask=drop.to(dev), keep_prob=0.8, alibi=alibi.to(dev), prev_block_num=1, next_block_num=2, scale=0.11)
    o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev), mask.to(dev), **kw)
    dq, dk, dv = ops.fa_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, do.to(dev), mask.to(dev), **kw)
    _status()
    okw = dict(attn_mask=mask.numpy(), drop_mask=drop.numpy(), keep_prob=0.8, alibi=_to_np16(alibi), prev_block_num=1,
               next_block_num=2, scale=0.11)
    qn, kn, vn, don = (_to_np16(t) for t in (q, k, v, do))
    o_ref, l_ref = ref.sa_fwd(qn, kn, vn, **okw)
    _check_o(o, o_ref, O_TOL if dtype == torch.float16 else BF16_O_TOL)
    assert float(np.max(np.abs(_np(lse) - l_ref))) <= O_TOL
    gq, gk, gv = ref.sa_grad(qn, kn, vn, don, **okw)
    for a, r, n in ((dq, gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
        _check_g(a, r, n)


def test_prescaled_16bit_dropout_mask_equals_uint8_form(dev):
    ops = _ops()
    B, N, S, D = 1, 2, 256, 64
    q, k, v = (_rand((B, N, S, D), 100 + i).to(dev) for i in range(3))
    keep = (torch.rand(B, N, S, S, device=dev) < 0.75)
    a, _ = ops.fa_forward(q, k, v, dropout_mask=keep.to(torch.uint8), keep_prob=0.75, scale=0.125)
    b, _ = ops.fa_forward(q, k, v, dropout_mask=(keep.to(torch.float16) / 0.75), scale=0.125)
    _status()
    assert float((a.float() - b.float()).abs().max()) <= 1e-3       # 1/0.75 rounded to fp16 in the second form


def test_strided_inputs(dev):
    # q, k, v as views into one packed [B, S, 3, N, D] projection output
    ops = _ops()
    B, N, S, D = 2, 4, 384, 128
    qkv = _rand((B, S, 3, N, D), 110).to(dev)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o, _ = ops.fa_forward(q, k, v, causal=True, scale=0.09)
    _status()
    o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), causal=True, scale=0.09)
    _check_o(o, o_ref)


def test_seq_lens_zero_and_full(dev):
    from acctransformer_b200 import flash_attention_tik
    B, N, S, D = 3, 2, 300, 64
    q, k, v = (_rand((B, N, S, D), 120 + i) for i in range(3))
    lens = torch.tensor([0, 300, 129], dtype=torch.int32)
    y = flash_attention_tik(q.to(dev), k.to(dev), v.to(dev), scale=0.125, seq_lens=lens.to(dev))
    _status()
    assert float(y[0].float().abs().max()) == 0.0              # no valid key: defined as zeros
    y_ref = ref.infer_fwd(q.numpy()[1:], k.numpy()[1:], v.numpy()[1:], scale=0.125, seq_lens=lens.numpy()[1:])
    _check_o(y[1:], y_ref)


def test_band_that_leaves_q_tiles_without_keys(dev):
    # S_q > S_k + prev_block_num * 128: the trailing Q tiles lie outside the band of every K/V tile.  Their rows are
    # defined as zeros (output and dQ; the reference leaves them undefined), and no K/V tile ever adds into their dQ,
    # so the backward cannot leave the 16-bit conversion of dQ to "the last tile that adds".
    ops = _ops()
    B, N, Sq, Sk, D = 1, 2, 640, 128, 64
    q, do = _rand((B, N, Sq, D), 140), _rand((B, N, Sq, D), 143)
    k, v = _rand((B, N, Sk, D), 141), _rand((B, N, Sk, D), 142)
    kw = dict(prev_block_num=1, scale=0.125)
    o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev), **kw)
    dq = torch.full((B, N, Sq, D), 7.0, dtype=torch.float16, device=dev)        # stale contents must not survive
    dk, dv = torch.empty(B, N, Sk, D, dtype=torch.float16, device=dev), torch.empty(B, N, Sk, D, dtype=torch.float16, device=dev)
    ops.fa_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, do.to(dev), out=(dq, dk, dv), **kw)
    _status()
    seen = 256                                                                   # rows of Q tiles 0 and 1
    assert float(o[:, :, seen:].float().abs().max()) == 0.0
    assert float(dq[:, :, seen:].float().abs().max()) == 0.0
    o_ref, _ = ref.sa_fwd(q.numpy()[:, :, :seen], k.numpy(), v.numpy(), **kw)
    _check_o(o[:, :, :seen], o_ref)
    gq, gk, gv = ref.sa_grad(q.numpy()[:, :, :seen], k.numpy(), v.numpy(), do.numpy()[:, :, :seen], **kw)
    for a, r, n in ((dq[:, :, :seen], gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
        _check_g(a, r, n)


@pytest.mark.parametrize("kw", [dict(causal=True), dict(), dict(prev_block_num=2, next_block_num=1), dict(tri_block=384)])
def test_deterministic_backward_is_bit_reproducible(dev, kw):
    # the reference requires run-to-run equality of its gradients (tests/train/flash_attention/st/test_sharding.py:91-115)
    ops = _ops()
    B, N, S, D = 2, 3, 1024 + 72, 128
    q, k, v, do = (_rand((B, N, S, D), 130 + i).to(dev) for i in range(4))
    o, lse = ops.fa_forward(q, k, v, scale=0.09, **kw)
    runs = [ops.fa_backward(q, k, v, o, lse, do, scale=0.09, deterministic=True, **kw) for _ in range(3)]
    _status()
    for other in runs[1:]:
        for a, b_ in zip(runs[0], other):
            assert torch.equal(a, b_)
    loose = ops.fa_backward(q, k, v, o, lse, do, scale=0.09, **kw)
    _status()
    for a, b_ in zip(runs[0], loose):
        assert float((a.float() - b_.float()).abs().max()) <= 1e-2 * float(a.float().abs().max())


# ---------------------------------------------------------------------------------------------
# size-independent properties at the benchmark's full sizes
# ---------------------------------------------------------------------------------------------
def test_headline_size_shard_equivalence_determinism_and_linearity(dev):
    ops = _ops()
    from acctransformer_b200.workloads import make_inputs
    inp = make_inputs("H", dev)
    q, k, v, do, scale = inp["q"], inp["k"], inp["v"], inp["do"], inp["scale"]
    o, lse = ops.fa_forward(q, k, v, causal=True, scale=scale)
    o_again, lse_again = ops.fa_forward(q, k, v, causal=True, scale=scale)
    assert torch.equal(o, o_again) and torch.equal(lse, lse_again)                 # run-to-run determinism
    # batch split: each half alone gives bit-identical results (tests/train/flash_attention/st/test_sharding.py:19-38)
    o_half, lse_half = ops.fa_forward(q[1:], k[1:], v[1:], causal=True, scale=scale)
    assert torch.equal(o_half, o[1:]) and torch.equal(lse_half, lse[1:])
    # linearity in V: doubling V doubles O exactly (power-of-two scaling commutes with every rounding)
    # except where the fp16 result is subnormal (below 2^-14), where one subnormal ulp (2^-24) may be lost
    o2, _ = ops.fa_forward(q, k, v * 2, causal=True, scale=scale)
    assert float((o2.float() - 2 * o.float()).abs().max()) <= 2.0 ** -23
    big = o.float().abs() >= 2.0 ** -13
    assert torch.equal(o2[big], (o * 2)[big])
    dq, dk, dv = ops.fa_backward(q, k, v, o, lse, do, causal=True, scale=scale)
    dq_h, dk_h, dv_h = ops.fa_backward(q[1:], k[1:], v[1:], o[1:], lse[1:], do[1:], causal=True, scale=scale)
    assert torch.equal(dk_h, dk[1:]) and torch.equal(dv_h, dv[1:])                 # dK, dV have a fixed summation order
    # dQ is reduced with floating-point atomics: order-dependent in the last bits only
    assert float((dq_h.float() - dq[1:].float()).abs().max()) <= 1e-2 * float(dq.float().abs().max())
    # linearity in dO
    dq2, dk2, dv2 = ops.fa_backward(q, k, v, o * 2, lse, do * 2, causal=True, scale=scale)
    assert float((dv2.float() - 2 * dv.float()).abs().max()) <= 2.0 ** -23
    _status()
    # the first and the last (batch, head) unit against the oracle at full length
    for sl in ((slice(0, 1), slice(0, 1)), (slice(1, 2), slice(31, 32))):
        qn, kn, vn, don = (_np(t[sl]).astype(np.float16) for t in (q, k, v, do))
        o_ref, l_ref = ref.sa_fwd(qn, kn, vn, causal=True, scale=scale)
        _check_o(o[sl], o_ref)
        assert float(np.max(np.abs(_np(lse[sl]) - l_ref))) <= O_TOL
        gq, gk, gv = ref.sa_grad(qn, kn, vn, don, causal=True, scale=scale)
        for a, r, n in ((dq, gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
            _check_g(a[sl], r, n)


def test_causal_mask_tensor_is_detected_and_not_read(dev):
    """A mask tensor that is exactly the causal mask is recognised once and replaced by the in-kernel triangle;
    any other mask keeps going through the tensor path.  Results agree with the oracle either way."""
    ops = _ops()
    from acctransformer_b200.flash_attention.nn.layer.flash_attention import FlashAttention
    from acctransformer_b200.triangle_attention.triangle_attention import TriangleAttention
    B, N, S, D = 2, 2, 512, 64
    q, k, v = (_rand((B, N, S, D), s).to(dev) for s in (21, 22, 23))
    causal = torch.triu(torch.ones(S, S), 1).half().expand(B, S, S).contiguous().to(dev)
    other = causal.clone()
    other[1, 100, 3] = 1.0                      # one extra masked position in batch entry 1
    assert ops.mask_is_causal(causal) and not ops.mask_is_causal(other)
    assert ops.mask_is_causal(causal[0]) and ops.mask_is_causal(causal.to(torch.uint8))
    # the answer follows in-place edits of the same tensor
    causal[0, 5, 2] = 1.0
    assert not ops.mask_is_causal(causal)
    causal[0, 5, 2] = 0.0
    assert ops.mask_is_causal(causal)
    # a NEW tensor at the address of a freed one is inspected afresh (the answer belongs to the object, not the address)
    tmp = torch.triu(torch.ones(S, S), 1).half().to(dev)
    assert ops.mask_is_causal(tmp)
    addr = tmp.data_ptr()
    del tmp
    tmp2 = torch.zeros(S, S, dtype=torch.float16, device=dev)
    if tmp2.data_ptr() == addr:                 # the caching allocator normally hands the block straight back
        assert not ops.mask_is_causal(tmp2)

    cell = FlashAttention(head_dim=D)
    scale = 1.0 / math.sqrt(D)
    for mask in (causal, other):
        o = cell(q, k, v, mask)
        o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), attn_mask=_np(mask), scale=scale)
        _check_o(o, o_ref)
    cell.detect_causal_mask = False
    o_tensor_path = cell(q, k, v, causal)
    o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), attn_mask=_np(causal), scale=scale)
    _check_o(o_tensor_path, o_ref)

    ta = TriangleAttention(block_size=128)
    qs = (q.float() * scale).half()             # the layer applies no scale: its callers pre-scale q
    for mask in (causal, other):
        o = ta(qs, k, v, mask)
        o_ref = ref.triangle_fwd(_np(qs), _np(k), _np(v), _np(mask), 128)
        _check_o(o, o_ref)
    _status()


def test_cell_with_the_128x128_tile_mask_form(dev):
    """have_attention_mask_batch=False: the [1,128,128] tile acts on the diagonal tiles only
    (flash_attention_fwd.py:352-361).  With next_block_num = 0 a strict-upper-triangle tile is the causal mask and the
    cell lets the kernels generate it; any other tile, or a band that reaches above the diagonal, is read."""
    from acctransformer_b200.flash_attention.nn.layer.flash_attention import FlashAttention
    B, N, S, D = 1, 2, 640, 64
    scale = 1.0 / math.sqrt(D)
    q, k, v = (_rand((B, N, S, D), s).to(dev).requires_grad_(True) for s in (31, 32, 33))
    triu = torch.triu(torch.ones(1, 128, 128), 1).half().to(dev)
    odd = triu.clone()
    odd[0, 7, 3] = 1.0                           # not the causal tile: must be read
    for tile, nxt in ((triu, 0), (odd, 0), (triu, 2)):
        cell = FlashAttention(head_dim=D, next_block_num=nxt, have_attention_mask_batch=False)
        o = cell(q, k, v, tile)
        full = ref.expand_tile_mask(_np(tile), S, S)
        o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), attn_mask=full, scale=scale, prev_block_num=65536, next_block_num=nxt)
        _check_o(o, o_ref)
        for t in (q, k, v):
            t.grad = None
        o.sum().backward()
        g_ref = ref.sa_grad(_np(q), _np(k), _np(v), np.ones_like(o_ref), attn_mask=full, scale=scale,
                            prev_block_num=65536, next_block_num=nxt)
        for t, want, name in zip((q, k, v), g_ref, ("dq", "dk", "dv")):
            _check_g(t.grad, want, name)
    _status()


@pytest.mark.parametrize("D, dtype, kw", [(160, torch.float16, dict(causal=True)),
                                          (256, torch.bfloat16, dict(prev_block_num=1, next_block_num=1)),
                                          (200, torch.float16, dict(tri_block=300)),
                                          (256, torch.float16, dict(causal=True, kv_heads=1))])
def test_backward_head_dims_above_128(dev, D, dtype, kw):
    """The reference cell accepts head_dim up to 256 (nn/layer/flash_attention.py:26,105-106; its Wukong shapes use
    40, 80 and 160).  Forward + backward at such widths, ragged lengths, fp32 and 16-bit gradients, grouped heads,
    deterministic dQ, and the cell itself."""
    ops = _ops()
    kw = dict(kw)
    n_kv = kw.pop("kv_heads", None)
    B, N, S_q, S_k = 2, 2, 333, 451
    if kw.get("causal") or "tri_block" in kw:
        S_k = S_q
    std = 0.5
    q, do = _rand((B, N, S_q, D), 160, dtype, std), _rand((B, N, S_q, D), 163, dtype, std)
    k, v = _rand((B, n_kv or N, S_k, D), 161, dtype, std), _rand((B, n_kv or N, S_k, D), 162, dtype, std)
    scale = 1.0 / math.sqrt(D)
    qd, kd, vd, dod = (t.to(dev) for t in (q, k, v, do))
    o, lse = ops.fa_forward(qd, kd, vd, scale=scale, **kw)
    qn, kn, vn, don = (_to_np16(t) for t in (q, k, v, do))
    okw = dict(kw)
    tri = okw.pop("tri_block", None)
    if tri:     # the oracle's TriangleAttention takes the group bound as an all-zero mask plus the block size
        o_ref = ref.triangle_fwd(qn * scale, kn, vn, np.zeros((B, S_q, S_k), np.float32), block_size=tri)
        gmask = (np.arange(S_k)[None, :] >= ((np.arange(S_q)[:, None] // tri + 1) * tri)).astype(np.float32)
        okw = dict(attn_mask=np.broadcast_to(gmask * 1e4, (B, S_q, S_k)))     # far below any score: excluded
        _check_o(o, o_ref, O_TOL if dtype == torch.float16 else BF16_O_TOL)
        g_ref = ref.sa_grad(qn, kn, vn, don, scale=scale, **okw)
    elif n_kv:
        g_ref = ref.gqa_grad(qn, kn, vn, don, scale=scale, **okw)
    else:
        o_ref, _ = ref.sa_fwd(qn, kn, vn, scale=scale, **okw)
        _check_o(o, o_ref, O_TOL if dtype == torch.float16 else BF16_O_TOL)
        g_ref = ref.sa_grad(qn, kn, vn, don, scale=scale, **okw)
    for fp32 in (False, True):
        grads = ops.fa_backward(qd, kd, vd, o, lse, dod, scale=scale, grads_fp32=fp32, **kw)
        _status()
        assert grads[0].dtype == (torch.float32 if fp32 else dtype)
        for g, want, name in zip(grads, g_ref, ("dq", "dk", "dv")):
            rel = float(np.max(np.abs(_np(g) - want)) / np.max(np.abs(want)))
            assert rel <= (G_TOL if dtype == torch.float16 or fp32 else 2e-2), f"{name} fp32={fp32}: {rel}"
    runs = [ops.fa_backward(qd, kd, vd, o, lse, dod, scale=scale, deterministic=True, **kw) for _ in range(2)]
    _status()
    for a, b_ in zip(*runs):
        assert torch.equal(a, b_)
    for a, b_ in zip(runs[0], grads):
        assert float((a.float() - b_.float()).abs().max()) <= 1e-2 * float(b_.float().abs().max())


def test_cell_trains_at_head_dim_160(dev):
    from acctransformer_b200 import FlashAttention
    B, N, S, D = 1, 2, 384, 160
    q, k, v, do = (_rand((B, N, S, D), 170 + i, std=0.5) for i in range(4))
    mask = torch.triu(torch.ones(1, S, S, dtype=torch.float16), diagonal=1)
    layer = FlashAttention(head_dim=D)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    o = layer(qd, kd, vd, mask.to(dev))
    o.backward(do.to(dev))
    _status()
    scale = 1.0 / math.sqrt(D)
    o_ref, _ = ref.sa_fwd(q.numpy(), k.numpy(), v.numpy(), mask.numpy(), scale=scale)
    _check_o(o, o_ref)
    for g, want, name in zip((qd.grad, kd.grad, vd.grad),
                             ref.sa_grad(q.numpy(), k.numpy(), v.numpy(), do.numpy(), mask.numpy(), scale=scale), ("dq", "dk", "dv")):
        _check_g(g, want, name)


def test_caller_provided_outputs_and_workspace(dev):
    """fa_forward / fa_backward write into tensors the caller brings (for step loops that must not allocate) and give
    the same bits as the allocating form."""
    ops = _ops()
    B, N, S, D = 2, 3, 300, 64
    q, k, v, do = (_rand((B, N, S, D), 180 + i).to(dev) for i in range(4))
    o_ref, lse_ref = ops.fa_forward(q, k, v, causal=True, scale=0.125)
    g_ref = ops.fa_backward(q, k, v, o_ref, lse_ref, do, causal=True, scale=0.125, deterministic=True)
    o, lse = torch.empty_like(q), torch.empty(B, N, S, dtype=torch.float32, device=dev)
    got = ops.fa_forward(q, k, v, causal=True, scale=0.125, out=o, lse_out=lse)
    assert got[0] is o and got[1] is lse and torch.equal(o, o_ref) and torch.equal(lse, lse_ref)
    outs = tuple(torch.empty_like(t) for t in (q, k, v))
    ws = torch.empty(ops.fa_backward_workspace_bytes(q, k) + 512, dtype=torch.uint8, device=dev)
    ws = ws[(-ws.data_ptr()) % 256:]
    for _ in range(2):          # the workspace is reused as it is: the call re-initialises what it needs
        g = ops.fa_backward(q, k, v, o, lse, do, causal=True, scale=0.125, deterministic=True, out=outs, workspace=ws)
        _status()
        for a, b_, c in zip(g, outs, g_ref):
            assert a is b_ and torch.equal(a, c)
    with pytest.raises(ValueError):
        ops.fa_backward(q, k, v, o, lse, do, workspace=ws[:1024])
