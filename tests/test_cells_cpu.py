"""Host-side behaviour of the Python layers that needs no GPU: constructor checks raise the
reference's ValueErrors, CPU tensors are refused (there is no CPU path), tile accounting."""
import pytest
import torch

from acctransformer_b200 import FlashAttention, TriangleAttention, flash_attention_tik
from acctransformer_b200.workloads import CONFIGS, band_fraction, fwd_bwd_flops, fwd_flops


def test_flash_attention_ctor_errors_match_reference():
    with pytest.raises(ValueError, match="head_dim too large"):
        FlashAttention(head_dim=257)
    FlashAttention(head_dim=256)
    FlashAttention(head_dim=128, alibi=True)        # accepted here; the reference raises


def test_flash_attention_head_count_check():
    layer = FlashAttention(head_dim=64)
    q = torch.zeros(1, 4, 128, 64, dtype=torch.float16)
    k = torch.zeros(1, 2, 128, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="head_num of query, key and value must be the same"):
        layer(q, k, k)


def test_cpu_tensors_are_refused():
    layer = FlashAttention(head_dim=64)
    q = torch.zeros(1, 2, 128, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        layer(q, q, q)
    with pytest.raises(ValueError, match="CUDA tensor"):
        flash_attention_tik(q, q, q)


@pytest.mark.parametrize("kw", [dict(block_size=0), dict(block_size=-3), dict(dropout_rate=1.0),
                                dict(dropout_rate=-0.1), dict(dp=0), dict(mp=0)])
def test_triangle_ctor_errors_match_reference(kw):
    with pytest.raises(ValueError):
        TriangleAttention(**kw)


def test_triangle_tile_accounting():
    # block 512 at S=4096: the reference computes 36/64 of the dense score matrix; at 128-tile
    # granularity the same trapezoid is 9/16 of the tiles
    ta = TriangleAttention(block_size=512)
    assert abs((1.0 - ta.tiles_skipped_fraction(4096)) - 36.0 / 64.0) < 1e-12
    causal = TriangleAttention(block_size=512, assume_causal=True)
    assert abs((1.0 - causal.tiles_skipped_fraction(4096)) - (32 * 33 / 2) / 1024.0) < 1e-12


def test_infer_shape_errors():
    q = torch.zeros(2, 128, 64, dtype=torch.float16)
    with pytest.raises(ValueError):
        flash_attention_tik(q.unsqueeze(0).unsqueeze(0), q, q)
    with pytest.raises(ValueError, match="same shape"):
        flash_attention_tik(q, q, torch.zeros(2, 64, 64, dtype=torch.float16))


def test_flop_accounting():
    assert abs(fwd_flops(CONFIGS["H"]) / 1e9 - 1099.5) < 0.1
    assert abs(fwd_bwd_flops(CONFIGS["H"]) / 1e9 - 3848.3) < 0.1
    assert abs(fwd_bwd_flops(CONFIGS["cfg2"]) / 1e9 - 240.5) < 0.1
    assert round(band_fraction(8192, 8192, 4, 4) * 4096) == 556
    assert abs(fwd_bwd_flops(CONFIGS["cfg3"]) / 1e9 - 1044.8) < 0.1


def test_band_tile_accounting_matches_the_band_predicate():
    """The tile counts behind the benchmark's flop figures equal a brute-force evaluation of the reference's band
    predicate  j - next <= i <= j + prev  on 128-tiles (flash_attention_fwd.py:444-445), for ragged sizes too."""
    import numpy as np
    from acctransformer_b200.workloads import band_fraction
    from oracle import attention_ref as ref
    rs = np.random.RandomState(0)
    for _ in range(40):
        s_q, s_k = int(rs.randint(1, 1500)), int(rs.randint(1, 1500))
        prev, nxt = int(rs.randint(0, 6)), int(rs.randint(0, 6))
        m = ref.band_mask(s_q, s_k, prev, nxt)
        tq, tk = (s_q + 127) // 128, (s_k + 127) // 128
        tiles = sum(bool(m[i * 128, j * 128]) for i in range(tq) for j in range(tk))
        assert abs(band_fraction(s_q, s_k, prev, nxt) - tiles / float(tq * tk)) < 1e-12
    assert band_fraction(8192, 8192, 4, 4) == 556 / 4096.0          # configuration 3: 556 of 4096 tiles


def test_triangle_skipped_tiles_match_the_row_group_bounds():
    """tiles_skipped_fraction() counts exactly the tiles that lie wholly past their rows' group end
    (triangle_attention.py:137-163: row group g sees keys [0, (g+1)*block_size))."""
    from acctransformer_b200.triangle_attention.triangle_attention import TriangleAttention
    for S, block in ((4096, 512), (1000, 300), (4608, 1024), (129, 128)):
        ta = TriangleAttention(block_size=block)
        nt = (S + 127) // 128
        computed = 0
        for i in range(nt):
            rows = range(i * 128, min(S, i * 128 + 128))
            q_end = max(min(S, (r // block + 1) * block) for r in rows)
            computed += sum(1 for j in range(nt) if j * 128 < q_end)
        assert abs(ta.tiles_skipped_fraction(S) - (1.0 - computed / float(nt * nt))) < 1e-12


def test_reference_import_paths_resolve_to_the_same_objects():
    """A user of the reference imports through ``acctransformer.*`` (train/setup.py:22-31 installs that package);
    the same statements work here and give this library's classes."""
    from acctransformer.flash_attention.nn.layer.flash_attention import FlashAttention
    from acctransformer.flash_attention.ops.flash_attention.flash_attention_impl import (get_flash_attention,
                                                                                         get_flash_attention_grad)
    from acctransformer.triangle_attention.triangle_attention import TriangleAttention
    import acctransformer_b200 as mine
    assert FlashAttention is mine.FlashAttention and TriangleAttention is mine.TriangleAttention
    assert get_flash_attention is mine.get_flash_attention and get_flash_attention_grad is mine.get_flash_attention_grad
    layer = FlashAttention(head_dim=128, dropout_rate=0.1, prev_block_num=4, next_block_num=0, dp=2, mp=4,
                           have_attention_mask_batch=False)
    assert layer.flash_attention.prev_block_num == 4 and layer.flash_attention.next_block_num == 0
    with pytest.raises(ValueError):
        FlashAttention(head_dim=512)
    with pytest.raises(ValueError):
        TriangleAttention(block_size=0)


def test_dropout_key_is_a_function_of_the_generator_state_alone():
    """Replaying the RNG state replays (seed, offset): a forward recomputed under torch.utils.checkpoint, which
    restores the RNG state first, gets the mask of the original forward."""
    import torch
    from acctransformer_b200.flash_attention.nn.layer.flash_attention import _draw_dropout_key
    g = torch.Generator().manual_seed(7)
    state = g.get_state()
    first = _draw_dropout_key(g)
    second = _draw_dropout_key(g)
    assert first != second
    g.set_state(state)
    assert _draw_dropout_key(g) == first
    # the default generator, which checkpointing saves and restores
    state = torch.get_rng_state()
    a = _draw_dropout_key()
    torch.set_rng_state(state)
    assert _draw_dropout_key() == a
    assert 0 <= a[0] < 2 ** 62 and 0 <= a[1] < 2 ** 32


def test_packaging_lists_both_packages_and_the_library():
    """setup.py installs the implementation, the reference's import paths and the shared library (reference:
    train/setup.py:22-31 installs a package named acctransformer)."""
    import ast
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = open(os.path.join(root, "setup.py")).read()
    ast.parse(src)
    from setuptools import find_packages
    pk = find_packages(where=root, include=["acctransformer", "acctransformer.*", "acctransformer_b200", "acctransformer_b200.*"])
    for want in ("acctransformer", "acctransformer.flash_attention.nn.layer", "acctransformer.triangle_attention",
                 "acctransformer_b200", "acctransformer_b200.infer", "acctransformer_b200.flash_attention.ops.flash_attention"):
        assert want in pk, want
    assert "libacct_b200.so" in src and "build_ext" in src
