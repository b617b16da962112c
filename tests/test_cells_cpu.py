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
