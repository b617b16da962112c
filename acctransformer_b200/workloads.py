"""Synthetic workloads with the shapes, dtypes and value distributions of the benchmark configurations.

The reference measures on no dataset: its tests draw random tensors at run time
(tests/train/flash_attention/st/test_fa_grad_precision.py:24-27).  Everything here is seeded
synthetic data of the same kind.

FLOP convention: forward = 4 * B * N * S_q * S_k * D * f, backward = 2.5 * forward, where f is
the fraction of the score matrix that is required: 1 dense, 1/2 causal, in-band tiles / all tiles
for block-band sparsity.  Recomputation, masked-tile waste and softmax work are not counted.
"""
from __future__ import annotations

import math

import torch

CONFIGS = {
    # headline metric: causal FA2 fwd+bwd at S = 8K, D = 128
    "H": dict(kind="fa", dtype="float16", B=2, N=32, S=8192, D=128, std=1.0, causal=True, seed=0),
    # the headline kernel at a size small enough for a full ncu capture (tensors still exceed the 126 MB L2)
    "P": dict(kind="fa", dtype="float16", B=2, N=16, S=4096, D=128, std=1.0, causal=True, seed=9),
    "cfg1": dict(kind="fa", dtype="float16", B=1, N=2, S=256, D=64, std=1.0, mask="triu", seed=1, fwd_only=True),
    "cfg2": dict(kind="fa", dtype="float16", B=4, N=16, S=2048, D=128, std=1.0, causal=True, alibi=True, seed=2),
    "cfg3": dict(kind="fa", dtype="bfloat16", B=2, N=32, S=8192, D=128, std=0.5, prev=4, next=4, keep_prob=0.9,
                 seed=3),
    "cfg4": dict(kind="triangle", dtype="float16", B=8, N=32, S=4096, D=128, std=1.0, block_size=512, seed=4),
    "cfg5a": dict(kind="prefill", dtype="float16", B=8, N=32, S=4096, D=128, std=1.0, causal=True, seed=5),
    "cfg5b": dict(kind="decode", dtype="float16", B=32, N=32, S=16384, D=128, std=1.0, len_lo=1024, seed=6),
}


def torch_dtype(name):
    return {"float16": torch.float16, "bfloat16": torch.bfloat16}[name]


def band_fraction(s_q, s_k, prev, nxt, block=128):
    tq, tk = (s_q + block - 1) // block, (s_k + block - 1) // block
    cnt = 0
    for i in range(tq):
        lo = max(0, i - prev)
        hi = min(tk - 1, i + nxt)
        cnt += max(0, hi - lo + 1)
    return cnt / float(tq * tk)


def fwd_flops(cfg, B=None, N=None):
    B = cfg["B"] if B is None else B
    N = cfg["N"] if N is None else N
    S, D = cfg["S"], cfg["D"]
    f = 1.0
    if cfg.get("causal") or cfg.get("mask") == "triu" or cfg["kind"] == "triangle":
        f = 0.5
    if "prev" in cfg:
        f = band_fraction(S, S, cfg["prev"], cfg["next"])
    return 4.0 * B * N * S * S * D * f


def fwd_bwd_flops(cfg, B=None, N=None):
    return 3.5 * fwd_flops(cfg, B, N)


def alibi_slopes(n_heads):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / n_heads) for h in range(n_heads)], dtype=torch.float32)


def make_inputs(name, device, B=None, N=None, seed_offset=0, with_mask_tensors=True):
    """Draw the tensors of configuration ``name`` on ``device`` (values are drawn in fp32 and then
    cast).  ``B`` / ``N`` override the batch / head counts (used to take a sub-sample or a shard)."""
    cfg = dict(CONFIGS[name])
    B = cfg["B"] if B is None else B
    N = cfg["N"] if N is None else N
    S, D, dt = cfg["S"], cfg["D"], torch_dtype(cfg["dtype"])
    g = torch.Generator(device=device).manual_seed(cfg["seed"] * 1000 + seed_offset)
    out = {"cfg": cfg, "B": B, "N": N}

    def draw(*shape):
        return (torch.randn(*shape, device=device, generator=g, dtype=torch.float32) * cfg["std"]).to(dt)

    if cfg["kind"] == "decode":
        out["q"] = draw(B, N, 1, D)
        out["k_cache"] = draw(B, N, S, D)
        out["v_cache"] = draw(B, N, S, D)
        gl = torch.Generator(device="cpu").manual_seed(7 + seed_offset)
        out["seq_lens"] = torch.randint(cfg["len_lo"], S + 1, (B,), generator=gl, dtype=torch.int32).to(device)
        out["scale"] = 1.0 / math.sqrt(D)
        return out
    out["q"], out["k"], out["v"] = draw(B, N, S, D), draw(B, N, S, D), draw(B, N, S, D)
    if not cfg.get("fwd_only") and cfg["kind"] != "prefill":
        out["do"] = draw(B, N, S, D)
    out["scale"] = 1.0 / math.sqrt(D)
    if with_mask_tensors:
        if cfg.get("mask") == "triu":
            out["attn_mask"] = torch.triu(torch.ones(1, S, S, device=device, dtype=torch.float16), diagonal=1)
        if cfg["kind"] == "triangle":
            out["attn_mask"] = torch.triu(torch.ones(S, S, device=device, dtype=torch.float16), diagonal=1) \
                .unsqueeze(0).expand(B, S, S).contiguous()
        if cfg.get("alibi"):
            sl = alibi_slopes(cfg["N"])[:N].to(device)
            out["alibi"] = (sl.view(1, N, 1, 1) * torch.arange(S, device=device, dtype=torch.float32).view(1, 1, 1, S)) \
                .expand(B, N, 1, S).to(dt).contiguous()
        if "keep_prob" in cfg:
            gm = torch.Generator(device=device).manual_seed(33 + seed_offset)
            m = torch.empty(B, N, S, S, device=device, dtype=torch.uint8)
            for b in range(B):         # drawn per batch entry to bound the fp32 temporary
                for h0 in range(0, N, 4):
                    h1 = min(N, h0 + 4)
                    m[b, h0:h1] = (torch.rand(h1 - h0, S, S, device=device, generator=gm) < cfg["keep_prob"]).to(torch.uint8)
            out["dropout_mask"] = m
    return out
