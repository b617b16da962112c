"""Randomly drawn shapes and option combinations of the training and decode operators against the CPU oracle.

The hand-picked cases of the other GPU tests cover what the reference's own tests cover; this file draws sizes (1 .. 900
rows, every head_dim family incl. the wide backward), head groupings, dtypes and option mixes (causal, band, mask
tensor of either type, alibi, dropout tensor, valid lengths, ordered dQ) from fixed seeds, so that index arithmetic at
odd sizes is exercised in combinations nobody thought of.  Tolerances are the stated ones: max|O - O_ref| <= 2e-3 (fp16;
bf16 inputs 1.6e-2), gradients within 1e-2 (bf16 3e-2) of the tensor's largest magnitude."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref as ref

pytestmark = pytest.mark.gpu


def _np(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("seed", [101, 102, 103])
def test_training_operators_on_random_shapes(seed):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    rs = np.random.RandomState(seed)
    for case in range(25):
        D = int(rs.choice([40, 64, 80, 128, 128, 128, 160, 256]))
        B, G, Nkv = int(rs.randint(1, 4)), int(rs.choice([1, 1, 1, 2, 4])), int(rs.randint(1, 4))
        N = Nkv * G
        Sq, Sk = int(rs.randint(1, 900)), int(rs.randint(2, 900))
        if rs.rand() < 0.4:
            Sq = Sk
        dt = torch.bfloat16 if rs.rand() < 0.3 else torch.float16
        std = 0.5 if dt == torch.bfloat16 else 1.0
        draw = lambda *s: (torch.tensor(rs.randn(*s).astype(np.float32)) * std).to(dt)
        q, do, k, v = draw(B, N, Sq, D), draw(B, N, Sq, D), draw(B, Nkv, Sk, D), draw(B, Nkv, Sk, D)
        kw = dict(scale=float(rs.choice([1 / math.sqrt(D), 0.1])))
        mode = str(rs.choice(["plain", "causal", "band", "mask", "alibi", "drop", "lens", "ordered", "mix"]))
        mask = None
        if mode in ("causal", "ordered") and Sq <= Sk:
            kw["causal"] = True
        if mode in ("band", "mix"):
            kw["prev_block_num"], kw["next_block_num"] = int(rs.randint(0, 4)), int(rs.randint(0, 4))
            # rows that no K/V tile reaches are undefined in the oracle (and zeros here): keep every Q tile in the band
            if (Sq + 127) // 128 - 1 - kw["prev_block_num"] > (Sk + 127) // 128 - 1:
                kw.pop("prev_block_num")
        if mode in ("mask", "mix"):
            m = rs.random_sample((B if rs.rand() < 0.5 else 1, Sq, Sk)) < 0.3
            mask = torch.tensor(m.astype(np.float16)).to(dt if rs.rand() < 0.5 else torch.uint8)
        if mode in ("alibi", "mix"):
            kw["alibi"] = (torch.tensor(ref.alibi_bias(B, N, Sk, np.float32)) * 0.05).to(dt)
        if mode in ("drop", "mix"):
            kw["dropout_mask"] = torch.tensor((rs.random_sample((B, N, Sq, Sk)) < 0.8).astype(np.uint8))
            kw["keep_prob"] = 0.8
        if mode == "lens":
            kw["seq_lens"] = torch.tensor(rs.randint(2, Sk + 1, size=(B,)).astype(np.int32))
        if mode == "ordered":
            kw["deterministic"] = True
        what = (seed, case, mode, (B, N, Nkv, Sq, Sk, D), str(dt), {a: b for a, b in kw.items() if not torch.is_tensor(b)})
        on_dev = {a: (b.to(dev) if torch.is_tensor(b) else b) for a, b in kw.items()}
        fwd_kw = {a: b for a, b in on_dev.items() if a != "deterministic"}
        md = None if mask is None else mask.to(dev)
        o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev), md, **fwd_kw)
        dq, dk, dv = ops.fa_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, do.to(dev), md, **on_dev)
        torch.cuda.synchronize()
        _lib.device_status()
        okw = {}
        for a, b in kw.items():
            if a == "dropout_mask":
                okw["drop_mask"] = b.numpy()
            elif a in ("alibi", "seq_lens"):
                okw[a] = _np(b) if a == "alibi" else b.numpy()
            elif a != "deterministic":
                okw[a] = b
        if mask is not None:
            okw["attn_mask"] = _np(mask)
        kn, vn = np.repeat(_np(k), G, axis=1), np.repeat(_np(v), G, axis=1)     # the reference's own prescription
        with np.errstate(all="ignore"):
            o_ref, _ = ref.sa_fwd(_np(q), kn, vn, **okw)
            gq, gk, gv = ref.sa_grad(_np(q), kn, vn, _np(do), **okw)
        gk, gv = (g.reshape(B, Nkv, G, Sk, D).sum(2) for g in (gk, gv))
        defined = np.isfinite(o_ref).all(-1, keepdims=True)                     # (a row whose every key is masked by the band)
        tol_o, tol_g = (2e-3, 1e-2) if dt == torch.float16 else (1.6e-2, 3e-2)
        assert float(np.abs(np.where(defined, _np(o) - o_ref, 0.0)).max()) <= tol_o, what
        for got, want, name in ((dq, gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
            want = np.nan_to_num(want)
            assert float(np.abs(_np(got) - want).max()) <= tol_g * max(float(np.abs(want).max()), 1e-3), (name, what)


@pytest.mark.parametrize("seed", [201, 202])
def test_decode_on_random_shapes(seed):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    rs = np.random.RandomState(seed)
    for case in range(40):
        D = int(rs.choice([40, 64, 80, 128, 128, 128, 256]))
        G = int(rs.choice([1, 1, 2, 3, 4, 8, 16])) if D <= 128 else int(rs.choice([1, 2, 4, 8]))
        Nkv, B = int(rs.randint(1, 5)), int(rs.randint(1, 9))
        N = Nkv * G
        S = int(rs.choice([1, 17, 100, 511, 512, 513, 1500, 3000, 5000]))
        dt = torch.bfloat16 if rs.rand() < 0.3 else torch.float16
        splits = min(int(rs.choice([0, 0, 0, 1, 3, 7])), S)
        draw = lambda *s: torch.tensor(rs.randn(*s).astype(np.float32)).to(dt)
        q, kc, vc = draw(B, N, 1, D), draw(B, Nkv, S, D), draw(B, Nkv, S, D)
        lens = torch.tensor(rs.randint(1, S + 1, size=(B,)).astype(np.int32))
        scale = 1 / math.sqrt(D)
        paged = bool(rs.rand() < 0.35 and S >= 16)
        what = (seed, case, (B, N, Nkv, S, D), str(dt), splits, paged)
        if paged:       # the same caches cut into pages that lie in the pool in a random order
            ps = int(rs.choice([16, 64, 128]))
            mp = (S + ps - 1) // ps
            table = rs.permutation(B * mp + 3)[:B * mp].reshape(B, mp)
            pools = []
            for cache in (kc, vc):
                padded = torch.zeros(B, Nkv, mp * ps, D, dtype=dt)
                padded[:, :, :S] = cache
                pool = torch.zeros(B * mp + 3, Nkv, ps, D, dtype=dt)
                pool[torch.tensor(table.reshape(-1))] = padded.reshape(B, Nkv, mp, ps, D).permute(0, 2, 1, 3, 4).reshape(B * mp, Nkv, ps, D)
                pools.append(pool.to(dev))
            y = ops.infer_decode(q.to(dev), pools[0], pools[1], lens.to(dev), scale=scale, num_splits=splits,
                                 block_table=torch.tensor(table.astype(np.int32)).to(dev))
        else:
            y = ops.infer_decode(q.to(dev), kc.to(dev), vc.to(dev), lens.to(dev), scale=scale, num_splits=splits)
        torch.cuda.synchronize()
        _lib.device_status()
        want = ref.decode_ref(_np(q), np.repeat(_np(kc), G, axis=1), np.repeat(_np(vc), G, axis=1), lens.numpy(), scale)
        assert float(np.abs(_np(y) - want).max()) <= (2e-3 if dt == torch.float16 else 1.6e-2), what


@pytest.mark.parametrize("seed", [301])
def test_inference_op_on_random_shapes(seed):
    """FlashAttentionTik(q, k, v) at rank 3 and 4 (op_proto/flash_attention_tik.cpp:163-185), with the scale / causal /
    seq_lens additions drawn at random."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib, flash_attention_tik
    dev = torch.device("cuda", 0)
    rs = np.random.RandomState(seed)
    for case in range(30):
        D = int(rs.choice([40, 64, 80, 128, 128, 200, 256]))
        B, N = int(rs.randint(1, 4)), int(rs.randint(1, 5))
        Sq, Sk = int(rs.randint(1, 1200)), int(rs.randint(1, 1200))
        dt = torch.bfloat16 if rs.rand() < 0.3 else torch.float16
        causal = bool(rs.rand() < 0.4)
        if causal:
            Sk = max(Sk, Sq)                       # every query row then sees at least key 0
        scale = float(rs.choice([1.0 / math.sqrt(D), 0.05]))
        std = 0.5 if dt == torch.bfloat16 else 1.0
        draw = lambda *s: (torch.tensor(rs.randn(*s).astype(np.float32)) * std).to(dt)
        q, k, v = draw(B, N, Sq, D), draw(B, N, Sk, D), draw(B, N, Sk, D)
        lens = torch.tensor(rs.randint(1, Sk + 1, size=(B,)).astype(np.int32)) if rs.rand() < 0.3 and not causal else None
        rank3 = bool(rs.rand() < 0.4) and lens is None
        what = (seed, case, (B, N, Sq, Sk, D), str(dt), causal, scale, lens is not None, rank3)
        shape = (lambda t: t.reshape(B * N, t.shape[2], D)) if rank3 else (lambda t: t)
        y = flash_attention_tik(shape(q).to(dev), shape(k).to(dev), shape(v).to(dev), scale=scale, causal=causal,
                                seq_lens=None if lens is None else lens.to(dev))
        torch.cuda.synchronize()
        _lib.device_status()
        assert tuple(y.shape) == tuple(shape(q).shape) and y.dtype == dt, what
        want = ref.infer_fwd(_np(shape(q)), _np(shape(k)), _np(shape(v)), scale=scale, causal=causal,
                             seq_lens=None if lens is None else lens.numpy())
        assert float(np.abs(_np(y) - want).max()) <= (2e-3 if dt == torch.float16 else 1.6e-2), what


@pytest.mark.parametrize("seed", [401])
def test_cells_on_random_shapes_through_autograd(seed):
    """The two cells with the reference's constructors and call signatures (nn/layer/flash_attention.py:49-130,
    triangle_attention.py:28-165), random sizes, masks and band limits, gradients through torch autograd."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import FlashAttention, TriangleAttention, _lib
    dev = torch.device("cuda", 0)
    rs = np.random.RandomState(seed)
    draw = lambda *s: torch.tensor((rs.randn(*s) * 0.7).astype(np.float32)).half()

    def grads_match(leaves, want, what):
        for t, w, name in zip(leaves, want, ("dq", "dk", "dv")):
            assert float(np.abs(_np(t.grad) - w).max()) <= 1e-2 * float(np.abs(w).max()), (name, what)

    for case in range(12):
        # ---- FlashAttention: the cell scales by head_dim^-1/2 in all (two fp16 multiplies by d^-1/4 in the reference)
        D = int(rs.choice([40, 64, 80, 128, 160]))
        B, N, S = int(rs.randint(1, 3)), int(rs.randint(1, 4)), int(rs.randint(2, 700))
        with_batch = bool(rs.rand() < 0.5)
        prev, nxt = (int(rs.randint(1, 4)), int(rs.randint(0, 3))) if rs.rand() < 0.4 else (65536, 65536)
        use_alibi = bool(rs.rand() < 0.3)
        m = rs.random_sample((B if with_batch else 1, S, S)) < 0.25
        m[..., np.arange(S), np.arange(S)] = False          # the diagonal stays visible: no row without keys
        mask = torch.tensor(m.astype(np.float16))
        q, k, v, do = draw(B, N, S, D), draw(B, N, S, D), draw(B, N, S, D), draw(B, N, S, D)
        alibi = (torch.tensor(ref.alibi_bias(B, N, S, np.float32)) * 0.05).half() if use_alibi else None
        what = ("FlashAttention", seed, case, (B, N, S, D), with_batch, prev, nxt, use_alibi)
        cell = FlashAttention(head_dim=D, prev_block_num=prev, next_block_num=nxt, have_attention_mask_batch=with_batch,
                              alibi=use_alibi)
        leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
        o = cell(*leaves, mask.to(dev), None if alibi is None else alibi.to(dev))
        o.backward(do.to(dev))
        torch.cuda.synchronize()
        _lib.device_status()
        okw = dict(attn_mask=_np(mask), scale=1.0 / math.sqrt(D), alibi=None if alibi is None else _np(alibi),
                   prev_block_num=prev if prev < 65536 else None, next_block_num=nxt if nxt < 65536 else None)
        o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), **okw)
        assert float(np.abs(_np(o) - o_ref).max()) <= 2e-3, what
        grads_match(leaves, ref.sa_grad(_np(q), _np(k), _np(v), _np(do), **okw), what)

        # ---- TriangleAttention: no scaling inside, row groups of block_size, any mask
        D = int(rs.choice([64, 128]))
        S, block = int(rs.randint(2, 1400)), int(rs.choice([100, 128, 256, 300, 512]))
        m = rs.random_sample((B, S, S)) < 0.25
        m[..., 0] = False                                   # key 0 lies in every row group
        mask = torch.tensor(m.astype(np.float16))
        q, k, v, do = (draw(B, N, S, D) * 0.4 for _ in range(4))
        what = ("TriangleAttention", seed, case, (B, N, S, D), block)
        leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
        o = TriangleAttention(block_size=block)(*leaves, mask.to(dev))
        o.backward(do.to(dev))
        torch.cuda.synchronize()
        _lib.device_status()
        assert float(np.abs(_np(o) - ref.triangle_fwd(_np(q), _np(k), _np(v), _np(mask), block_size=block)).max()) <= 2e-3, what
        # keys past the end of a row's group do not exist for it: as a mask, for the gradient oracle
        rows = np.arange(S)
        beyond = np.arange(S)[None, :] >= ((rows // block + 1) * block)[:, None]
        grads_match(leaves, ref.sa_grad(_np(q), _np(k), _np(v), _np(do), np.maximum(_np(mask), beyond[None].astype(np.float32))), what)
