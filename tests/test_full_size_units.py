"""The benchmark configurations at their REAL batch and head counts, checked unit by unit.

The CPU oracle is O(S^2) per (batch, head) unit, so the other parity tests cut the batch and head
counts down.  That leaves the index arithmetic that depends on the unit number (rows of the
dropout mask and of the alibi tensor, the batch entry of the attention mask, the key/value head
of a cache) exercised only at small unit counts.  Here every configuration is drawn by
``workloads.make_inputs`` at full B and N on the device, the product path runs once over all of
it, and the FIRST and the LAST unit are compared with the oracle: O, L, dQ, dK, dV (decode: the
first and last sequence of the first and last head).

Tolerances as everywhere: max|O - O_ref| <= 2e-3 (bf16 outputs: 8e-3), max|L - L_ref| <= 2e-3,
max|g - g_ref| / max|g_ref| <= 1e-2.
"""
import numpy as np
import pytest
import torch

from oracle import attention_ref as ref

pytestmark = pytest.mark.gpu

O_TOL, BF16_O_TOL, G_TOL = 2e-3, 8e-3, 1e-2


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib
    _lib.load()
    return torch.device("cuda", 0)


def _np(t):
    return t.detach().float().cpu().numpy()


def _status():
    from acctransformer_b200 import _lib
    torch.cuda.synchronize()
    _lib.device_status()


def _first_and_last(B, N):
    return ((0, 0), (B - 1, N - 1))


def _check_unit(name, got, want, b, n, o_tol):
    o, lse, dq, dk, dv = got
    o_ref, l_ref, gq, gk, gv = want
    err = float(np.max(np.abs(_np(o[b, n]) - o_ref[0, 0])))
    assert err <= o_tol, f"{name} unit ({b},{n}): max|O - O_ref| = {err}"
    if lse is not None:
        err = float(np.max(np.abs(_np(lse[b, n]) - l_ref[0, 0])))
        assert err <= O_TOL, f"{name} unit ({b},{n}): max|L - L_ref| = {err}"
    for g, r, what in ((dq, gq, "dq"), (dk, gk, "dk"), (dv, gv, "dv")):
        if g is None:
            continue
        rel = float(np.max(np.abs(_np(g[b, n]) - r[0, 0])) / np.max(np.abs(r)))
        assert rel <= G_TOL, f"{name} unit ({b},{n}) {what}: relative error {rel}"


def _unit(t, b, n):
    """[1,1,S,D] NumPy view of one unit, in the 16-bit values the kernels saw."""
    return _np(t[b:b + 1, n:n + 1])


@pytest.mark.parametrize("form", ["tensor", "in_kernel"])
def test_config3_band_dropout_at_full_batch_and_heads(dev, form):
    from acctransformer_b200 import ops
    from acctransformer_b200.workloads import make_inputs
    inp = make_inputs("cfg3", dev, with_mask_tensors=(form == "tensor"))
    B, N = inp["B"], inp["N"]
    q, k, v, do, scale = inp["q"], inp["k"], inp["v"], inp["do"], inp["scale"]
    S = q.shape[2]
    kw = dict(prev_block_num=4, next_block_num=4, scale=scale, keep_prob=0.9)
    if form == "tensor":
        kw["dropout_mask"] = inp["dropout_mask"]
    else:
        kw.update(dropout_seed=1234, dropout_offset=9)
    o, lse = ops.fa_forward(q, k, v, **kw)
    dq, dk, dv = ops.fa_backward(q, k, v, o, lse, do, **kw)
    _status()
    for b, n in _first_and_last(B, N):
        if form == "tensor":
            dm = inp["dropout_mask"][b:b + 1, n:n + 1].cpu().numpy()
            keep = 0.9
        else:
            # the generator is a function of (unit number, query, key): the oracle's own restatement, for this unit
            dm = ref.dropout_mask_philox(B, N, S, S, 0.9, 1234, 9, units=[b * N + n])
            keep = ref.dropout_threshold(0.9) / 256.0
        okw = dict(drop_mask=dm, keep_prob=keep, prev_block_num=4, next_block_num=4, scale=scale)
        args = [_unit(t, b, n) for t in (q, k, v)]
        o_ref, l_ref = ref.sa_fwd(*args, **okw)
        gq, gk, gv = ref.sa_grad(*args, _unit(do, b, n), **okw)
        _check_unit("cfg3/" + form, (o, lse, dq, dk, dv), (o_ref, l_ref, gq, gk, gv), b, n, BF16_O_TOL)


def test_in_kernel_dropout_mask_of_the_last_unit_matches_the_oracle_generator(dev):
    """The mask tensor the library writes for (seed, offset) equals the oracle's Philox restatement on the last unit of
    a 64-unit problem (the unit number is a counter word of the generator)."""
    from acctransformer_b200 import ops
    B, N, S = 2, 32, 256
    m = ops.dropout_mask(B, N, S, S, 0.9, 1234, 9, device=dev)
    want = ref.dropout_mask_philox(B, N, S, S, 0.9, 1234, 9)
    assert np.array_equal(m[B - 1, N - 1].cpu().numpy(), want[B - 1, N - 1])
    assert np.array_equal(m[0, 0].cpu().numpy(), want[0, 0])


@pytest.mark.parametrize("mask_path", ["tensor+summary", "elided"])
def test_config4_triangle_attention_at_full_batch_and_heads(dev, mask_path):
    from acctransformer_b200 import TriangleAttention
    from acctransformer_b200.workloads import make_inputs
    inp = make_inputs("cfg4", dev)
    B, N = inp["B"], inp["N"]
    S, D = inp["q"].shape[2], inp["q"].shape[3]
    q = (inp["q"].float() * inp["scale"]).to(torch.float16)          # the caller pre-scales q
    k, v, do, mask = inp["k"], inp["v"], inp["do"], inp["attn_mask"]
    layer = TriangleAttention(block_size=512)
    layer.detect_causal_mask = (mask_path == "elided")
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = layer(qd, kd, vd, mask)
    o.backward(do)
    _status()
    for b, n in _first_and_last(B, N):
        args = [_unit(t, b, n) for t in (q, k, v)]
        m = _np(mask[b:b + 1])
        o_ref = ref.triangle_fwd(*args, m, block_size=512)
        gq, gk, gv = ref.sa_grad(*args, _unit(do, b, n), m)
        _check_unit("cfg4/" + mask_path, (o, None, qd.grad, kd.grad, vd.grad), (o_ref, None, gq, gk, gv), b, n, O_TOL)


def test_config2_alibi_rows_of_the_last_unit(dev):
    from acctransformer_b200 import ops
    from acctransformer_b200.workloads import make_inputs
    inp = make_inputs("cfg2", dev)
    B, N = inp["B"], inp["N"]
    q, k, v, do, scale, alibi = inp["q"], inp["k"], inp["v"], inp["do"], inp["scale"], inp["alibi"]
    kw = dict(causal=True, alibi=alibi, scale=scale)
    o, lse = ops.fa_forward(q, k, v, **kw)
    dq, dk, dv = ops.fa_backward(q, k, v, o, lse, do, **kw)
    _status()
    for b, n in _first_and_last(B, N):
        okw = dict(causal=True, alibi=_np(alibi[b:b + 1, n:n + 1]), scale=scale)
        args = [_unit(t, b, n) for t in (q, k, v)]
        o_ref, l_ref = ref.sa_fwd(*args, **okw)
        gq, gk, gv = ref.sa_grad(*args, _unit(do, b, n), **okw)
        _check_unit("cfg2", (o, lse, dq, dk, dv), (o_ref, l_ref, gq, gk, gv), b, n, O_TOL)


def test_config5_prefill_and_decode_at_full_batch_and_heads(dev):
    from acctransformer_b200 import flash_attention_decode, flash_attention_tik
    from acctransformer_b200.workloads import make_inputs
    inp = make_inputs("cfg5a", dev)
    B, N = inp["B"], inp["N"]
    q, k, v, scale = inp["q"], inp["k"], inp["v"], inp["scale"]
    y = flash_attention_tik(q, k, v, scale=scale, causal=True)
    _status()
    for b, n in _first_and_last(B, N):
        y_ref = ref.infer_fwd(*[_unit(t, b, n) for t in (q, k, v)], scale=scale, causal=True)
        err = float(np.max(np.abs(_np(y[b, n]) - y_ref[0, 0])))
        assert err <= O_TOL, f"prefill unit ({b},{n}): {err}"
    del q, k, v, y, inp
    torch.cuda.empty_cache()

    inp = make_inputs("cfg5b", dev)
    B, N = inp["B"], inp["N"]
    q, kc, vc, lens, scale = inp["q"], inp["k_cache"], inp["v_cache"], inp["seq_lens"], inp["scale"]
    y = flash_attention_decode(q, kc, vc, lens, scale=scale)
    _status()
    # sequences 0 and B-1 of heads 0 and N-1
    for b in (0, B - 1):
        for n in (0, N - 1):
            y_ref = ref.decode_ref(_unit(q, b, n), _unit(kc, b, n), _unit(vc, b, n), lens[b:b + 1].cpu().numpy(), scale)
            err = float(np.max(np.abs(_np(y[b, n]) - y_ref[0, 0])))
            assert err <= O_TOL, f"decode sequence {b} head {n}: {err}"


# ---------------------------------------------------------------------------------------------
# guard bands: nothing is written outside the outputs
# ---------------------------------------------------------------------------------------------
GUARD = 4096      # bytes on either side of every output


class _Guarded:
    """An output tensor carved out of a larger byte buffer with a pattern-filled band on both sides."""

    def __init__(self, shape, dtype, dev):
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        pad = (-n) % 256
        self.buf = torch.full((GUARD + n + pad + GUARD,), 0xA5, dtype=torch.uint8, device=dev)
        self.n, self.pad = n, pad
        self.t = self.buf[GUARD:GUARD + n].view(dtype).view(shape)

    def check(self, name):
        lo = self.buf[:GUARD]
        hi = self.buf[GUARD + self.n:]
        assert bool((lo == 0xA5).all()), f"{name}: bytes BEFORE the tensor were overwritten"
        assert bool((hi == 0xA5).all()), f"{name}: bytes AFTER the tensor were overwritten"


@pytest.mark.parametrize("grads_fp32", [False, True])
def test_ragged_outputs_stay_inside_their_guard_bands(dev, grads_fp32):
    """Ragged lengths and a head_dim that is not a tile width: the kernels work on 128-row tiles padded to 64 / 128
    columns, and every store (TMA store, TMA reduce-add, plain stores of the epilogues) has to clip."""
    import ctypes as C

    from acctransformer_b200 import _lib, ops
    lib = _lib.load()
    B, N, Sq, Sk, D = 2, 3, 333, 451, 80
    g = torch.Generator(device=dev).manual_seed(5)
    q, do = (torch.randn(B, N, Sq, D, device=dev, generator=g).half() for _ in range(2))
    k, v = (torch.randn(B, N, Sk, D, device=dev, generator=g).half() for _ in range(2))
    gdt = torch.float32 if grads_fp32 else torch.float16
    o, lse = _Guarded((B, N, Sq, D), torch.float16, dev), _Guarded((B, N, Sq), torch.float32, dev)
    dq, dk, dv = _Guarded((B, N, Sq, D), gdt, dev), _Guarded((B, N, Sk, D), gdt, dev), _Guarded((B, N, Sk, D), gdt, dev)
    a, keep = ops._fill_fa_args(q, k, v, o.t, lse.t, None, False, False, None, 1.0, None, None, 1, 2, 0.11, None,
                                flags=_lib.FLAG_GRAD_F32 if grads_fp32 else 0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.acct_fa_fwd(C.byref(a), stream))
    nbytes = lib.acct_fa_bwd_workspace_bytes(C.byref(a))
    ws = _Guarded((nbytes,), torch.uint8, dev)
    io = _lib.FaBwdIO()
    io.d_o, io.dq, io.dk, io.dv = do.data_ptr(), dq.t.data_ptr(), dk.t.data_ptr(), dv.t.data_ptr()
    io.workspace, io.workspace_bytes = ws.t.data_ptr(), nbytes
    _lib.check(lib.acct_fa_bwd(C.byref(a), C.byref(io), stream))
    _status()
    for name, t in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv), ("workspace", ws)):
        t.check(name)
    okw = dict(prev_block_num=1, next_block_num=2, scale=0.11)
    o_ref, l_ref = ref.sa_fwd(_np(q), _np(k), _np(v), **okw)
    assert float(np.max(np.abs(_np(o.t) - o_ref))) <= O_TOL
    for got, want in zip((dq, dk, dv), ref.sa_grad(_np(q), _np(k), _np(v), _np(do), **okw)):
        assert float(np.max(np.abs(_np(got.t) - want)) / np.max(np.abs(want))) <= G_TOL


def test_decode_output_stays_inside_its_guard_bands(dev):
    import ctypes as C

    from acctransformer_b200 import _lib
    lib = _lib.load()
    B, N, S, D = 3, 5, 777, 40
    g = torch.Generator(device=dev).manual_seed(6)
    q = torch.randn(B, N, 1, D, device=dev, generator=g).half()
    kc, vc = (torch.randn(B, N, S, D, device=dev, generator=g).half() for _ in range(2))
    lens = torch.tensor([1, 777, 300], dtype=torch.int32, device=dev)
    y = _Guarded((B, N, 1, D), torch.float16, dev)
    a = _lib.DecodeArgs()
    a.dtype = _lib.ACCT_F16
    a.B, a.N, a.S_max, a.D = B, N, S, D
    a.q, a.k_cache, a.v_cache, a.y = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), y.t.data_ptr()
    a.seq_lens = lens.data_ptr()
    a.scale = 0.2
    a.num_splits = 3
    ws = _Guarded((lib.acct_infer_decode_workspace_bytes(C.byref(a)),), torch.uint8, dev)
    a.workspace, a.workspace_bytes = ws.t.data_ptr(), ws.n
    _lib.check(lib.acct_infer_decode(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    _status()
    y.check("y")
    ws.check("workspace")
    want = ref.decode_ref(_np(q), _np(kc), _np(vc), lens.cpu().numpy(), 0.2)
    assert float(np.max(np.abs(_np(y.t) - want))) <= O_TOL


# ---------------------------------------------------------------------------------------------
# ordered dQ on sequences with more K/V tiles than the GPU has SMs
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("causal", [True, False])
def test_deterministic_backward_with_more_key_tiles_than_sms(dev, causal):
    """160 K/V tiles per (batch, head) slice: the CTA of a tile waits for the CTAs of the later tiles, so those must
    have been started first whatever the number of SMs.  Three runs are bit-equal, no wait runs out, and the result
    agrees with the unordered reduction.  The reference demands run-to-run equality of its gradients
    (tests/train/flash_attention/st/test_sharding.py:91-115) at the lengths it advertises (up to 128K tokens)."""
    from acctransformer_b200 import ops
    B, N, S, D = 1, 1, 160 * 128, 64
    g = torch.Generator(device=dev).manual_seed(11)
    q, k, v, do = (torch.randn(B, N, S, D, device=dev, generator=g).half() for _ in range(4))
    o, lse = ops.fa_forward(q, k, v, causal=causal, scale=0.125)
    runs = [ops.fa_backward(q, k, v, o, lse, do, causal=causal, scale=0.125, deterministic=True) for _ in range(3)]
    _status()
    for other in runs[1:]:
        for a, b_ in zip(runs[0], other):
            assert torch.equal(a, b_)
    loose = ops.fa_backward(q, k, v, o, lse, do, causal=causal, scale=0.125)
    _status()
    for a, b_ in zip(runs[0], loose):
        assert float((a.float() - b_.float()).abs().max()) <= 1e-2 * float(a.float().abs().max())
