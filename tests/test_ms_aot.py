"""The operators behind MindSpore's ops.Custom(func_type="aot") calling convention
(int f(nparam, params, ndims, shapes, dtypes, stream, extra)).  MindSpore itself is not needed: the tests make
the call the way its runtime does, with inputs followed by outputs.  CPU tests cover the argument unpacking (it
happens before any device work); the GPU tests compare the results with the CPU oracle."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from acctransformer_b200 import _lib, build as _build
from oracle import attention_ref as ref

ERR_SHAPE, ERR_DTYPE, ERR_WORKSPACE = 2, 3, 6
MS_NAMES = {torch.float16: b"float16", torch.bfloat16: b"bfloat16", torch.float32: b"float32", torch.uint8: b"uint8",
            torch.bool: b"bool"}


@pytest.fixture(scope="module")
def lib():
    _build.build()
    lb = _lib.load()
    for name in ("acct_ms_fa_fwd", "acct_ms_fa_grad", "acct_ms_infer_fa"):
        fn = getattr(lb, name)
        fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int64)),
                       C.POINTER(C.c_char_p), C.c_void_p, C.c_void_p]
        fn.restype = C.c_int
    lb.acct_ms_set_fa_attrs.argtypes = [C.c_int, C.c_int, C.c_float, C.c_float, C.c_int]
    lb.acct_ms_set_fa_attrs.restype = None
    return lb


def aot_call(fn, tensors, stream=None, fake_ptr=False):
    """Calls `fn` the way MindSpore's AOT custom-op runtime does; `tensors` = inputs then outputs.
    Entries are torch tensors or (shape, ms_dtype_name) pairs (for calls that must fail before touching memory)."""
    n = len(tensors)
    params = (C.c_void_p * n)()
    ndims = (C.c_int * n)()
    shapes = (C.POINTER(C.c_int64) * n)()
    dtypes = (C.c_char_p * n)()
    keep = []
    for i, t in enumerate(tensors):
        if isinstance(t, tuple):
            shape, name = t
            params[i] = 0x1000 * (i + 1)      # never dereferenced
        else:
            shape, name = tuple(t.shape), MS_NAMES[t.dtype]
            params[i] = t.data_ptr()
        arr = (C.c_int64 * max(len(shape), 1))(*shape)
        keep.append(arr)
        ndims[i] = len(shape)
        shapes[i] = C.cast(arr, C.POINTER(C.c_int64))
        dtypes[i] = name
    return fn(n, params, ndims, shapes, dtypes, stream, None)


# ------------------------------------------------------------------------------------------ CPU: unpacking
def test_wrong_parameter_counts_and_ranks_are_rejected(lib):
    q = ((1, 2, 256, 64), b"float16")
    lse = ((1, 2, 256), b"float32")
    assert aot_call(lib.acct_ms_fa_fwd, [q, q, q, q]) == ERR_SHAPE                       # too few
    assert aot_call(lib.acct_ms_fa_fwd, [q] * 9) == ERR_SHAPE                            # too many
    assert aot_call(lib.acct_ms_fa_fwd, [((2, 256, 64), b"float16"), q, q, q, lse]) == ERR_SHAPE   # rank-3 query
    assert aot_call(lib.acct_ms_fa_fwd, [((1, 2, 256, 64), b"float32"), q, q, q, lse]) == ERR_SHAPE  # fp32 query
    assert aot_call(lib.acct_ms_fa_fwd, [q, q, q, q, ((1, 2, 256), b"float16")]) == ERR_DTYPE        # fp16 rowsum
    # an optional input whose shape fits none of attn_mask / dropout_mask / alibi_mask
    assert aot_call(lib.acct_ms_fa_fwd, [q, q, q, ((1, 2, 7, 9), b"float16"), q, lse]) == ERR_SHAPE
    # two attention masks
    m = ((1, 256, 256), b"float16")
    assert aot_call(lib.acct_ms_fa_fwd, [q, q, q, m, m, q, lse]) == ERR_SHAPE


def test_grad_requires_fp32_outputs_and_a_workspace_tensor(lib):
    q = ((1, 2, 256, 64), b"float16")
    lse = ((1, 2, 256), b"float32")
    g32 = ((1, 2, 256, 64), b"float32")
    ws = ((4096,), b"uint8")
    assert aot_call(lib.acct_ms_fa_grad, [q, q, q, q, q, lse, g32, g32, g32]) == ERR_SHAPE          # no workspace
    assert aot_call(lib.acct_ms_fa_grad, [q, q, q, q, q, lse, q, g32, g32, ws]) == ERR_DTYPE        # fp16 dq
    assert aot_call(lib.acct_ms_fa_grad, [q, q, q, q, q, lse, g32, g32, g32, g32]) == ERR_WORKSPACE  # rank-4 "workspace"
    # too small a workspace is caught by the library proper (before any device work)
    assert aot_call(lib.acct_ms_fa_grad, [q, q, q, q, q, lse, g32, g32, g32, ((16,), b"uint8")]) == ERR_WORKSPACE


def test_infer_shape_checks_follow_the_reference(lib):
    # flash_attention_tik.cpp:163-185: rank 3 or 4, q/k/v agree on batch*heads and head_dim, k and v same shape
    q3, k3 = ((8, 128, 64), b"float16"), ((8, 256, 64), b"float16")
    assert aot_call(lib.acct_ms_infer_fa, [q3, k3, ((8, 128, 64), b"float16"), q3]) == ERR_SHAPE     # k/v lengths differ
    assert aot_call(lib.acct_ms_infer_fa, [q3, ((4, 256, 64), b"float16"), k3, q3]) == ERR_SHAPE     # heads differ
    assert aot_call(lib.acct_ms_infer_fa, [q3, ((8, 256, 32), b"float16"), k3, q3]) == ERR_SHAPE     # head_dim differs
    assert aot_call(lib.acct_ms_infer_fa, [((128, 64), b"float16")] * 4) == ERR_SHAPE                # rank 2
    assert aot_call(lib.acct_ms_infer_fa, [((8, 128, 64), b"float32"), k3, k3, q3]) == ERR_DTYPE


# ------------------------------------------------------------------------------------------ GPU: parity
def _np(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.gpu
def test_forward_and_grad_through_the_aot_convention():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    _build.build()
    lb = _lib.load()
    for name in ("acct_ms_fa_fwd", "acct_ms_fa_grad", "acct_ms_infer_fa"):
        fn = getattr(lb, name)
        fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int64)),
                       C.POINTER(C.c_char_p), C.c_void_p, C.c_void_p]
        fn.restype = C.c_int
    lb.acct_ms_set_fa_attrs.argtypes = [C.c_int, C.c_int, C.c_float, C.c_float, C.c_int]
    lb.acct_ms_set_fa_attrs.restype = None
    dev = torch.device("cuda", 0)
    B, N, S, D = 2, 3, 384, 64
    rs = np.random.RandomState(11)
    q, k, v, do = (torch.tensor(rs.randn(B, N, S, D).astype(np.float32)).half().to(dev) for _ in range(4))
    mask = torch.triu(torch.ones(S, S), 1).half().expand(B, S, S).contiguous().to(dev)   # 1 = masked
    alibi_np = np.ascontiguousarray(ref.alibi_bias(B, N, S))                             # [B,N,1,S] fp16
    alibi = torch.tensor(alibi_np).to(dev)
    scale = 1.0 / math.sqrt(D)
    lb.acct_ms_set_fa_attrs(65536, 65536, 1.0, scale, 0)
    try:
        o = torch.empty_like(q)
        lse = torch.empty(B, N, S, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        assert aot_call(lb.acct_ms_fa_fwd, [q, k, v, mask, alibi, o, lse], stream) == 0
        o_ref, lse_ref = ref.sa_fwd(_np(q), _np(k), _np(v), attn_mask=_np(mask), alibi=alibi_np.astype(np.float32),
                                    scale=scale)
        assert np.max(np.abs(_np(o) - o_ref)) <= 2e-3
        assert np.max(np.abs(_np(lse) - lse_ref)) <= 2e-3

        dq, dk, dv = (torch.empty(B, N, S, D, dtype=torch.float32, device=dev) for _ in range(3))
        ws_bytes = B * N * S * 4 * 2 + B * N * S * D * 4 + 4096 * 4     # generous upper bound: row sums, counters, dQ
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        assert aot_call(lb.acct_ms_fa_grad, [q, k, v, o, do, lse, mask, alibi, dq, dk, dv, ws], stream) == 0
        torch.cuda.synchronize()
        _lib.device_status()
        g_ref = ref.sa_grad(_np(q), _np(k), _np(v), _np(do), attn_mask=_np(mask), alibi=alibi_np.astype(np.float32),
                            scale=scale)
        for got, want, name in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
            err = np.max(np.abs(_np(got) - want)) / np.max(np.abs(want))
            assert err <= 1e-2, (name, err)
    finally:
        lb.acct_ms_set_fa_attrs(65536, 65536, 1.0, 1.0, 0)

    # inference op, rank 3, as the reference registers it (no scale, no mask)
    q3 = (torch.tensor(rs.randn(4, 256, 64).astype(np.float32)) * 0.3).half().to(dev)
    k3 = (torch.tensor(rs.randn(4, 384, 64).astype(np.float32)) * 0.3).half().to(dev)
    v3 = torch.tensor(rs.randn(4, 384, 64).astype(np.float32)).half().to(dev)
    y3 = torch.empty_like(q3)
    assert aot_call(lb.acct_ms_infer_fa, [q3, k3, v3, y3], torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    y_ref = ref.infer_fwd(_np(q3), _np(k3), _np(v3))
    assert np.max(np.abs(_np(y3) - y_ref)) <= 2e-3
