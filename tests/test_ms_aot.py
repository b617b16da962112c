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


# ------------------------------------------------------------------------------------------ attribute slots, shapes
def test_attribute_slots_are_per_tuple_and_reused(lib):
    lib.acct_ms_fa_attrs_slot.argtypes = [C.c_int, C.c_int, C.c_float, C.c_float, C.c_int]
    lib.acct_ms_fa_attrs_slot.restype = C.c_int
    a = lib.acct_ms_fa_attrs_slot(4, 4, 0.9, 0.125, 0)
    b = lib.acct_ms_fa_attrs_slot(65536, 0, 1.0, 0.125, 1)
    assert a >= 0 and b >= 0 and a != b
    assert lib.acct_ms_fa_attrs_slot(4, 4, 0.9, 0.125, 0) == a        # the same tuple keeps its slot
    for k in (a, b):
        assert hasattr(lib, f"acct_ms_fa_fwd_s{k}") and hasattr(lib, f"acct_ms_fa_grad_s{k}")


def _slot_fn(lib, kind, k):
    fn = getattr(lib, f"acct_ms_fa_{kind}_s{k}")
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int64)),
                   C.POINTER(C.c_char_p), C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    return fn


def test_declared_optional_inputs_are_taken_by_position_and_checked_by_name(lib):
    """A primitive bound to a slot that declares its optional inputs (ACCT_MS_HAS_* bits) gets exactly those, in the
    reference's order attn_mask, dropout_mask, alibi_mask; shapes no longer decide what an input is.
    No call here may get as far as a kernel (the pointers are fake): every one carries a rowsum / dq of the wrong
    type, which is looked at right AFTER the optional inputs -- so ACCT_ERR_DTYPE means "the optional inputs were
    accepted" and ACCT_ERR_SHAPE "they were not"."""
    lib.acct_ms_fa_attrs_slot_ex.argtypes = [C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int]
    lib.acct_ms_fa_attrs_slot_ex.restype = C.c_int
    MASK, DROP, ALIBI = 1, 2, 4
    assert lib.acct_ms_fa_attrs_slot_ex(65536, 65536, 1.0, 1.0, 0, 8) == -1              # not a sum of the three bits
    plain = lib.acct_ms_fa_attrs_slot_ex(65536, 65536, 1.0, 0.25, 0, -1)
    only_alibi = lib.acct_ms_fa_attrs_slot_ex(65536, 65536, 1.0, 0.25, 0, ALIBI)
    mask_alibi = lib.acct_ms_fa_attrs_slot_ex(65536, 65536, 1.0, 0.25, 0, MASK | ALIBI)
    none = lib.acct_ms_fa_attrs_slot_ex(65536, 65536, 1.0, 0.25, 0, 0)
    assert len({plain, only_alibi, mask_alibi, none}) == 4 and min(plain, only_alibi, mask_alibi, none) >= 0
    assert lib.acct_ms_fa_attrs_slot_ex(65536, 65536, 1.0, 0.25, 0, ALIBI) == only_alibi  # the same tuple, the same slot
    ACCEPTED, REFUSED = ERR_DTYPE, ERR_SHAPE
    # decode-like shapes, S_q = 1: [B,N,1,S_k] is an alibi_mask where the slot says so ...
    q = ((2, 4, 1, 64), b"float16")
    k = ((2, 4, 384, 64), b"float16")
    bad_lse = ((2, 4, 1), b"float16")
    row16, row8 = ((2, 4, 1, 384), b"float16"), ((2, 4, 1, 384), b"uint8")
    fwd = lambda slot: _slot_fn(lib, "fwd", slot)
    assert aot_call(fwd(only_alibi), [q, k, k, row16, q, bad_lse]) == ACCEPTED
    assert aot_call(fwd(only_alibi), [q, k, k, row8, q, bad_lse]) == REFUSED             # an alibi has q's type
    assert aot_call(fwd(plain), [q, k, k, row8, q, bad_lse]) == ACCEPTED                 # by shape: a uint8 dropout mask
    # ... the count must match the declaration ...
    assert aot_call(fwd(only_alibi), [q, k, k, q, bad_lse]) == REFUSED                   # declared, not passed
    assert aot_call(fwd(none), [q, k, k, row16, q, bad_lse]) == REFUSED                  # passed, not declared
    assert aot_call(fwd(none), [q, k, k, q, bad_lse]) == ACCEPTED
    # ... and so must the order: attn_mask before alibi_mask
    q2, o2, bad_l2 = ((2, 4, 256, 64), b"float16"), ((2, 4, 256, 64), b"float16"), ((2, 4, 256), b"float16")
    m, al = ((2, 256, 384), b"float16"), ((2, 4, 1, 384), b"float16")
    assert aot_call(fwd(mask_alibi), [q2, k, k, m, al, o2, bad_l2]) == ACCEPTED
    assert aot_call(fwd(mask_alibi), [q2, k, k, al, m, o2, bad_l2]) == REFUSED
    assert aot_call(fwd(plain), [q2, k, k, al, m, o2, bad_l2]) == ACCEPTED               # by shape: any order
    # the grad primitive reads the same declaration (dq of the wrong type stops the accepted calls)
    g32 = lambda shp: (shp, b"float32")
    l2 = ((2, 4, 256), b"float32")
    outs = [((2, 4, 256, 64), b"float16"), g32((2, 4, 384, 64)), g32((2, 4, 384, 64)), ((1 << 20,), b"uint8")]
    grad = _slot_fn(lib, "grad", only_alibi)
    assert aot_call(grad, [q2, k, k, o2, o2, l2, al] + outs) == ACCEPTED
    assert aot_call(grad, [q2, k, k, o2, o2, l2, m] + outs) == REFUSED                   # an attn_mask where an alibi is due
    from acctransformer_b200 import mindspore_adapter as ad
    assert ad.attrs_slot(65536, 65536, 1.0, 0.25, False, ad.HAS_ALIBI_MASK) == only_alibi
    with pytest.raises(ValueError):
        ad.attrs_slot(optional_inputs=9)


def test_mismatched_key_value_and_mask_shapes_are_rejected_before_any_read(lib):
    q = ((2, 4, 256, 64), b"float16")
    o, l = ((2, 4, 256, 64), b"float16"), ((2, 4, 256), b"float32")
    ok_k = ((2, 4, 384, 64), b"float16")
    # (the device pointers are fake: a call that got past the checks would reach the CUDA layer, never these tensors)
    bad = [
        [q, ((2, 4, 384, 32), b"float16"), ((2, 4, 384, 32), b"float16"), o, l],        # head_dim differs
        [q, ok_k, ((2, 4, 256, 64), b"float16"), o, l],                                   # v shaped unlike k
        [q, ((2, 3, 384, 64), b"float16"), ((2, 3, 384, 64), b"float16"), o, l],          # 3 heads do not divide 4
        [q, ((1, 4, 384, 64), b"float16"), ((1, 4, 384, 64), b"float16"), o, l],          # batch differs
        [q, ok_k, ((2, 4, 384, 64), b"bfloat16"), o, l],                                  # v of another type
        [q, ok_k, ok_k, ((2, 100, 384), b"float16"), o, l],                               # mask rows != S_q
        [q, ok_k, ok_k, ((3, 256, 384), b"float16"), o, l],                               # mask batch neither 1 nor B
        [q, ok_k, ok_k, ((2, 4, 256, 32), b"float16"), l],                                # output shaped unlike q
        [q, ok_k, ok_k, o, ((2, 4, 128), b"float32")],                                    # rowsum shaped unlike [B,N,S_q]
    ]
    for tensors in bad:
        assert aot_call(lib.acct_ms_fa_fwd, tensors) == ERR_SHAPE, tensors
    # grouped key/value heads are derived from k's own shape: dk and dv must then have k's shape
    kv2 = ((2, 2, 384, 64), b"float16")
    g32 = lambda shp: (shp, b"float32")
    grad = [q, kv2, kv2, o, o, l, g32((2, 4, 256, 64)), g32((2, 4, 384, 64)), g32((2, 4, 384, 64)), ((1024,), b"uint8")]
    assert aot_call(lib.acct_ms_fa_grad, grad) == ERR_SHAPE


def test_mindspore_adapter_shape_inference_and_strategy_tables():
    """The parts of the MindSpore adapter that are plain Python: output shapes and dtypes of the two primitives
    (flash_attention_impl.py:99-105,132-140) and the attributes the cell's shard() sets
    (nn/layer/flash_attention.py:132-177)."""
    from acctransformer_b200 import mindspore_adapter as ad
    assert ad.forward_out_shape((2, 8, 512, 128), (2, 8, 512, 128), (2, 8, 512, 128)) == ((2, 8, 512, 128), (2, 8, 512))
    assert ad.forward_out_dtype("float16", "float16", "float16") == ("float16", "float32")
    dq, dk, dv, ws = ad.grad_out_shape((2, 8, 512, 128), (2, 4, 640, 128), (2, 4, 640, 128), None, None, None)
    assert (dq, dk, dv) == ((2, 8, 512, 128), (2, 4, 640, 128), (2, 4, 640, 128))
    assert ws == (ad.bwd_workspace_bytes((2, 8, 512, 128)),) and ws[0] >= 2 * 8 * 512 * 4
    assert ad.grad_out_dtype(*["float16"] * 6) == ("float32", "float32", "float32", "uint8")
    s = ad.attrs_slot(4, 4, 0.9, 0.125, False)
    assert ad.attrs_slot(4, 4, 0.9, 0.125, False) == s
    assert ad.aot_func("fwd", s).endswith(f"libacct_b200.so:acct_ms_fa_fwd_s{s}")
    assert ad.aot_func("grad", s).endswith(f":acct_ms_fa_grad_s{s}")
    at = ad.shard_attrs(((2, 4, 1, 1), (2, 4, 1, 1), (2, 4, 1, 1)), have_attention_mask_batch=True, enable_dropout=True)
    assert at["dev_matrix_shape"] == [2, 4, 1, 1]
    assert at["inputs_tensor_map"] == [[3, 2, 1, 0]] * 3 + [[3, 1, 0], [3, 2, 1, 0]]
    assert at["outputs_tensor_map"] == [[3, 2, 1, 0], [3, 2, 1]] and at["empty_mirror_ops"] == 1
    at = ad.shard_attrs(None, have_attention_mask_batch=False, alibi=True, enable_dropout=True)
    assert at["inputs_tensor_map"][3] == [-1, 1, 0] and at["empty_mirror_ops"] == 0 and at["dev_matrix_shape"] == [1, 1, 1, 1]
    try:
        import mindspore  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError):
            ad.get_flash_attention()


@pytest.mark.gpu
def test_two_primitives_with_different_attributes_in_one_process():
    """Two layers of one graph with different band widths and scales: each is bound to its own attribute slot and
    keeps its own values, as primitives of the reference do (flash_attention_impl.py:146-152)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import mindspore_adapter as ad
    lb = _lib.load()
    sig = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int64)), C.POINTER(C.c_char_p),
           C.c_void_p, C.c_void_p]
    dev = torch.device("cuda", 0)
    B, N, S, D = 1, 2, 512, 64
    rs = np.random.RandomState(12)
    q, k, v = (torch.tensor(rs.randn(B, N, S, D).astype(np.float32)).half().to(dev) for _ in range(3))
    layers = [dict(prev_block_num=1, next_block_num=0, scale=0.125, causal=True),
              dict(prev_block_num=65536, next_block_num=65536, scale=0.05, causal=False)]
    slots = [ad.attrs_slot(keep_prob=1.0, **kw) for kw in layers]
    assert slots[0] != slots[1]
    outs = []
    stream = torch.cuda.current_stream().cuda_stream
    for slot in slots + slots[:1]:          # interleaved: the first layer again after the second
        fn = getattr(lb, f"acct_ms_fa_fwd_s{slot}")
        fn.argtypes, fn.restype = sig, C.c_int
        o = torch.empty_like(q)
        lse = torch.empty(B, N, S, dtype=torch.float32, device=dev)
        assert aot_call(fn, [q, k, v, o, lse], stream) == 0
        outs.append(o)
    torch.cuda.synchronize()
    _lib.device_status()
    for o, kw in zip(outs, layers + layers[:1]):
        o_ref, _ = ref.sa_fwd(_np(q), _np(k), _np(v), scale=kw["scale"], causal=kw["causal"],
                              prev_block_num=kw["prev_block_num"], next_block_num=kw["next_block_num"])
        assert np.max(np.abs(_np(o) - o_ref)) <= 2e-3
    assert torch.equal(outs[0], outs[2]) and not torch.equal(outs[0], outs[1])


@pytest.mark.gpu
def test_one_query_row_with_a_declared_alibi_mask():
    """S_q = 1: by shape alone [B,N,1,S_k] would be taken for a dropout mask; a slot that declares the input as the
    alibi_mask gets the bias added (against the CPU oracle), through the forward and the grad primitive."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import mindspore_adapter as ad
    lb = _lib.load()
    sig = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int64)), C.POINTER(C.c_char_p),
           C.c_void_p, C.c_void_p]
    dev = torch.device("cuda", 0)
    B, N, S_k, D = 2, 4, 384, 64
    rs = np.random.RandomState(13)
    q, do = (torch.tensor(rs.randn(B, N, 1, D).astype(np.float32)).half().to(dev) for _ in range(2))
    k, v = (torch.tensor(rs.randn(B, N, S_k, D).astype(np.float32)).half().to(dev) for _ in range(2))
    alibi_np = np.ascontiguousarray(ref.alibi_bias(B, N, S_k))                           # [B,N,1,S_k] fp16
    alibi = torch.tensor(alibi_np).to(dev)
    slot = ad.attrs_slot(scale=0.125, optional_inputs=ad.HAS_ALIBI_MASK)
    stream = torch.cuda.current_stream().cuda_stream
    fwd, grad = getattr(lb, f"acct_ms_fa_fwd_s{slot}"), getattr(lb, f"acct_ms_fa_grad_s{slot}")
    fwd.argtypes, fwd.restype, grad.argtypes, grad.restype = sig, C.c_int, sig, C.c_int
    o = torch.empty_like(q)
    lse = torch.empty(B, N, 1, dtype=torch.float32, device=dev)
    assert aot_call(fwd, [q, k, v, alibi, o, lse], stream) == 0
    dq = torch.empty(B, N, 1, D, dtype=torch.float32, device=dev)
    dk, dv = (torch.empty(B, N, S_k, D, dtype=torch.float32, device=dev) for _ in range(2))
    ws = torch.empty(ad.bwd_workspace_bytes((B, N, 1, D)), dtype=torch.uint8, device=dev)
    assert aot_call(grad, [q, k, v, o, do, lse, alibi, dq, dk, dv, ws], stream) == 0
    torch.cuda.synchronize()
    _lib.device_status()
    o_ref, l_ref = ref.sa_fwd(_np(q), _np(k), _np(v), alibi=alibi_np, scale=0.125)
    assert np.max(np.abs(_np(o) - o_ref)) <= 2e-3 and np.max(np.abs(_np(lse) - l_ref)) <= 2e-3
    o_plain, _ = ref.sa_fwd(_np(q), _np(k), _np(v), scale=0.125)
    assert np.max(np.abs(o_ref - o_plain)) > 2e-2                   # (the bias matters at these sizes)
    for got, want in zip((dq, dk, dv), ref.sa_grad(_np(q), _np(k), _np(v), _np(do), alibi=alibi_np, scale=0.125)):
        assert np.max(np.abs(_np(got) - want)) <= 1e-2 * np.max(np.abs(want))
