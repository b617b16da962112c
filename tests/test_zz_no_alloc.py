"""The allocation-free decode entry point, acct_infer_decode_static, against the regular one.

Some callers cannot call cudaMalloc when they need a decode step (their memory pool is fixed at
start-up, or they sit inside a framework that forbids allocation mid-step), so the library also
offers the decode step with its split-KV scratch built in.  This test drives both entry points
through the C ABI on the same inputs, several times in a row with different inputs, so that whatever
one call left in the shared scratch is shown not to leak into the next; the results must be
bit-identical between the two entry points and within tolerance of the CPU oracle.  It lives in its own
file, collected last, so a run that stops at the first failure has already run everything else.
"""
import ctypes as C
import math

import pytest
import torch

from oracle import attention_ref as ref

pytestmark = pytest.mark.gpu

TOL = 2e-3      # the decode tolerance used by the other GPU tests (max-abs on y), here against the CPU oracle


def _args(lib_mod, q, kc, vc, lens, y, scale, splits, ws=None):
    a = lib_mod.DecodeArgs()
    a.dtype = lib_mod.ACCT_BF16 if q.dtype == torch.bfloat16 else lib_mod.ACCT_F16
    a.B, a.N, a.S_max, a.D = q.shape[0], q.shape[1], kc.shape[2], q.shape[3]
    a.N_kv = kc.shape[1]
    a.q, a.k_cache, a.v_cache, a.y = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), y.data_ptr()
    a.seq_lens = lens.data_ptr()
    a.scale = scale
    a.num_splits = splits
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


def test_static_scratch_decode_matches_regular_decode_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, N, S, D = 4, 8, 4096, 128
    scale = 1.0 / math.sqrt(D)
    # second and third call: other inputs, another split count, then grouped key/value heads in bf16
    for call, (seed, splits, n_kv, dt) in enumerate(((1, 0, N, torch.float16), (2, 5, N, torch.float16),
                                                      (3, 3, N // 4, torch.bfloat16))):
        g = torch.Generator(device=dev).manual_seed(seed)
        q = torch.randn(B, N, 1, D, device=dev, generator=g).to(dt)
        kc = torch.randn(B, n_kv, S, D, device=dev, generator=g).to(dt)
        vc = torch.randn(B, n_kv, S, D, device=dev, generator=g).to(dt)
        lens = torch.randint(1, S + 1, (B,), device=dev, generator=g, dtype=torch.int32)
        y_ref = torch.zeros_like(q)
        y_new = torch.zeros_like(q)
        probe = _args(_lib, q, kc, vc, lens, y_ref, scale, splits)
        ws = torch.empty(lib.acct_infer_decode_workspace_bytes(C.byref(probe)), dtype=torch.uint8, device=dev)
        _lib.check(lib.acct_infer_decode(C.byref(_args(_lib, q, kc, vc, lens, y_ref, scale, splits, ws)), stream))
        # no workspace is passed to the static variant
        _lib.check(lib.acct_infer_decode_static(C.byref(_args(_lib, q, kc, vc, lens, y_new, scale, splits)), stream))
        torch.cuda.synchronize()
        _lib.device_status()
        # the two entry points run the same kernels with the same split count: the results are the same bits
        assert torch.equal(y_new, y_ref), f"call {call}: static-scratch decode differs from the regular decode"
        assert float(y_ref.float().abs().max()) > 0.0
        # and both agree with the CPU oracle (key/value heads repeated for the grouped case, as the reference prescribes)
        rep = N // n_kv
        want = ref.decode_ref(q.float().cpu().numpy(), kc.float().cpu().numpy().repeat(rep, axis=1),
                              vc.float().cpu().numpy().repeat(rep, axis=1), lens.cpu().numpy(), scale)
        err = float((y_new.float().cpu() - torch.tensor(want)).abs().max())
        assert err <= (TOL if dt == torch.float16 else 4 * TOL), f"call {call}: max|y_static - y_oracle| = {err}"


def test_static_scratch_decode_refuses_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, N, S, D, splits = 32, 32, 256, 128, 64          # 32*32*64*130*4 bytes = 34 MB > 8 MiB
    q = torch.zeros(B, N, 1, D, device=dev, dtype=torch.float16)
    kc = torch.zeros(B, N, S, D, device=dev, dtype=torch.float16)
    lens = torch.full((B,), S, device=dev, dtype=torch.int32)
    y = torch.zeros_like(q)
    rc = lib.acct_infer_decode_static(C.byref(_args(_lib, q, kc, kc, lens, y, 0.1, splits)), None)
    assert rc == 6       # ACCT_ERR_WORKSPACE
    msg = lib.acct_last_error().decode()
    assert "built-in scratch" in msg and str(_lib.DECODE_STATIC_SCRATCH_BYTES) in msg


def test_static_scratch_decode_lowers_an_automatic_split_count_to_what_fits():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from acctransformer_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 4 096 (sequence, head) slices of up to 2 048 keys: the automatic choice would be 4 key ranges (17 MB of partial
    # results); the 8 MiB array holds 3, and the call must use 3 rather than fail
    B, N, S, D = 64, 64, 2048, 128
    assert B * N * 4 * (D + 2) * 4 > _lib.DECODE_STATIC_SCRATCH_BYTES >= B * N * 3 * (D + 2) * 4
    g = torch.Generator(device=dev).manual_seed(11)
    q = torch.randn(B, N, 1, D, device=dev, generator=g).to(torch.float16)
    kc = torch.randn(B, N, S, D, device=dev, generator=g, dtype=torch.float16)
    lens = torch.randint(1, S + 1, (B,), device=dev, generator=g, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    y_auto, y_three = torch.zeros_like(q), torch.zeros_like(q)
    _lib.check(lib.acct_infer_decode_static(C.byref(_args(_lib, q, kc, kc, lens, y_auto, scale, 0)), stream))
    probe = _args(_lib, q, kc, kc, lens, y_three, scale, 3)
    ws = torch.empty(lib.acct_infer_decode_workspace_bytes(C.byref(probe)), dtype=torch.uint8, device=dev)
    _lib.check(lib.acct_infer_decode(C.byref(_args(_lib, q, kc, kc, lens, y_three, scale, 3, ws)), stream))
    torch.cuda.synchronize()
    _lib.device_status()
    assert torch.equal(y_auto, y_three)
    for b in (0, B - 1):           # first and last sequence against the CPU oracle
        want = ref.decode_ref(q[b:b + 1].float().cpu().numpy(), kc[b:b + 1].float().cpu().numpy(),
                              kc[b:b + 1].float().cpu().numpy(), lens[b:b + 1].cpu().numpy(), scale)
        assert float((y_auto[b:b + 1].float().cpu() - torch.tensor(want)).abs().max()) <= TOL
