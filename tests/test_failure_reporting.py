"""A bounded wait that runs out is reported to the host and leaves the GPU usable.

Every wait inside the kernels has a limit; a wait that runs out sets a status word instead of
hanging.  Nothing in a healthy run makes that happen, so the library carries a self-test kernel
whose only wait is on a barrier nothing arrives at.  The failure is made without faulting,
trapping or hanging anything: the kernel returns normally after about a thousand polls.
"""
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref as ref

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_once_and_the_next_call_is_clean():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ctypes as C

    from acctransformer_b200 import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.cuda.synchronize()
    _lib.device_status()                                      # clean to begin with
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.acct_selftest_wait_timeout(stream))
    with pytest.raises(_lib.AcctError, match="ACCT_ERR_DEVICE_TIMEOUT") as info:
        _lib.device_status()
    assert info.value.code == 8 and "code 3" in str(info.value)   # 3 = a hand-off wait
    _lib.device_status()                                      # reading the word cleared it

    # the context is intact: a forward + backward right after it is correct and reports nothing
    B, N, S, D = 1, 2, 300, 64
    g = torch.Generator(device="cpu").manual_seed(3)
    q, k, v, do = (torch.randn(B, N, S, D, generator=g).half() for _ in range(4))
    scale = 1.0 / math.sqrt(D)
    o, lse = ops.fa_forward(q.to(dev), k.to(dev), v.to(dev), causal=True, scale=scale)
    dq, dk, dv = ops.fa_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, do.to(dev), causal=True, scale=scale)
    torch.cuda.synchronize()
    _lib.device_status()
    o_ref, _ = ref.sa_fwd(q.numpy(), k.numpy(), v.numpy(), causal=True, scale=scale)
    assert float(np.max(np.abs(o.float().cpu().numpy() - o_ref))) <= 2e-3
    for got, want in zip((dq, dk, dv), ref.sa_grad(q.numpy(), k.numpy(), v.numpy(), do.numpy(), causal=True, scale=scale)):
        assert float(np.max(np.abs(got.float().cpu().numpy() - want)) / np.max(np.abs(want))) <= 1e-2
