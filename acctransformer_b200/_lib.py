"""ctypes binding of ``libacct_b200.so`` (declared in ``include/acct_b200.h``).

This is the only place Python touches the C ABI.  There is no fallback: if the shared library
is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libacct_b200.so")

ACCT_F16, ACCT_BF16, ACCT_U8, ACCT_F32 = 0, 1, 2, 3
MASK_NONE, MASK_FULL, MASK_TILE128 = 0, 1, 2
BAND_UNBOUNDED = 65536
ABI_VERSION = 3       # ACCT_ABI_VERSION of include/acct_b200.h these mirrors were written for
FLAG_GRAD_F32, FLAG_DETERMINISTIC, FLAG_DROPOUT_PHILOX = 1, 2, 4
DECODE_STATIC_SCRATCH_BYTES = 8 * 1024 * 1024

ERR_NAMES = {
    1: "ACCT_ERR_NULL", 2: "ACCT_ERR_SHAPE", 3: "ACCT_ERR_DTYPE", 4: "ACCT_ERR_UNSUPPORTED_D",
    5: "ACCT_ERR_ALIGN", 6: "ACCT_ERR_WORKSPACE", 7: "ACCT_ERR_CUDA", 8: "ACCT_ERR_DEVICE_TIMEOUT",
    9: "ACCT_ERR_NO_DEVICE",
}

EXPORTS = [
    "acct_fa_fwd", "acct_fa_bwd_workspace_bytes", "acct_fa_bwd", "acct_infer_prefill",
    "acct_infer_decode_workspace_bytes", "acct_infer_decode", "acct_infer_decode_static", "acct_device_status",
    "acct_last_error", "acct_abi_version",
    "acct_ms_set_fa_attrs", "acct_ms_fa_fwd", "acct_ms_fa_grad", "acct_ms_infer_fa", "acct_dropout_mask",
    "acct_mask_is_causal", "acct_mask_tiles_bytes", "acct_mask_classify_tiles", "acct_mask_tiles_scratch",
    "acct_selftest_wait_timeout", "acct_ms_fa_attrs_slot", "acct_ms_fa_attrs_slot_ex",
] + [f"acct_ms_fa_{kind}_s{k}" for k in range(32) for kind in ("fwd", "grad")]


class AcctError(RuntimeError):
    """A non-zero return from the C ABI."""

    def __init__(self, code, message):
        super().__init__(f"{ERR_NAMES.get(code, code)}: {message}")
        self.code = code


class FaArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("N", C.c_int32), ("S_q", C.c_int32), ("S_k", C.c_int32),
        ("D", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("o_stride", C.c_int64 * 3),
        ("mask_kind", C.c_int32), ("mask_dtype", C.c_int32), ("mask_batch", C.c_int32), ("causal", C.c_int32),
        ("attn_mask", C.c_void_p), ("dropout_mask", C.c_void_p),
        ("dropout_dtype", C.c_int32), ("keep_prob", C.c_float),
        ("alibi", C.c_void_p), ("alibi_slopes", C.c_void_p),
        ("prev_block_num", C.c_int32), ("next_block_num", C.c_int32),
        ("scale", C.c_float),
        ("seq_lens", C.c_void_p),
        ("flags", C.c_uint32), ("tri_block", C.c_int32),
        ("dropout_seed", C.c_uint64), ("dropout_offset", C.c_uint64), ("N_kv", C.c_int32),
        ("mask_tiles", C.c_void_p),
    ]


class FaBwdIO(C.Structure):
    _fields_ = [
        ("d_o", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("ev_kernel_start", C.c_void_p), ("ev_kernel_stop", C.c_void_p),
    ]


class InferArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("rank", C.c_int32), ("B", C.c_int32), ("N", C.c_int32), ("S_q", C.c_int32),
        ("S_k", C.c_int32), ("D", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("y", C.c_void_p),
        ("causal", C.c_int32), ("scale", C.c_float), ("seq_lens", C.c_void_p), ("N_kv", C.c_int32),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("N", C.c_int32), ("S_max", C.c_int32), ("D", C.c_int32),
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("kv_stride", C.c_int64 * 3),
        ("seq_lens", C.c_void_p), ("y", C.c_void_p),
        ("scale", C.c_float), ("num_splits", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("N_kv", C.c_int32),
        ("block_table", C.c_void_p), ("page_size", C.c_int32), ("max_pages", C.c_int32),
    ]


_lib = None


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m acctransformer_b200.build` "
            "(needs nvcc); there is no fallback path")
    lib = C.CDLL(LIB_PATH)
    lib.acct_fa_fwd.argtypes = [C.POINTER(FaArgs), C.c_void_p]
    lib.acct_fa_fwd.restype = C.c_int
    lib.acct_fa_bwd_workspace_bytes.argtypes = [C.POINTER(FaArgs)]
    lib.acct_fa_bwd_workspace_bytes.restype = C.c_size_t
    lib.acct_fa_bwd.argtypes = [C.POINTER(FaArgs), C.POINTER(FaBwdIO), C.c_void_p]
    lib.acct_fa_bwd.restype = C.c_int
    lib.acct_infer_prefill.argtypes = [C.POINTER(InferArgs), C.c_void_p]
    lib.acct_infer_prefill.restype = C.c_int
    lib.acct_infer_decode_workspace_bytes.argtypes = [C.POINTER(DecodeArgs)]
    lib.acct_infer_decode_workspace_bytes.restype = C.c_size_t
    lib.acct_infer_decode.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
    lib.acct_infer_decode.restype = C.c_int
    lib.acct_infer_decode_static.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
    lib.acct_infer_decode_static.restype = C.c_int
    lib.acct_device_status.argtypes = [C.c_void_p]
    lib.acct_device_status.restype = C.c_int
    lib.acct_last_error.argtypes = []
    lib.acct_last_error.restype = C.c_char_p
    lib.acct_dropout_mask.argtypes = [C.POINTER(FaArgs), C.c_void_p, C.c_void_p]
    lib.acct_dropout_mask.restype = C.c_int
    lib.acct_mask_is_causal.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32),
                                        C.c_void_p]
    lib.acct_mask_is_causal.restype = C.c_int
    lib.acct_mask_tiles_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32]
    lib.acct_mask_tiles_bytes.restype = C.c_size_t
    lib.acct_mask_classify_tiles.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.acct_mask_classify_tiles.restype = C.c_int
    lib.acct_selftest_wait_timeout.argtypes = [C.c_void_p]
    lib.acct_selftest_wait_timeout.restype = C.c_int
    lib.acct_abi_version.argtypes = []
    lib.acct_abi_version.restype = C.c_int
    if lib.acct_abi_version() != ABI_VERSION:
        raise ImportError("libacct_b200.so was built from a different header version")
    _lib = lib
    return lib


def check(rc):
    if rc != 0:
        raise AcctError(rc, load().acct_last_error().decode("utf-8", "replace"))


def device_status(stream=0):
    """Raise if a kernel reported a bounded wait running out since the last call."""
    check(load().acct_device_status(C.c_void_p(stream)))
