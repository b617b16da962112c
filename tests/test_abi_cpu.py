"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares,
the ctypes mirrors match the C struct layout, and argument validation returns the documented codes
(validation happens before any device work, so no GPU is needed)."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

from acctransformer_b200 import _lib, build as _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "acct_b200.h")


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return _lib.load()


def test_library_exports_every_declared_symbol(lib):
    with open(HEADER) as f:
        text = f.read()
    declared = re.findall(r"ACCT_API\s+[\w\s\*]+?\b(acct_\w+)\s*\(", text)
    # the numbered MindSpore entry points are declared through a macro, one pair per slot
    slots = [int(k) for k in re.findall(r"ACCT_MS_SLOT_ENTRY\((\d+)\)", text)]
    assert slots == list(range(32))
    declared = [d for d in declared if "##" not in d and not d.endswith("_s")]
    declared += [f"acct_ms_fa_{kind}_s{k}" for k in slots for kind in ("fwd", "grad")]
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(set(declared)) == sorted(set(_lib.EXPORTS) | (set(declared) - set(_lib.EXPORTS)))
    assert set(_lib.EXPORTS) <= set(declared)
    assert lib.acct_abi_version() == 3


def test_ctypes_mirrors_match_c_layout(tmp_path):
    src = tmp_path / "layout.c"
    fields = {
        "acct_fa_args": ["dtype", "q", "lse", "q_stride", "o_stride", "mask_kind", "attn_mask", "dropout_mask",
                         "dropout_dtype", "keep_prob", "alibi", "alibi_slopes", "prev_block_num", "scale",
                         "seq_lens", "flags", "tri_block", "dropout_seed", "dropout_offset", "N_kv", "mask_tiles"],
        "acct_fa_bwd_io": ["d_o", "dq", "workspace", "workspace_bytes", "ev_kernel_start", "ev_kernel_stop"],
        "acct_infer_args": ["dtype", "rank", "D", "q", "y", "causal", "scale", "seq_lens", "N_kv"],
        "acct_decode_args": ["dtype", "D", "q", "kv_stride", "seq_lens", "y", "scale", "num_splits", "workspace",
                             "workspace_bytes", "N_kv", "block_table", "page_size", "max_pages"],
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', 'int main(void){']
    for st, fs in fields.items():
        lines.append(f'printf("{st} %zu\\n", sizeof({st}));')
        for f_ in fs:
            lines.append(f'printf("{st}.{f_} %zu\\n", offsetof({st}, {f_}));')
    lines.append('return 0;}')
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    mirrors = {"acct_fa_args": _lib.FaArgs, "acct_fa_bwd_io": _lib.FaBwdIO, "acct_infer_args": _lib.InferArgs,
               "acct_decode_args": _lib.DecodeArgs}
    for ln in out.strip().splitlines():
        key, val = ln.split()
        if "." in key:
            st, f_ = key.split(".")
            assert getattr(mirrors[st], f_).offset == int(val), key
        else:
            assert C.sizeof(mirrors[key]) == int(val), key


def _args(**kw):
    a = _lib.FaArgs()
    a.dtype = _lib.ACCT_F16
    a.B, a.N, a.S_q, a.S_k, a.D = 1, 1, 128, 128, 64
    a.q = a.k = a.v = a.o = 0x1000
    a.scale, a.keep_prob = 1.0, 1.0
    a.prev_block_num = a.next_block_num = _lib.BAND_UNBOUNDED
    for k, v in kw.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize("kw, code", [
    (dict(q=None), 1),                       # ACCT_ERR_NULL
    (dict(S_q=0), 2),                        # ACCT_ERR_SHAPE
    (dict(dtype=7), 3),                      # ACCT_ERR_DTYPE
    (dict(D=300), 4),                        # beyond the reference cell's 256 limit
    (dict(D=60), 4),                         # not a multiple of 8
    (dict(q=0x1008), 5),                     # ACCT_ERR_ALIGN
    (dict(scale=0.0), 2),
    (dict(mask_kind=1), 1),                  # full mask announced, pointer missing
    (dict(prev_block_num=-1), 2),
    (dict(tri_block=-5), 2),
    (dict(mask_tiles=0x5000), 2),            # a tile summary without a full mask tensor
])
def test_forward_validation_codes(lib, kw, code):
    a = _args(**kw)
    rc = lib.acct_fa_fwd(C.byref(a), None)
    assert rc == code, lib.acct_last_error()
    assert lib.acct_last_error() != b""


def test_head_dim_limit_is_the_reference_cells_for_forward_and_backward(lib):
    # forward, prefill and backward all take head_dim up to 256, the reference cell's limit
    # (nn/layer/flash_attention.py:26,105-106); above it, or not a multiple of 8, is refused
    a = _args(D=160, lse=0x2000)
    assert lib.acct_fa_fwd(C.byref(a), None) in (0, 9)          # passes validation; 9 = no sm_100 device on this machine
    g = _lib.FaBwdIO()
    g.d_o = g.dq = g.dk = g.dv = 0x3000
    g.workspace, g.workspace_bytes = 0x4000, 1 << 30
    assert lib.acct_fa_bwd(C.byref(a), C.byref(g), None) in (0, 9)
    for bad in (264, 100):
        a = _args(D=bad, lse=0x2000)
        assert lib.acct_fa_fwd(C.byref(a), None) == 4
        assert lib.acct_fa_bwd(C.byref(a), C.byref(g), None) == 4
    # two turn counters per Q tile above head_dim 128 (two CTAs share a K/V tile there)
    lo, hi = _args(D=128, S_q=128 * 1024), _args(D=136, S_q=128 * 1024)
    extra = lib.acct_fa_bwd_workspace_bytes(C.byref(hi)) - lib.acct_fa_bwd_workspace_bytes(C.byref(lo))
    assert extra == 128 * 1024 * 8 * 4 + 1024 * 4


def test_null_struct_pointers(lib):
    assert lib.acct_fa_fwd(None, None) == 1
    assert lib.acct_fa_bwd(None, None, None) == 1
    assert lib.acct_infer_prefill(None, None) == 1
    assert lib.acct_infer_decode(None, None) == 1
    assert lib.acct_fa_bwd_workspace_bytes(None) == 0
    assert lib.acct_infer_decode_workspace_bytes(None) == 0


def test_mask_tile_summary_size_and_argument_checks(lib):
    assert lib.acct_mask_tiles_bytes(2, 300, 1000) == 2 * 3 * 8        # one byte per 128x128 tile, edges rounded up
    assert lib.acct_mask_tiles_bytes(1, 128, 128) == 1
    assert lib.acct_mask_tiles_bytes(0, 128, 128) == 0
    assert lib.acct_mask_classify_tiles(None, _lib.ACCT_U8, 1, 128, 128, 0x1000, None) == 1
    assert lib.acct_mask_classify_tiles(0x1000, _lib.ACCT_U8, 1, 128, 128, None, None) == 1
    assert lib.acct_mask_classify_tiles(0x1000, 7, 1, 128, 128, 0x2000, None) == 3      # ACCT_ERR_DTYPE
    assert lib.acct_mask_classify_tiles(0x1000, _lib.ACCT_U8, 1, 0, 128, 0x2000, None) == 2


def test_backward_workspace_size_and_rejection(lib):
    a = _args(B=2, N=3, S_q=200, S_k=300, D=128, lse=0x2000)
    rows = 2 * 3 * 200
    q_tiles = 2 * 3 * 2          # ceil(200 / 128) Q tiles per (batch, head) slice
    need = ((rows * 4 + 255) // 256) * 256 + ((q_tiles * 4 + 255) // 256) * 256 + rows * 128 * 4
    assert lib.acct_fa_bwd_workspace_bytes(C.byref(a)) == need
    a.flags = _lib.FLAG_GRAD_F32      # fp32 gradients accumulate in dq itself: no accumulator in the workspace
    assert lib.acct_fa_bwd_workspace_bytes(C.byref(a)) == need - rows * 128 * 4
    a.flags = 0
    g = _lib.FaBwdIO()
    g.d_o = g.dq = g.dk = g.dv = 0x3000
    g.workspace, g.workspace_bytes = 0x4000, need - 1
    assert lib.acct_fa_bwd(C.byref(a), C.byref(g), None) == 6       # ACCT_ERR_WORKSPACE
    g.workspace, g.workspace_bytes = None, need
    assert lib.acct_fa_bwd(C.byref(a), C.byref(g), None) == 6


def test_infer_shape_checks_follow_the_reference_op(lib):
    a = _lib.InferArgs()
    a.dtype, a.rank, a.B, a.N, a.S_q, a.S_k, a.D = _lib.ACCT_F16, 5, 1, 1, 128, 128, 64
    a.q = a.k = a.v = a.y = 0x1000
    a.scale = 1.0
    assert lib.acct_infer_prefill(C.byref(a), None) == 2            # rank must be 3 or 4
    a.rank, a.B = 3, 2
    assert lib.acct_infer_prefill(C.byref(a), None) == 2            # rank 3 is [B*N,S,D]
    a.rank, a.B, a.y = 4, 1, None
    assert lib.acct_infer_prefill(C.byref(a), None) == 1


def test_decode_validation(lib):
    a = _lib.DecodeArgs()
    a.dtype, a.B, a.N, a.S_max, a.D = _lib.ACCT_F16, 2, 2, 1024, 128
    a.q = a.k_cache = a.v_cache = a.y = 0x1000
    a.scale = 0.1
    a.num_splits = 4
    assert lib.acct_infer_decode_workspace_bytes(C.byref(a)) == 2 * 2 * 4 * 130 * 4
    a.num_splits = 100
    assert lib.acct_infer_decode(C.byref(a), None) == 2
    a.num_splits, a.D = 4, 12
    assert lib.acct_infer_decode(C.byref(a), None) == 4


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libacct_b200.so")
    with pytest.raises(ImportError):
        _lib.load()


def test_a_plain_c_caller_can_bind_the_library(tmp_path, lib):
    """The boundary is a C ABI: a C99 program that includes the header, loads the library with dlopen and calls it
    gets the documented status codes (argument checks run before any device work, so no GPU is needed)."""
    src = tmp_path / "caller.c"
    src.write_text(r'''
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>
#include "acct_b200.h"
typedef int (*fwd_fn)(const acct_fa_args*, void*);
typedef int (*ver_fn)(void);
typedef const char* (*err_fn)(void);
typedef size_t (*ws_fn)(const acct_fa_args*);
int main(int argc, char** argv) {
  void* h = dlopen(argv[1], RTLD_NOW);
  if (!h) { printf("dlopen failed: %s\n", dlerror()); return 1; }
  ver_fn ver = (ver_fn)dlsym(h, "acct_abi_version");
  fwd_fn fwd = (fwd_fn)dlsym(h, "acct_fa_fwd");
  err_fn err = (err_fn)dlsym(h, "acct_last_error");
  ws_fn ws = (ws_fn)dlsym(h, "acct_fa_bwd_workspace_bytes");
  if (!ver || !fwd || !err || !ws) { printf("missing symbol\n"); return 2; }
  printf("version %d (header %d)\n", ver(), ACCT_ABI_VERSION);
  acct_fa_args a;
  memset(&a, 0, sizeof a);
  printf("null args -> %d\n", fwd(NULL, NULL));
  a.dtype = ACCT_F16; a.B = 1; a.N = 2; a.S_q = 256; a.S_k = 256; a.D = 60;   /* head_dim not a multiple of 8 */
  a.scale = 1.0f; a.keep_prob = 1.0f;
  printf("bad head_dim -> %d (%s)\n", fwd(&a, NULL), err());
  a.D = 64;
  printf("null tensors -> %d\n", fwd(&a, NULL));
  printf("workspace bytes %zu\n", ws(&a));
  return 0;
}
''')
    exe = tmp_path / "caller"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src),
                    "-ldl"], check=True)
    out = subprocess.run([str(exe), _lib.LIB_PATH], check=True, capture_output=True, text=True).stdout
    assert "version 3 (header 3)" in out
    assert "null args -> 1" in out                      # ACCT_ERR_NULL
    assert "bad head_dim -> 4" in out                   # ACCT_ERR_UNSUPPORTED_D
    assert "null tensors -> 1" in out
    ws_line = [ln for ln in out.splitlines() if ln.startswith("workspace bytes")][0]
    assert int(ws_line.split()[-1]) >= 1 * 2 * 256 * 64 * 4     # at least the fp32 dQ accumulator
