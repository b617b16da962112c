"""Regenerates the golden fixtures in this folder from the reference checkout.

Run once, on a machine that has a checkout of the reference project, with ``--ref`` pointing at
it; the ``.npz`` files it writes are committed, so nothing at test time needs the reference.

What it runs, unmodified:

* ``np_impl_sa_fwd``, ``np_impl_sa_grad`` and ``data_compare`` from
  tests/train/flash_attention/st/common.py (lines 110-132, 147-175, 178-192).  That
  module imports MindSpore at the top, which is not installed, so the three function
  definitions are pulled out of the file's syntax tree and executed on their own; they
  are pure NumPy.
* tests/infer/flash_attention/tik/data_gen.py ``main(batch, heads, q_tokens, kv_tokens,
  embed)``, which seeds torch with 42 and writes query/key/value/golden ``.npy``.

Inputs for the training cases come from ``numpy.random.RandomState(seed)`` (a frozen
legacy generator), drawn as the reference tests draw them: uniform [0,1) for forward,
standard normal for gradients, cast to fp16.  Inputs are stored next to the outputs so
that a change in a random generator can never silently invalidate a fixture.
"""
import argparse
import ast
import os
import runpy
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_functions(ref_root):
    path = os.path.join(ref_root, "tests/train/flash_attention/st/common.py")
    with open(path, "r", encoding="utf-8") as f:
        tree = ast.parse(f.read())
    wanted = {"np_impl_sa_fwd", "np_impl_sa_grad", "data_compare"}
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in wanted]
    assert {n.name for n in body} == wanted
    ns = {"np": np}
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    return ns


def train_case(ns, seed, shape, mask_kind, dist):
    rs = np.random.RandomState(seed)
    b, n, s, d = shape
    draw = (lambda: rs.random_sample(shape)) if dist == "uniform" else (lambda: rs.randn(*shape))
    q = draw().astype(np.float16)
    k = draw().astype(np.float16)
    v = draw().astype(np.float16)
    do = rs.randn(*shape).astype(np.float16)
    mask = None
    if mask_kind == "triu":
        mask = np.triu(np.ones((1, s, s), dtype=np.float16), k=1)
    o, (e, p, row_sum, row_max) = ns["np_impl_sa_fwd"](q, k, v, mask)
    lse = np.squeeze(row_max.astype(np.float32) + np.log(row_sum), axis=-1)
    dq, dk, dv = ns["np_impl_sa_grad"](q, k, v, p, o, do)
    return dict(q=q, k=k, v=v, do=do, o=o, lse=lse, dq=dq, dk=dk, dv=dv,
                mask_kind=np.array(mask_kind), dist=np.array(dist), seed=np.array(seed))


def infer_case(ref_root, args5):
    script = os.path.join(ref_root, "tests/infer/flash_attention/tik/data_gen.py")
    mod = runpy.run_path(script, run_name="data_gen_ref")
    cwd = os.getcwd()
    with tempfile.TemporaryDirectory() as tmp:
        os.chdir(tmp)
        try:
            mod["main"](*args5)
            out = {name: np.load(name + ".npy") for name in ("query", "key", "value", "golden")}
        finally:
            os.chdir(cwd)
    out["args"] = np.array(args5)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the reference project's checkout")
    a = ap.parse_args()
    ns = load_reference_functions(a.ref)

    cases = {
        # benchmark configuration 1's shape, gradient-test distribution, full triu mask
        "fa_cfg1_randn_triu": (11, (1, 2, 256, 64), "triu", "randn"),
        # reference ST shape (1,1,128,80) with both distributions
        "fa_st_128x80_uniform_triu": (12, (1, 1, 128, 80), "triu", "uniform"),
        "fa_st_128x80_randn_triu": (13, (1, 1, 128, 80), "triu", "randn"),
        # unmasked (next_block_num = k_seq_len in the reference test)
        "fa_st_1x2x256x128_uniform_nomask": (14, (1, 2, 256, 128), "none", "uniform"),
    }
    for name, (seed, shape, mk, dist) in cases.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **train_case(ns, seed, shape, mk, dist))
        print("wrote", name)

    # data_compare known answers on a fixed perturbation
    rs = np.random.RandomState(5)
    gt = rs.randn(64, 64).astype(np.float32)
    pr = gt + rs.randn(64, 64).astype(np.float32) * 2e-3
    pr[3, 4] += 1.0
    res = [ns["data_compare"](gt, pr), ns["data_compare"](gt, gt),
           ns["data_compare"](gt, pr, 0.005, 0.005, 0.005)]
    np.savez_compressed(os.path.join(HERE, "data_compare_kat.npz"), gt=gt, pr=pr,
                        results=np.array([[r[0] == "Pass", r[1], r[2]] for r in res], dtype=np.float64))
    print("wrote data_compare_kat")

    for name, args5 in {"infer_1x2x256x384x64": (1, 2, 256, 384, 64),
                        "infer_1x1x512x512x40": (1, 1, 512, 512, 40)}.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **infer_case(a.ref, args5))
        print("wrote", name)


if __name__ == "__main__":
    sys.exit(main())
