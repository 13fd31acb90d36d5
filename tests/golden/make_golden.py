"""Generates tests/golden/golden.npz: known answers that pin the CPU oracle to the reference's own checking code.

Run in a container that has the reference checkout (it is imported, never copied):

    python tests/golden/make_golden.py /path/to/reference

For every case (seeded data from libcertex_b200.synthetic, so only answers are stored):
  * `ids`, `scores`  : the oracle's exact top-k (oracle/exact_knn.c);
  * `ref_best`       : the k smallest fp64 scores per query computed by the reference's test helper
                       `exact_k` (tests/test_exact.py:64-77), run on the CPU;
  * `ref_scores_ids` : the reference helper `scores` (tests/test_exact.py:49-61) applied to the oracle's ids;
  * `ref_verify`     : the value of the reference's `certex.verify` (certex/index.py:487-548) for the oracle's ids
                       (must be 1.0) and `ref_verify_bad` for ids with one neighbour replaced by a far vector (< 1).
The reference code runs unmodified; since this container has no GPU, `.cuda()` and `device="cuda"` are redirected to
the CPU while it runs. The reference helpers define inner-product scores as -<q,x> and cosine scores on normalised
vectors; the generator stores them as they come, the tests convert.
"""

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from libcertex_b200 import synthetic  # noqa: E402
from oracle import oracle  # noqa: E402

CASES = [
    # name, n, dim, nq, k, dtype, metric, unequal_norms, duplicates
    ("f32_l2", 3000, 32, 40, 10, "float32", "l2", False, 0),
    ("f32_ip", 3000, 32, 40, 10, "float32", "ip", True, 0),
    ("f32_cos", 3000, 32, 40, 10, "float32", "cosine", True, 0),
    ("f16_l2", 2000, 24, 30, 7, "float16", "l2", False, 0),
    ("u8_l2", 4000, 32, 40, 10, "uint8", "l2", False, 0),
    ("u8_l2_dups", 4000, 32, 40, 10, "uint8", "l2", False, 300),
    ("i8_l2", 4000, 32, 40, 10, "int8", "l2", False, 0),
    ("i8_ip", 4000, 32, 40, 10, "int8", "ip", False, 0),
    ("u8_l2_k100", 4000, 128, 20, 100, "uint8", "l2", False, 0),
]


def make_case(name, n, dim, nq, k, dtype, metric, unequal, dups, seed=7):
    x = synthetic.correlated(n, dim, seed=seed, dtype=dtype, unequal_norms=unequal)
    q = synthetic.correlated(nq, dim, seed=seed + 1, dtype=dtype)
    for c in range(1, min(dups, n - 1) + 1):
        x[c] = x[0]
    return x, q


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    # the reference checks run on "cuda"; redirect to the CPU for the duration of this script
    torch.Tensor.cuda = lambda self, *a, **kw: self
    for fn in ("full", "arange", "zeros", "empty", "as_tensor", "tensor"):
        orig = getattr(torch, fn)

        def wrap(*a, __orig=orig, **kw):
            if kw.get("device") == "cuda":
                kw["device"] = "cpu"
            return __orig(*a, **kw)

        setattr(torch, fn, wrap)
    import certex  # the reference package
    import test_exact as ref_tests  # the reference's test helpers

    ref_tests.DEV = "cpu"
    out = {}
    for case in CASES:
        name, n, dim, nq, k, dtype, metric = case[:7]
        x, q = make_case(*case)
        ids, sc = oracle.knn(x, q, k, metric)
        X, Q = torch.from_numpy(x.astype(np.float32) if dtype != "float16" else x), torch.from_numpy(
            q.astype(np.float32) if dtype != "float16" else q)
        ref_best = ref_tests.exact_k(X, Q, k, metric).numpy()
        ref_sc = torch.sort(ref_tests.scores(X, Q, torch.from_numpy(ids), metric), 1).values.numpy()
        v_ok = certex.verify(X, Q, torch.from_numpy(ids), metric=metric, sample=None)
        # a wrong answer: the last neighbour of every query replaced by the farthest vector of the oracle's full ranking
        far, _ = oracle.knn(x, q, n, metric)
        bad = ids.copy()
        bad[:, -1] = far[:, -1]
        v_bad = certex.verify(X, Q, torch.from_numpy(bad), metric=metric, sample=None)
        print(f"{name}: verify(oracle ids) = {v_ok}, verify(bad ids) = {v_bad}, "
              f"max |ref_best - sorted ref scores of oracle ids| = {np.abs(ref_best - ref_sc).max():.3e}")
        out[f"{name}/ids"] = ids
        out[f"{name}/scores"] = sc
        out[f"{name}/ref_best"] = ref_best
        out[f"{name}/ref_scores_ids"] = ref_sc
        out[f"{name}/ref_verify"] = np.float64(v_ok)
        out[f"{name}/ref_verify_bad"] = np.float64(v_bad)
        out[f"{name}/data_sha256"] = np.array(digest(x, q))
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
