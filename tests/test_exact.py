"""End-to-end parity on the GPU, through the C ABI: neighbour ids and fp64 scores must equal the CPU oracle's bit for
bit (integer and float inputs alike: the kernels round every product and sum as the sequential CPU loop does), ties
to the smaller id. The cases follow the reference's parameter table (cpp/tests/neighbors/ann_certex.cuh:277-319) and
its Python suite (tests/test_exact.py): three metrics, four element types, k in {1, 10, 100, 1024, 2048}, build +
extend shares, unequal norms, duplicates, tiny sets, many queries."""

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from libcertex_b200 import synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu

CASES = [
    # n, dim, nq, k, metric, dtype, build_share, unequal_norms, duplicates
    (30000, 96, 200, 10, "l2", "uint8", 1.0, False, 0),
    (30000, 96, 200, 10, "l2", "int8", 0.33, False, 0),
    (30000, 96, 200, 10, "ip", "int8", 1.0, True, 0),
    (30000, 96, 200, 10, "ip", "uint8", 0.5, True, 0),
    (30000, 96, 100, 100, "l2", "uint8", 1.0, False, 0),
    (30000, 96, 50, 1024, "l2", "uint8", 1.0, False, 0),
    (20000, 128, 200, 10, "l2", "uint8", 1.0, False, 500),
    (20000, 128, 200, 10, "l2", "int8", 1.0, False, 500),
    (25, 32, 50, 10, "l2", "uint8", 1.0, False, 0),
    (5000, 32, 3001, 10, "l2", "uint8", 1.0, False, 0),
    (60000, 200, 300, 10, "l2", "uint8", 1.0, False, 0),
    (40000, 500, 150, 5, "l2", "int8", 1.0, False, 0),
    (8000, 600, 40, 10, "l2", "uint8", 1.0, False, 0),
    (30000, 96, 200, 10, "l2", "float32", 1.0, False, 0),
    (30000, 96, 200, 10, "l2", "float32", 0.33, False, 0),
    (30000, 96, 200, 10, "ip", "float32", 1.0, True, 0),
    (30000, 96, 200, 10, "cosine", "float32", 0.5, True, 0),
    (30000, 96, 100, 100, "l2", "float16", 1.0, False, 0),
    (30000, 96, 20, 1024, "l2", "float32", 1.0, False, 0),
    (20000, 128, 100, 10, "l2", "float32", 1.0, False, 500),
    (20000, 128, 100, 10, "cosine", "float16", 1.0, True, 0),
    (25, 32, 50, 10, "l2", "float32", 1.0, False, 0),
    (3000, 33, 40, 2048, "ip", "float32", 1.0, True, 0),
    # more than 128 float dimensions / 256 bytes: code rows of several K blocks
    (30000, 200, 300, 10, "l2", "float32", 1.0, False, 0),
    (20000, 768, 150, 100, "cosine", "float32", 0.5, True, 0),
    (20000, 768, 50, 10, "ip", "float16", 1.0, True, 0),
    (12000, 2048, 20, 10, "l2", "float32", 1.0, False, 0),
    (20000, 1024, 200, 10, "l2", "uint8", 1.0, False, 0),
    (6000, 4096, 30, 10, "ip", "int8", 1.0, False, 0),
    (3000, 2100, 10, 10, "l2", "float32", 1.0, False, 0),
    # three quarters of the rows identical: thousands of equal group maxima and equal scores
    (20000, 64, 100, 10, "l2", "uint8", 1.0, False, 15000),
    (20000, 64, 100, 10, "ip", "float32", 1.0, True, 15000),
    (20000, 64, 60, 300, "l2", "int8", 1.0, False, 15000),
]


def make(n, dim, nq, dtype, unequal, dups, seed=42):
    x = synthetic.correlated(n, dim, seed=seed, dtype=dtype, unequal_norms=unequal)
    q = synthetic.correlated(nq, dim, seed=seed + 1, dtype=dtype)
    for c in range(1, min(dups, n - 1) + 1):
        x[c] = x[0]
    return x, q


def check(index, x, q, k, metric, **kw):
    D, I, S = index.search(torch.from_numpy(q).cuda(), k=k, return_scores=True, **kw)
    ids, scores = oracle.knn(x, q, k, metric)
    I, S, D = I.cpu().numpy(), S.cpu().numpy(), D.cpu().numpy().astype(np.float64)
    assert np.array_equal(I, ids), f"{(I != ids).any(1).sum()} of {len(ids)} queries differ"
    assert np.array_equal(S, scores)
    # returned values follow the reference's conventions: squared distance, inner product, cosine similarity
    xs, qs = x.astype(np.float64), q.astype(np.float64)
    if metric == "l2":
        want = scores
    elif metric == "ip":
        want = np.einsum("qd,qkd->qk", qs, xs[ids])
    else:
        want = 1 - scores / 2
    assert np.allclose(D, want, rtol=1e-4, atol=1e-4 * (1 + np.abs(want).max()))


@pytest.mark.parametrize("n,dim,nq,k,metric,dtype,share,unequal,dups", CASES)
def test_exact_against_oracle(n, dim, nq, k, metric, dtype, share, unequal, dups):
    x, q = make(n, dim, nq, dtype, unequal, dups)
    n0 = max(1, int(share * n))
    index = certex.Index(dim, metric=metric)
    ids0 = index.add(torch.from_numpy(x[:n0]).cuda())
    assert ids0[0] == 0 and ids0[-1] == n0 - 1
    if n0 < n:
        index.add(x[n0:])  # a host array: streamed in by the library
    assert index.ntotal == n
    check(index, x, q, k, metric)


def test_which_searches_the_tensor_cores_screen():
    x, q = make(50000, 128, 100, "uint8", False, 0)
    index = certex.Index(128)
    index.add(x)
    with certex.search_stats() as st:
        index.search(q, k=10)
    assert st.queries == 100 and st.dense_queries == 0 and 1000 <= st.survivors < 100 * 50000 // 10
    # float vectors of up to 128 dimensions: fp16 codes, certified threshold
    xf, qf = make(50000, 96, 100, "float32", False, 0)
    fidx = certex.Index(96)
    fidx.add(xf)
    with certex.search_stats() as st:
        check(fidx, xf, qf, 10, "l2")
    assert st.dense_queries == 0 and 1000 <= st.survivors < 100 * 50000 // 10
    # float vectors of up to 2048 dimensions are screened too (several K blocks per code row)
    xw, qw = make(20000, 200, 10, "float32", False, 0)
    widx = certex.Index(200)
    widx.add(xw)
    with certex.search_stats() as st:
        widx.search(qw, k=10)
    assert st.dense_queries == 0 and st.survivors < 10 * 20000 // 10
    # wider vectors still, tiny sets and filtered searches: every vector is scored
    xv, qv = make(3000, 2100, 10, "float32", False, 0)
    vidx = certex.Index(2100)
    vidx.add(xv)
    with certex.search_stats() as st:
        vidx.search(qv, k=10)
    assert st.dense_queries == 10
    with certex.search_stats() as st:
        fidx.search(qf, k=10, filter=np.ones(50000, dtype=bool))  # one mask for all queries keeps the screen
    assert st.dense_queries == 0
    with certex.search_stats() as st:
        fidx.search(qf, k=10, filter=np.ones((100, 50000), dtype=bool))  # a mask per query does not
    assert st.dense_queries == 100


def test_fp16_screen_keeps_near_ties_and_large_values():
    """Rows that differ from a query by less than the fp16 rounding of their coordinates, rows of very different
    norms, and values near the fp16 range: the certified threshold must keep every true neighbour."""
    rng = np.random.default_rng(0)
    n, d = 40000, 64
    x = rng.standard_normal((n, d)).astype(np.float32) * rng.choice([0.01, 1.0, 300.0], (n, 1)).astype(np.float32)
    q = x[rng.choice(n, 150, replace=False)].copy()
    for j in range(150):  # 30 near-copies of every query, apart by a few float32 ulps to a few fp16 ulps
        rows = rng.choice(n, 30, replace=False)
        x[rows] = q[j] * (1 + rng.standard_normal((30, d)).astype(np.float32) * rng.choice([1e-7, 1e-5, 1e-3], (30, 1)))
    for metric in ("l2", "ip", "cosine"):
        index = certex.Index(d, metric=metric)
        index.add(x)
        with certex.search_stats() as st:
            check(index, x, q, 10, metric)
            check(index, x, q, 40, metric)
    big = rng.standard_normal((20000, 32)).astype(np.float32) * 3e4  # some coordinates beyond 65504: no fp16 code
    bidx = certex.Index(32)
    bidx.add(big)
    with certex.search_stats() as st:
        check(bidx, big, big[:20].copy(), 5, "l2")
    assert st.dense_queries == 20


@pytest.mark.parametrize("batch", [1, 100, 128, 1000, 2048, 100000])
def test_batch_sizes(batch):
    x, q = make(40000, 64, 700, "uint8", False, 0)
    index = certex.Index(64)
    index.add(x)
    check(index, x, q, 10, "l2", batch=batch)


def test_more_queries_than_one_pass_takes():
    """40 000 queries in one call: a pass holds at most 32 768, whatever batch size is asked for."""
    x, q = make(50000, 16, 40000, "uint8", False, 0)
    index = certex.Index(16)
    index.add(x)
    with certex.search_stats() as st:
        check(index, x, q, 10, "l2", batch=100000)
    assert st.screen_passes == 2 and st.dense_queries == 0


@pytest.mark.parametrize("dtype,metric", [("uint8", "l2"), ("int8", "ip"), ("float32", "l2"), ("float32", "cosine"),
                                          ("float16", "ip")])
def test_overflowing_candidate_lists_are_screened_again_then_searched_densely(dtype, metric):
    """A query whose candidate list overflows takes a tighter threshold from the candidates it did list and is screened
    once more; what overflows again is searched without the screen."""
    x, q = make(40000, 64, 300, dtype, metric != "l2", 0)
    index = certex.Index(64, metric=metric)
    index.add(x)
    index._test_mode(2, cap=64)  # candidate lists of 64 entries: most queries overflow, the second pass fits
    with certex.search_stats() as st:
        check(index, x, q, 10, metric)
    assert 0 < st.rescreened <= 300 and st.dense_queries < st.rescreened
    index._test_mode(2, cap=12)  # hardly more than k entries: the second pass overflows too
    with certex.search_stats() as st:
        check(index, x, q, 10, metric)
    assert 0 < st.dense_queries <= st.rescreened <= 300
    index._test_mode(1)  # dense path only
    check(index, x, q, 10, metric)


@pytest.mark.parametrize("dtype,dim,metric", [("uint8", 300, "l2"), ("float32", 200, "cosine")])
def test_second_pass_on_rows_of_several_k_blocks(dtype, dim, metric):
    x, q = make(20000, dim, 150, dtype, metric != "l2", 0)
    index = certex.Index(dim, metric=metric)
    index.add(x)
    index._test_mode(2, cap=64)
    with certex.search_stats() as st:
        check(index, x, q, 10, metric)
    assert st.rescreened > 0


def test_dense_path_on_long_rows():
    """Rows longer than 2^18 are selected from in chunks by separate blocks and merged; ties across chunks go to the
    smaller id."""
    x = synthetic.correlated(700_000, 16, seed=9, dtype="float32")
    q = synthetic.correlated(24, 16, seed=10, dtype="float32")
    x[150_000] = x[7]
    x[420_001] = x[7]
    x[699_999] = x[7]
    q[0] = x[7]
    index = certex.Index(16)
    index.add(x)
    check(index, x, q, 10, "l2")
    check(index, x, q, 300, "l2")
    xi = synthetic.correlated(400_000, 32, seed=11, dtype="uint8")
    qi = synthetic.correlated(16, 32, seed=12, dtype="uint8")
    ii = certex.Index(32)
    ii.add(xi)
    ii._test_mode(1)  # the dense path on an integer index
    check(ii, xi, qi, 10, "l2")


def test_gaussian_configuration_at_full_size():
    """100 000 base and 1 000 query vectors of dimension 128, float32 i.i.d. N(0, 1) from one default_rng(0) stream,
    k = 10, L2: ids and fp64 scores equal the exhaustive CPU search, through the fp16 screen."""
    xb, xq = synthetic.gaussian_f32(100_000, 1000, 128, seed=0)
    index = certex.Index(128)
    index.add(xb)
    with certex.search_stats() as st:
        check(index, xb, xq, 10, "l2")
    assert st.dense_queries == 0 and st.survivors < 1000 * 100_000 // 50


def test_mixture_sample():
    """The benchmark's data distribution at a size the oracle finishes quickly."""
    xb = synthetic.mixture_u8(1_000_000, seed=0)
    xq = synthetic.mixture_u8(256, seed=1)
    index = certex.Index(128)
    index.add(xb)
    check(index, xb.cpu().numpy(), xq.cpu().numpy(), 10, "l2", batch=10240)


def test_one_call_search_numpy_roundtrip_and_single_vector():
    x, q = make(20000, 32, 200, "uint8", False, 0)
    D, I = certex.search(x, q.astype(np.float32), k=5)
    assert isinstance(D, np.ndarray) and I.dtype == np.int64
    ids, _ = oracle.knn(x, q, 5, "l2")
    assert np.array_equal(I, ids)
    index = certex.Index(32)
    index.add(x)
    D1, I1 = index.search(q[3], k=5)
    assert I1.shape == (5,) and np.array_equal(I1, ids[3])
    with pytest.raises(ValueError):
        index.search(q.astype(np.float32) + 0.5, k=5)  # an integer index takes integral queries only
    with pytest.raises(ValueError):
        index.search(q, k=0)
    with pytest.raises(ValueError):
        index.search(q, k=20001)


def test_golden_fixtures_on_gpu():
    """The committed known answers (pinned to the reference's own checkers) through the GPU path."""
    import os
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "golden"))
    import make_golden

    g = np.load(os.path.join(here, "golden", "golden.npz"))
    for case in make_golden.CASES:
        name, n, dim, nq, k, dtype, metric = case[:7]
        x, q = make_golden.make_case(*case)
        assert make_golden.digest(x, q) == str(g[f"{name}/data_sha256"])
        index = certex.Index(dim, metric=metric)
        index.add(x)
        _, I, S = index.search(q, k=k, return_scores=True)
        assert np.array_equal(I, g[f"{name}/ids"]) and np.array_equal(S, g[f"{name}/scores"]), name


@pytest.mark.parametrize("dtype,metric", [("uint8", "l2"), ("float32", "cosine")])
def test_a_call_short_of_memory_is_answered_in_halves(dtype, metric):
    """A call whose temporaries cannot be allocated is split in halves, recursively, like the reference's batches
    (cpp/src/neighbors/certex/certex.cu:1477-1502). The shortage is simulated on the host (test mode 4: calls of more
    than 40 queries fail as an allocation failure would), for plain, labeled and per-query-filtered searches."""
    x = synthetic.correlated(20000, 64, seed=51, dtype=dtype, unequal_norms=metric != "l2")
    q = synthetic.correlated(300, 64, seed=52, dtype=dtype)
    rng = np.random.default_rng(53)
    lab = rng.integers(0, 4, 20000).astype(np.int32)
    ql = rng.integers(0, 4, 300).astype(np.int32)
    index = certex.Index(64, metric=metric)
    index.add(x, labels=lab)
    index._test_mode(4, 40)
    _, I, S = index.search(q, k=10, return_scores=True)
    ids, scores = oracle.knn(x, q, 10, metric)
    assert np.array_equal(I, ids) and np.array_equal(S, scores)
    _, I, S = index.search(q, k=10, labels=ql, return_scores=True)
    ids, scores = oracle.knn(x, q, 10, metric, row_labels=lab, query_labels=ql)
    assert np.array_equal(I, ids) and np.array_equal(S, scores)
    index._test_mode(4, 70)  # a bitmap is cut at whole words of query rows: pieces of 64 queries are the smallest
    per_query = rng.random((300, 20000)) < 0.05
    _, I, S = index.search(q, k=10, filter=per_query, return_scores=True)
    ids, scores = oracle.knn(x, q, 10, metric, keep_pair=per_query.astype(np.uint8))
    assert np.array_equal(I, ids) and np.array_equal(S, scores)
    index._test_mode(4, 0)
    with pytest.raises(certex.CertexError, match="out of device memory"):
        index.search(q[:1], k=10)


def test_merge_of_more_candidates_than_one_block_sorts():
    """8 shards x k = 2048 = 16 384 candidates per query: merged in rounds, equal to the oracle's merge."""
    rng = np.random.default_rng(7)
    parts, nq, k = 8, 12, 2048
    s = np.sort(rng.integers(0, 5000, (parts, nq, k)).astype(np.float64), axis=2)
    i = rng.permutation(parts * nq * k).reshape(parts, nq, k).astype(np.int64)
    i[3, :, 2000:] = -1
    s[3, :, 2000:] = np.inf
    q = torch.zeros((nq, 8), dtype=torch.float32, device="cuda")
    D, I, S = certex.merge_shards(q, torch.from_numpy(s).cuda(), torch.from_numpy(i).cuda(), "l2", return_scores=True)
    wi, ws = oracle.merge(i, s)
    assert np.array_equal(I.cpu().numpy(), wi) and np.array_equal(S.cpu().numpy(), ws)


@pytest.mark.parametrize("dtype,metric,dim", [("uint8", "l2", 128), ("float32", "l2", 96), ("float32", "cosine", 300),
                                             ("int8", "ip", 64)])
def test_chained_and_exact_threshold_stages_agree(dtype, metric, dim):
    """Plain searches take their thresholds from the chained bound of the anchor pass (a value below each group's exact
    maximum); with test mode 5 from the exact group maxima, as searches with a bitset filter do. Both are exact, and
    the bound costs hardly any extra survivors."""
    x, q = make(60000, dim, 200, dtype, metric != "l2", 0, seed=71)
    index = certex.Index(dim, metric=metric)
    index.add(x)
    with certex.search_stats() as chained:
        check(index, x, q, 10, metric)
    index._test_mode(5)
    with certex.search_stats() as exact:
        check(index, x, q, 10, metric)
    assert chained.dense_queries == 0 and exact.dense_queries == 0
    assert exact.survivors <= chained.survivors <= 1.25 * exact.survivors + 200 * 16
