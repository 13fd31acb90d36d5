"""Updates and filtered search on the GPU against the CPU oracle with a keep predicate: removals (including every
query's true nearest neighbour), additions after removals, labels at several selectivities, labels after extend and
remove, bitset and bitmap filters, save / load, a reader concurrent with a writer. The scenarios follow the reference's
cpp/tests/neighbors/ann_certex/test_updates.cu:92-591 and tests/test_exact.py."""

import threading

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from libcertex_b200 import synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu


def data(n, dim, nq, dtype, seed=5):
    return synthetic.correlated(n, dim, seed=seed, dtype=dtype), synthetic.correlated(nq, dim, seed=seed + 1, dtype=dtype)


def same(index, x, q, k, metric="l2", keep_row=None, keep_pair=None, row_labels=None, query_labels=None, **kw):
    _, I, S = index.search(q, k=k, return_scores=True, **kw)
    ids, scores = oracle.knn(x, q, k, metric, keep_row=keep_row, keep_pair=keep_pair, row_labels=row_labels,
                             query_labels=query_labels)
    assert np.array_equal(I, ids), f"{(I != ids).any(1).sum()} of {len(ids)} queries differ"
    assert np.array_equal(S, scores)


@pytest.mark.parametrize("dtype", ["uint8", "float32"])
def test_remove_then_add(dtype):
    x, q = data(30000, 48, 300, dtype)
    index = certex.Index(48, capacity=12000)
    index.add(x[:20000])
    same(index, x[:20000], q, 10)
    # remove every query's nearest neighbour and a random 5 %
    nn, _ = oracle.knn(x[:20000], q, 1, "l2")
    rng = np.random.default_rng(0)
    gone = np.unique(np.concatenate([nn[:, 0], rng.choice(20000, 1000, replace=False)]))
    index.remove(gone)
    index.remove(gone[:10])  # removing twice changes nothing
    keep = np.ones(20000, dtype=np.uint8)
    keep[gone] = 0
    assert index.ntotal == 20000 - len(gone)
    same(index, x[:20000], q, 10, keep_row=keep)
    # ids continue after the removed ones and are never reused
    new_ids = index.add(x[20000:])
    assert new_ids[0] == 20000 and new_ids[-1] == 29999
    keep = np.concatenate([keep, np.ones(10000, dtype=np.uint8)])
    same(index, x, q, 10, keep_row=keep)


@pytest.mark.parametrize("dtype", ["uint8", "float32"])
def test_many_small_appends_keep_the_screen_tight(dtype):
    """An L2 index grown by a thousand appends of a few dozen rows, with removals in between: the answers are the
    oracle's, and the screen keeps about as many pairs as on the same rows added in one call (small sorted runs are
    sorted together as the index grows)."""
    n, step, dim = 60000, 37, 128
    x = synthetic.mixture_u8(n, seed=3).cpu().numpy()
    q = synthetic.mixture_u8(400, seed=4).cpu().numpy()
    if dtype == "float32":
        x, q = x.astype(np.float32) / 16, q.astype(np.float32) / 16
    grown = certex.Index(dim)
    grown.add(x[:20000])
    rng = np.random.default_rng(2)
    keep = np.ones(n, dtype=np.uint8)
    for lo in range(20000, n, step):
        grown.add(x[lo : lo + step])
        if lo % (step * 100) == 20000 % (step * 100):  # every hundredth append: some of the newest rows go
            gone = rng.choice(np.arange(max(lo - 2000, 0), lo + step), 50, replace=False)
            grown.remove(gone)
            keep[gone] = 0
    whole = certex.Index(dim)
    whole.add(x)
    whole.remove(np.flatnonzero(keep == 0))
    with certex.search_stats() as st_grown:
        same(grown, x, q, 10, keep_row=keep)
    with certex.search_stats() as st_whole:
        same(whole, x, q, 10, keep_row=keep)
    assert st_grown.dense_queries == 0 and st_grown.rescreened == 0
    assert st_grown.survivors <= 1.25 * st_whole.survivors + 400 * 16


@pytest.mark.parametrize("n_labels", [5, 50, 500, 5000])
def test_search_by_label(n_labels):
    x, q = data(20000, 32, 200, "uint8")
    rng = np.random.default_rng(1)
    lab = rng.integers(0, n_labels, 20000).astype(np.int32)
    ql = rng.integers(0, n_labels, 200).astype(np.int32)
    index = certex.Index(32)
    index.add(x, labels=lab)
    same(index, x, q, 10, row_labels=lab, query_labels=ql, labels=ql)
    with pytest.raises(ValueError):
        index.add(x[:5])  # a labeled index needs labels with every addition


def test_labels_after_extend_and_remove():
    x, q = data(24000, 40, 150, "float32")
    rng = np.random.default_rng(2)
    lab = rng.integers(0, 16, 24000).astype(np.int32)
    ql = rng.integers(0, 17, 150).astype(np.int32)  # label 16 has no vectors: all -1
    index = certex.Index(40)
    index.add(x[:16000], labels=lab[:16000])
    index.add(x[16000:], labels=lab[16000:])
    gone = rng.choice(24000, 2000, replace=False)
    index.remove(gone)
    masked = lab.copy()
    masked[gone] = -1  # the oracle treats -1 as "matches nothing"
    D, I, S = index.search(q, k=10, labels=ql, return_scores=True)
    ids, scores = oracle.knn(x, q, 10, "l2", row_labels=masked, query_labels=ql)
    assert np.array_equal(I, ids) and np.array_equal(S, scores)
    assert (I[ql == 16] == -1).all() and np.isinf(D[ql == 16]).all()


def test_label_partition_with_newer_vectors():
    """The partition made at 20 000 vectors stays while 1 500 more arrive (less than an eighth): the search then scores
    the label's partition entries and the newer vectors together. Partitioned and unpartitioned searches agree."""
    x, q = data(21500, 24, 400, "float32", seed=11)
    rng = np.random.default_rng(12)
    lab = rng.integers(0, 32, 21500).astype(np.int32)
    ql = rng.integers(-1, 34, 400).astype(np.int32)  # -1 and the labels 32, 33 match nothing
    index = certex.Index(24, partition_labels="lazy")
    index.add(x[:20000], labels=lab[:20000])
    assert index.info()["n_partitioned"] == 20000
    index.add(x[20000:], labels=lab[20000:])  # fewer than an eighth of the vectors: the partition stays
    assert index.info()["n_partitioned"] == 20000
    gone = rng.choice(21500, 1500, replace=False)
    index.remove(gone)
    masked = lab.copy()
    masked[gone] = -1
    same(index, x, q, 10, row_labels=masked, query_labels=ql, labels=ql)
    Dp, Ip, Sp = index.search(q, k=10, labels=ql, return_scores=True)
    index._test_mode(1)  # the label test over every vector instead of the partition
    Du, Iu, Su = index.search(q, k=10, labels=ql, return_scores=True)
    index._test_mode(0)
    assert np.array_equal(Ip, Iu) and np.array_equal(Sp, Su) and np.array_equal(Dp, Du)
    assert (Ip[(ql < 0) | (ql >= 32)] == -1).all()


@pytest.mark.parametrize("dtype,dim,metric,k", [("uint8", 64, "l2", 10), ("int8", 300, "ip", 10), ("float32", 96, "l2", 10),
                                               ("float32", 768, "cosine", 100), ("float16", 200, "ip", 20)])
def test_labels_are_screened_against_their_own_rows(dtype, dim, metric, k):
    """Labels with at least 2k groups of 64 rows go through the routed tensor-core pass (label-ordered copy of the code
    rows, one block of whole tiles per label); the answers equal the oracle's and those of the dense label groups.
    Label 0 is large, label 7 small (dense), some queries ask for labels without rows; rows are removed in between."""
    n, nq = 60000, 500
    x, q = data(n, dim, nq, dtype, seed=31)
    rng = np.random.default_rng(32)
    lab = rng.choice(8, n, p=[0.4, 0.2, 0.15, 0.1, 0.08, 0.04, 0.0295, 0.0005]).astype(np.int32)
    ql = rng.integers(0, 10, nq).astype(np.int32)
    index = certex.Index(dim, metric=metric)
    index.add(x, labels=lab)
    with certex.search_stats() as st:
        same(index, x, q, k, metric=metric, row_labels=lab, query_labels=ql, labels=ql)
    assert st.routed_queries >= (ql == 0).sum() and 0 < st.dense_queries < nq
    gone = rng.choice(n, 3000, replace=False)
    index.remove(gone)
    masked = lab.copy()
    masked[gone] = -1
    with certex.search_stats() as st:
        _, Ir, Sr = index.search(q, k=k, labels=ql, return_scores=True)
    assert st.routed_queries > 0
    ids, scores = oracle.knn(x, q, k, metric, row_labels=masked, query_labels=ql)
    assert np.array_equal(Ir, ids) and np.array_equal(Sr, scores)
    index._test_mode(3)  # dense label groups only
    with certex.search_stats() as st:
        _, Id, Sd = index.search(q, k=k, labels=ql, return_scores=True)
    assert st.routed_queries == 0 and np.array_equal(Ir, Id) and np.array_equal(Sr, Sd)


@pytest.mark.parametrize("n", [450000, 210000])
def test_routed_pass_with_many_labels_and_uneven_query_counts(n):
    """300 labels of about 1500 rows (k = 10 needs 1280 for groups of 64 rows) or of about 700 rows (thresholds from
    the maxima of single chains of 16 rows): most are routed, every label's block is a few tiles and the segments of
    many labels share a CTA; one label has 400 queries (several query tiles), most have one or none."""
    dim, nq = 32, 1200
    x, q = data(n, dim, nq, "uint8", seed=33)
    rng = np.random.default_rng(34)
    lab = rng.integers(0, 300, n).astype(np.int32)
    ql = rng.integers(0, 300, nq).astype(np.int32)
    ql[:400] = 17
    index = certex.Index(dim)
    index.add(x, labels=lab)
    with certex.search_stats() as st:
        same(index, x, q, 10, row_labels=lab, query_labels=ql, labels=ql)
    assert st.routed_queries > 400


def test_more_queries_of_one_label_than_a_routed_pass_takes():
    """36 000 queries of one label (a routed pass holds 32 768 query slots) and 1 000 of another."""
    n, dim = 200000, 16
    x = synthetic.correlated(n, dim, seed=41, dtype="uint8")
    q = synthetic.correlated(37000, dim, seed=42, dtype="uint8")
    rng = np.random.default_rng(43)
    lab = rng.integers(0, 2, n).astype(np.int32)
    ql = np.zeros(37000, dtype=np.int32)
    ql[rng.choice(37000, 1000, replace=False)] = 1
    index = certex.Index(dim)
    index.add(x, labels=lab)
    with certex.search_stats() as st:
        same(index, x, q, 10, row_labels=lab, query_labels=ql, labels=ql)
    assert st.routed_queries >= 37000


def test_label_partition_small_labels_and_large_k():
    """Labels with fewer than k vectors pad with -1; one query per label; labels that are not consecutive numbers."""
    x, q = data(6000, 16, 64, "uint8", seed=13)
    rng = np.random.default_rng(14)
    lab = (rng.integers(0, 300, 6000) * 1000 + 7).astype(np.int32)  # about 20 vectors per label
    ql = (np.arange(64) * 1000 + 7).astype(np.int32)
    index = certex.Index(16)
    index.add(x, labels=lab)
    _, I, S = index.search(q, k=50, labels=ql, return_scores=True)
    ids, scores = oracle.knn(x, q, 50, "l2", row_labels=lab, query_labels=ql)
    assert np.array_equal(I, ids) and np.array_equal(S, scores)
    assert (I == -1).any() and (I[:, 0] >= 0).all()


def test_label_partition_long_labels():
    """Two labels of about 600 000 vectors each (2 344 tiles: the thresholds come from every second tile); with the
    dense label groups the score rows are long enough to be selected from in chunks."""
    x, q = data(1200000, 8, 24, "uint8", seed=15)
    rng = np.random.default_rng(16)
    lab = rng.integers(0, 2, 1200000).astype(np.int32)
    ql = rng.integers(0, 2, 24).astype(np.int32)
    index = certex.Index(8)
    index.add(x, labels=lab)
    same(index, x, q, 100, row_labels=lab, query_labels=ql, labels=ql)
    index._test_mode(3)  # dense label groups
    same(index, x, q, 100, row_labels=lab, query_labels=ql, labels=ql)


def test_relabeling_voids_the_partition():
    x, q = data(8000, 16, 100, "float32", seed=17)
    rng = np.random.default_rng(18)
    lab = rng.integers(0, 8, 8000).astype(np.int32)
    ql = rng.integers(0, 8, 100).astype(np.int32)
    index = certex.Index(16)
    index.add(x, labels=lab)
    assert index.info()["n_partitioned"] == 8000
    lab2 = rng.integers(0, 8, 8000).astype(np.int32)
    index.set_labels(lab2, first=0)
    assert index.info()["n_partitioned"] == 0
    same(index, x, q, 10, row_labels=lab2, query_labels=ql, labels=ql)
    index.partition_by_labels()
    assert index.info()["n_partitioned"] == 8000
    same(index, x, q, 10, row_labels=lab2, query_labels=ql, labels=ql)


def test_labeled_cosine_with_churn():
    """The shape of the filtered workload at a small scale: unit vectors of dimension 768, cosine, k = 100, one of 64
    labels per vector and query, and between query batches 1 % of the vectors removed and as many added."""
    n, dim, nq, k = 20000, 768, 96, 100
    x = synthetic.clustered_unit_f32(n + 600, dim, n_clusters=256, seed=19).cpu().numpy()
    q = synthetic.clustered_unit_f32(nq, dim, n_clusters=256, seed=20).cpu().numpy()
    rng = np.random.default_rng(21)
    lab = rng.integers(0, 64, n + 600).astype(np.int32)
    ql = rng.integers(0, 64, nq).astype(np.int32)
    index = certex.Index(dim, metric="cosine")
    index.add(x[:n], labels=lab[:n])
    live = lab.copy()
    live[n:] = -1
    size = n
    for step in range(3):
        _, I, S = index.search(q, k=k, labels=ql, return_scores=True)
        ids, scores = oracle.knn(x[:size], q, k, "cosine", row_labels=live[:size], query_labels=ql)
        assert np.array_equal(I, ids), f"step {step}: {(I != ids).any(1).sum()} queries differ"
        assert np.array_equal(S, scores)
        alive = np.flatnonzero(live[:size] >= 0)
        gone = rng.choice(alive, 200, replace=False)
        index.remove(gone)
        live[gone] = -1
        index.add(x[size:size + 200], labels=lab[size:size + 200])
        live[size:size + 200] = lab[size:size + 200]
        size += 200


@pytest.mark.parametrize("dtype", ["uint8", "float16"])
def test_bitset_and_bitmap(dtype):
    x, q = data(15000, 64, 120, dtype)
    rng = np.random.default_rng(3)
    index = certex.Index(64)
    index.add(x)
    mask = rng.random(15000) < 0.3
    with certex.search_stats() as st:
        same(index, x, q, 10, keep_row=mask.astype(np.uint8), filter=mask)
    assert st.dense_queries == 0 and st.survivors < 120 * 15000 // 4  # screened: thresholds from the kept anchors
    rare = rng.random(15000) < 0.004  # about 60 kept vectors: too few anchors pass, the lists overflow
    same(index, x, q, 10, keep_row=rare.astype(np.uint8), filter=rare)
    per_query = rng.random((120, 15000)) < 0.05
    per_query[7] = False  # a query with no admitted vector
    per_query[8, :3] = True
    per_query[8, 3:] = False  # fewer than k admitted
    D, I, S = index.search(q, k=10, filter=per_query, return_scores=True)
    ids, scores = oracle.knn(x, q, 10, "l2", keep_pair=per_query.astype(np.uint8))
    assert np.array_equal(I, ids) and np.array_equal(S, scores)
    assert (I[7] == -1).all() and (I[8, 3:] == -1).all() and (I[8, :3] >= 0).all()
    gone = rng.choice(15000, 3000, replace=False)  # removed vectors and a mask together
    index.remove(gone)
    both = mask.copy()
    both[gone] = False
    same(index, x, q, 10, keep_row=both.astype(np.uint8), filter=mask)


@pytest.mark.parametrize("dtype,metric", [("uint8", "l2"), ("float32", "cosine")])
def test_save_load(tmp_path, dtype, metric):
    x, q = data(12000, 32, 100, dtype)
    index = certex.Index(32, metric=metric)
    rng = np.random.default_rng(4)
    lab = rng.integers(0, 4, 12000).astype(np.int32)
    index.add(x, labels=lab)
    gone = rng.choice(12000, 500, replace=False)
    index.remove(gone)
    D0, I0 = index.search(q, k=10)
    path = tmp_path / "index.bin"
    index.save(path)
    loaded = certex.Index.load(path)
    assert loaded.ntotal == index.ntotal and loaded.metric == metric
    D1, I1 = loaded.search(q, k=10)
    assert np.array_equal(I0, I1) and np.array_equal(D0, D1)
    ql = rng.integers(0, 4, 100).astype(np.int32)
    _, Ia = index.search(q, k=5, labels=ql)
    _, Ib = loaded.search(q, k=5, labels=ql)
    assert np.array_equal(Ia, Ib)


def test_search_concurrent_with_extend():
    """A search sees one consistent snapshot: its result equals the exact answer over one of the published prefixes
    (the reference's cpp/tests/neighbors/ann_certex/test_updates.cu:504-591)."""
    x, q = data(40000, 32, 64, "uint8")
    index = certex.Index(32)
    index.add(x[:10000])
    prefixes = [10000, 20000, 30000, 40000]
    answers = [oracle.knn(x[:p], q, 10, "l2")[0] for p in prefixes]
    results, errors = [], []

    def reader():
        try:
            for _ in range(30):
                _, I = index.search(q, k=10)
                results.append(I)
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    def writer():
        try:
            for p0, p1 in zip(prefixes[:-1], prefixes[1:]):
                index.add(x[p0:p1])
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=reader) for _ in range(3)] + [threading.Thread(target=writer)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for I in results:
        assert any(np.array_equal(I, a) for a in answers)
    _, I = index.search(q, k=10)
    assert np.array_equal(I, answers[-1])


def test_removed_rows_exceeding_k_leave_missing_entries():
    x, q = data(64, 16, 20, "uint8")
    index = certex.Index(16)
    index.add(x)
    index.remove(np.arange(60))
    D, I = index.search(q, k=10)
    assert (I[:, 4:] == -1).all() and (I[:, :4] >= 60).all() and np.isinf(D[:, 4:]).all()


def _write_reference_file(path, x, metric_code, removed, labels, int8_rows, width=27, stride=16):
    """A file in the layout the reference's serialize writes (cpp/src/neighbors/certex/certex_serialize.cu:40-132):
    the 4-byte dtype prefix, then one .npy record per scalar and array, in its order. The projection, certificate rows
    and anchors hold filler values: they are the reference's own screening data."""
    from numpy.lib import format as npy

    n, d = x.shape
    prefix = {"uint8": b"|u1\0", "int8": b"|i1\0", "float32": b"<f4\0", "float16": b"<f2\0"}[str(x.dtype)]
    mp = 64
    with open(path, "wb") as f:
        def put(value, dtype=None):
            npy.write_array(f, np.asarray(value, dtype=dtype), version=(1, 0))

        f.write(prefix)
        put(0x43455258, np.int32), put(1, np.int32), put(metric_code, np.int32), put(d, np.int64), put(width, np.int32)
        put(stride, np.int32), put(0, np.int32), put(n, np.int64), put(int(removed.sum()), np.int64)
        put(0 if labels is None else 1, np.int32), put(1 if int8_rows else 0, np.int32)
        for v in (0.5, 1.0, 2.0, 3.0, 4.0, 5.0):  # alpha and the certificate maxima
            put(v, np.float64)
        put(np.zeros(d, np.float32)), put(np.zeros((width, d), np.float32))  # center, basis
        if int8_rows:
            put(7.0, np.float64), put(np.zeros((n, 64), np.int8)), put(np.zeros((n, 5), np.float32))
        else:
            put(np.zeros((n, mp), np.float16))
        na = (n + stride - 1) // stride
        put(np.zeros((na, mp), np.float16)), put(np.zeros((na, d), x.dtype))
        put(x), put(removed.astype(np.uint8))
        if labels is not None:
            put(labels.astype(np.int32))
        put(0, np.int32)  # no k-means lists


@pytest.mark.parametrize("dtype,metric,int8_rows,labeled", [("uint8", "l2", True, True), ("float32", "cosine", False, False),
                                                            ("float16", "ip", False, True)])
def test_load_a_file_in_the_reference_layout(tmp_path, dtype, metric, int8_rows, labeled):
    x, q = data(15000, 40, 100, dtype, seed=21)
    rng = np.random.default_rng(4)
    removed = (rng.random(15000) < 0.03)
    lab = rng.integers(0, 6, 15000).astype(np.int32) if labeled else None
    path = tmp_path / "reference_layout.bin"
    _write_reference_file(path, x, {"l2": 0, "cosine": 2, "ip": 6}[metric], removed, lab, int8_rows)
    loaded = certex.Index.load(path)
    assert loaded.ntotal == 15000 - int(removed.sum()) and loaded.metric == metric
    keep = (~removed).astype(np.uint8)
    same(loaded, x, q, 10, metric, keep_row=keep)
    if labeled:
        ql = rng.integers(0, 6, 100).astype(np.int32)
        same(loaded, x, q, 10, metric, keep_row=keep, row_labels=lab, query_labels=ql, labels=ql)
    # a file with k-means lists is refused, not misread
    with open(path, "r+b") as f:
        f.seek(-4, 2)
        f.write(np.int32(3).tobytes())
    with pytest.raises(Exception, match="lists"):
        certex.Index.load(path)
