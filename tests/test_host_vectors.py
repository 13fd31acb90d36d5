"""Vectors kept in page-locked host memory (index_params.host_vectors, the reference's storage option of
cpp/include/cuvs/neighbors/certex.hpp:56-61 and certex/index.py `storage="host"`): every answer must equal the one of
an index with its vectors on the device, i.e. the CPU oracle's, bit for bit, through additions that regrow the index,
removals, labels, a mask over the ids and a mask per query."""

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from libcertex_b200 import synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu


def _same(index, x, q, k, metric, **kw):
    search_kw = {}
    if "query_labels" in kw:
        search_kw["labels"] = kw["query_labels"]
    if "keep_row" in kw:
        search_kw["filter"] = kw["keep_row"].astype(bool)
    if "keep_pair" in kw:
        search_kw["filter"] = kw["keep_pair"].astype(bool)
    _, I, S = index.search(q, k=k, return_scores=True, **search_kw)
    ids, scores = oracle.knn(x, q, k, metric, **kw)
    assert np.array_equal(np.asarray(I), ids), f"{(np.asarray(I) != ids).any(1).sum()} of {len(ids)} queries differ"
    assert np.array_equal(np.asarray(S), scores)


@pytest.mark.parametrize("dtype,metric,dim", [("uint8", "l2", 128), ("int8", "ip", 96), ("float32", "cosine", 200),
                                             ("float16", "l2", 64)])
def test_host_storage_answers_like_device_storage(dtype, metric, dim):
    n, nq, k = 30000, 150, 10
    x = synthetic.correlated(n, dim, seed=61, dtype=dtype, unequal_norms=metric != "l2")
    q = synthetic.correlated(nq, dim, seed=62, dtype=dtype)
    rng = np.random.default_rng(63)
    lab = rng.integers(0, 5, n).astype(np.int32)
    ql = rng.integers(0, 5, nq).astype(np.int32)
    index = certex.Index(dim, metric=metric, storage="host")
    index.add(x[:7000], labels=lab[:7000])
    index.add(torch.from_numpy(x[7000:]).cuda(), labels=lab[7000:])  # regrows: host block to host block, device rows in
    assert index.info()["storage"] == "host" and index.ntotal == n
    with certex.search_stats() as st:
        _same(index, x, q, k, metric)
    assert st.dense_queries == 0, "a plain search of a host-stored index must still be screened"
    with certex.search_stats() as st:
        _same(index, x, q, k, metric, row_labels=lab, query_labels=ql)
    assert st.routed_queries > 0
    gone = rng.choice(n, 900, replace=False)
    index.remove(gone)
    keep = np.ones(n, dtype=np.uint8)
    keep[gone] = 0
    _same(index, x, q, k, metric, keep_row=keep)  # removed ids never come back; the mask only states the same
    mask = (rng.random(n) < 0.4).astype(np.uint8) & keep
    _, I, S = index.search(q, k=k, filter=mask.astype(bool), return_scores=True)
    ids, scores = oracle.knn(x, q, k, metric, keep_row=mask)
    assert np.array_equal(np.asarray(I), ids) and np.array_equal(np.asarray(S), scores)
    per_query = ((rng.random((nq, n)) < 0.03) & keep.astype(bool)[None, :]).astype(np.uint8)  # every vector scored, from the host
    _, I, S = index.search(q, k=k, filter=per_query.astype(bool), return_scores=True)
    ids, scores = oracle.knn(x, q, k, metric, keep_pair=per_query)
    assert np.array_equal(np.asarray(I), ids) and np.array_equal(np.asarray(S), scores)


def test_host_storage_survives_save_and_load(tmp_path):
    x = synthetic.correlated(9000, 32, seed=64, dtype="uint8")
    q = synthetic.correlated(40, 32, seed=65, dtype="uint8")
    index = certex.Index(32, storage="host")
    index.add(x)
    index.save(tmp_path / "host.idx")
    again = certex.Index.load(tmp_path / "host.idx")
    _same(again, x, q, 10, "l2")
