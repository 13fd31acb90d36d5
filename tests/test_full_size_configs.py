"""The filtered workload and the sparse-attention workload at their full sizes, bit-for-bit against the CPU oracle.

* 1 000 000 x 768 float32 unit vectors (anisotropic mixture of 4 096 clusters), cosine, k = 100, one of 64 labels per
  vector and per query, 10 000 queries per batch searched by label; between the batches 1 % of the live vectors are
  removed and as many fresh ones added. Every batch: 256 sampled queries against the oracle (ids and fp64 scores
  equal), and for all 10 000 queries the order, the labels and the liveness of what came back.
* 8 KV heads x 131 072 bf16 keys of dimension 128 with 4 outlier channels per head scaled by 20, 32 query heads x 16
  queries, inner product, k = 2048: all 512 queries against the oracle.

The conventions checked are those of the reference's tests (tests/test_exact.py:49-84: best first, exact fp64 scores;
certex/attention.py:84-106: query head h reads KV head h // group, ids are key positions)."""

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from libcertex_b200 import synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_filtered_cosine_workload_at_full_size():
    n, dim, nq, k, n_labels, sample = 1_000_000, 768, 10_000, 100, 64, 256
    churn, batches = n // 100, 3
    total = n + (batches - 1) * churn
    x_dev = synthetic.clustered_unit_f32(total, dim, seed=0)
    q_dev = synthetic.clustered_unit_f32(nq, dim, seed=1)
    g = torch.Generator().manual_seed(3)
    lab = torch.randint(0, n_labels, (total,), generator=g, dtype=torch.int32)
    ql = torch.randint(0, n_labels, (nq,), generator=g, dtype=torch.int32)
    xh, qh = x_dev.cpu().numpy(), q_dev.cpu().numpy()
    ql_dev = ql.cuda()
    index = certex.Index(dim, metric="cosine")
    index.add(x_dev[:n], labels=lab[:n].cuda())
    live = lab.numpy().copy()  # label of every live id, -1 for removed and not yet added ones
    live[n:] = -1
    rng = np.random.default_rng(5)
    size = n
    for step in range(batches):
        with certex.search_stats() as st:
            D, I, S = index.search(q_dev, k=k, labels=ql_dev, batch=10240, return_scores=True)
        torch.cuda.synchronize()
        assert st.routed_queries >= nq, "the searches by label did not go through the routed tensor-core pass"
        Ih, Sh, Dh = I.cpu().numpy(), S.cpu().numpy(), D.cpu().numpy()
        # every list: live vectors of the query's label, best first, equal scores by ascending id, similarity = 1 - s/2
        assert Ih.min() >= 0 and Ih.max() < size  # every label holds far more than k vectors
        assert (live[Ih] == ql.numpy()[:, None]).all()
        assert (Sh[:, 1:] >= Sh[:, :-1]).all()
        tie = Sh[:, 1:] == Sh[:, :-1]
        assert (Ih[:, 1:][tie] > Ih[:, :-1][tie]).all()
        assert np.array_equal(Dh, 1 - (Sh / 2).astype(np.float32))
        pick = np.sort(rng.choice(nq, sample, replace=False))
        ids, scores = oracle.knn(xh[:size], qh[pick], k, "cosine", row_labels=live[:size], query_labels=ql.numpy()[pick])
        assert np.array_equal(Ih[pick], ids), f"batch {step}: {(Ih[pick] != ids).any(1).sum()} of {sample} queries differ"
        assert np.array_equal(Sh[pick], scores), f"batch {step}: fp64 scores differ"
        if step + 1 < batches:
            gone = rng.choice(np.flatnonzero(live[:size] >= 0), churn, replace=False)
            index.remove(torch.from_numpy(gone).cuda())
            live[gone] = -1
            index.add(x_dev[size:size + churn], labels=lab[size:size + churn].cuda())
            live[size:size + churn] = lab.numpy()[size:size + churn]
            size += churn


def test_keycache_workload_at_full_size():
    n_kv, n_heads, n, d, m, k = 8, 32, 131_072, 128, 16, 2048
    keys = synthetic.keys_with_outliers(n_kv, n, d, n_outlier=4, scale=20.0, seed=0)
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((n_heads, m, d), generator=g, device="cuda").to(torch.bfloat16)
    cache = certex.KeyCache(n_kv, d, k=k).append(keys)
    with certex.search_stats() as st:
        scores, ids = cache.topk(q)
    torch.cuda.synchronize()
    assert ids.shape == (n_heads, m, k) and scores.shape == (n_heads, m, k)
    assert st.dense_queries == 0 and st.routed_queries >= n_heads * m, "the keys were not screened per head"
    # bf16 keys are searched as float16 where that loses nothing but range (certex/attention.py:37-41)
    kf, qf = keys.half().cpu().numpy(), q.half().cpu().numpy()
    assert np.isfinite(kf).all()
    group = n_heads // n_kv
    got_ids, got_sc = ids.cpu().numpy(), scores.cpu().numpy()
    # the exact fp64 scores of the same search (|q|^2 - 2 <q, key>), through the index the cache holds
    heads = (torch.arange(n_heads, dtype=torch.int32, device="cuda") // group).repeat_interleave(m)
    Q = q.half().reshape(n_heads * m, d).contiguous()
    D, I, S = cache.index.search(Q, k=k, labels=heads, return_scores=True)
    pos = cache._position[I].reshape(n_heads, m, k).cpu().numpy()
    S = S.reshape(n_heads, m, k).cpu().numpy()
    assert np.array_equal(pos, got_ids)
    for h in range(n_heads):
        want_ids, want_s = oracle.knn(kf[h // group], qf[h], k, "ip")
        assert np.array_equal(got_ids[h], want_ids), f"query head {h}: ids differ from the oracle"
        assert np.array_equal(S[h], want_s), f"query head {h}: fp64 scores differ from the oracle"
        # returned similarity: <q, key> = (|q|^2 - score) / 2 as float32, descending
        qq = (qf[h].astype(np.float64) ** 2).sum(1)
        np.testing.assert_allclose(got_sc[h], ((qq[:, None] - want_s) / 2), rtol=1e-5, atol=1e-4)
        assert (got_sc[h][:, :-1] >= got_sc[h][:, 1:]).all()
