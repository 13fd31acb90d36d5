"""KeyCache / topk against torch.topk semantics with exact fp64 inner products (the reference's tests/test_attention.py):
grouped-query mapping, appended keys, single-vector queries, large k."""

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from oracle import oracle

pytestmark = pytest.mark.gpu


def exact_topk(keys, q, k, group):
    """ids [H, m, k] by the CPU oracle: head h reads KV head h // group; inner products descending, ties to the smaller
    key position."""
    H, m, d = q.shape
    out = np.empty((H, m, k), dtype=np.int64)
    for h in range(H):
        ids, _ = oracle.knn(keys[h // group], q[h], k, "ip")
        out[h] = ids
    return out


def test_topk_matches_oracle_with_gqa_and_append():
    g = torch.Generator().manual_seed(0)
    n_kv, n_heads, d, n, m, k = 2, 8, 64, 6000, 5, 37
    keys = torch.randn(n_kv, n, d, generator=g).half()
    q = torch.randn(n_heads, m, d, generator=g).half()
    cache = certex.KeyCache(n_kv, d, k=k)
    cache.append(keys[:, :4000].cuda())
    cache.append(keys[:, 4000:].cuda())
    scores, ids = cache.topk(q.cuda())
    want = exact_topk(keys.numpy(), q.numpy(), k, n_heads // n_kv)
    assert np.array_equal(ids.cpu().numpy(), want)
    ip = torch.einsum("hmd,hmkd->hmk", q.double(), keys.double()[torch.arange(n_heads)[:, None, None] // 4, ids.cpu()])
    assert torch.allclose(scores.cpu().double(), ip, rtol=1e-3, atol=1e-3)
    assert (scores[..., :-1] >= scores[..., 1:]).all()
    s1, i1 = cache.topk(q[:, 0].cuda(), k=5)
    assert i1.shape == (n_heads, 5) and np.array_equal(i1.cpu().numpy(), want[:, 0, :5])


def test_one_call_topk_large_k_bf16_with_outliers():
    g = torch.Generator().manual_seed(1)
    keys = torch.randn(2, 5000, 32, generator=g)
    keys[:, :, [3, 17]] *= 20  # outlier channels
    keys = keys.bfloat16()
    q = torch.randn(4, 3, 32, generator=g).bfloat16()
    scores, ids = certex.topk(q.cuda(), keys.cuda(), k=2048)
    kf, qf = keys.half().numpy(), q.half().numpy()  # bf16 inputs are searched as float16 when that is exact enough
    assert np.isfinite(kf).all()
    want = exact_topk(kf, qf, 2048, 2)
    assert np.array_equal(ids.cpu().numpy(), want)


def test_keys_appended_after_the_partition_are_found():
    """A few keys appended after the cache was partitioned by head stay outside the partition (it is renewed once an
    eighth of the keys is newer); they are scored next to the partitioned keys of their head."""
    g = torch.Generator().manual_seed(2)
    n_kv, n_heads, d, m, k = 2, 4, 32, 6, 20
    keys = torch.randn(n_kv, 9000, d, generator=g).half()
    q = torch.randn(n_heads, m, d, generator=g).half()
    cache = certex.KeyCache(n_kv, d, k=k)
    cache.append(keys[:, :8500].cuda())
    for lo in range(8500, 9000, 100):  # decoding steps
        cache.append(keys[:, lo : lo + 100].cuda())
    assert cache.index.info()["n_partitioned"] < 2 * 9000
    scores, ids = cache.topk(q.cuda())
    want = exact_topk(keys.numpy(), q.numpy(), k, n_heads // n_kv)
    assert np.array_equal(ids.cpu().numpy(), want)
