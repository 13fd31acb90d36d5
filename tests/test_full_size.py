"""The headline configuration at its full size (10 000 000 x 128 uint8 mixture rows, 10 000 queries, k = 10, L2),
checked through properties that need no exhaustive answer for every query: order and uniqueness of every list, rows
of the base as their own nearest neighbours, equality of the answers of two half shards merged with the answer of one
index, and the CPU oracle on a sample of the queries."""

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from libcertex_b200 import synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu
N, NQ, K = 10_000_000, 10_000, 10


@pytest.fixture(scope="module")
def full():
    xb = synthetic.mixture_u8(N, seed=0)
    xq = synthetic.mixture_u8(NQ, seed=1)
    index = certex.Index(128)
    index.add(xb)
    with certex.search_stats() as st:
        D, I, S = index.search(xq, k=K, batch=10240, return_scores=True)
    torch.cuda.synchronize()
    return xb, xq, index, D, I, S, st


def test_every_list_is_ordered_unique_and_screened(full):
    xb, xq, index, D, I, S, st = full
    assert st.dense_queries == 0 and st.survivors < NQ * 2048
    assert I.shape == (NQ, K) and int(I.min()) >= 0 and int(I.max()) < N
    assert bool((S[:, 1:] >= S[:, :-1]).all())
    tie = S[:, 1:] == S[:, :-1]
    assert bool((I[:, 1:][tie] > I[:, :-1][tie]).all())  # equal scores: ascending ids
    assert bool((torch.sort(I, dim=1).values[:, 1:] != torch.sort(I, dim=1).values[:, :-1]).all())
    assert torch.equal(D.double(), S.float().double())  # L2: the returned distance is the score, as float32
    # the scores are the exact squared distances of the returned rows
    rows = xb[I.reshape(-1)].reshape(NQ, K, 128).long()
    exact = ((rows - xq[:, None, :].long()) ** 2).sum(2).double()
    assert torch.equal(exact, S)


def test_rows_of_the_base_find_themselves(full):
    xb, _, index, *_ = full
    g = torch.Generator().manual_seed(7)
    pick = torch.randint(0, N, (2000,), generator=g).cuda()
    D, I, S = index.search(xb[pick].contiguous(), k=K, return_scores=True)
    assert bool((S[:, 0] == 0).all())
    assert bool((I[:, 0] <= pick).all())  # the row itself, or an identical row with a smaller id
    assert bool((xb[I[:, 0]] == xb[pick]).all())


def test_two_half_shards_merge_to_the_same_answer(full):
    xb, xq, _, _, I, S, _ = full
    q = xq[:500].contiguous()
    parts_s, parts_i = [], []
    for lo, hi in ((0, N // 2), (N // 2, N)):
        shard = certex.Index(128)
        shard.add(xb[lo:hi])
        _, i, s = shard.search(q, k=K, return_scores=True, id_base=lo)
        parts_s.append(s)
        parts_i.append(i)
        del shard
    _, Im, Sm = certex.merge_shards(q, torch.stack(parts_s), torch.stack(parts_i), "l2", return_scores=True)
    assert torch.equal(Im, I[:500]) and torch.equal(Sm, S[:500])


def test_a_sample_of_the_queries_against_the_oracle(full):
    xb, xq, _, _, I, S, _ = full
    pick = np.arange(0, NQ, NQ // 48)[:48]
    ids, scores = oracle.knn(xb.cpu().numpy(), xq[pick].cpu().numpy(), K, "l2")
    assert np.array_equal(I[pick].cpu().numpy(), ids) and np.array_equal(S[pick].cpu().numpy(), scores)
