"""ExactTopK / top_k (the FlashInfer-style selection) against the CPU oracle: every (row, query head) pair must get
exactly the positions of the k largest fp64 inner products within its own sequence and KV head, ties to the smaller
position. The scenarios are those of the reference's tests/test_flashinfer.py: three sequences in named slots fed in
steps, one shorter than k; ragged offsets; a shuffled page table; single-head rows; released slots; one-call top_k."""

import numpy as np
import pytest
import torch

from libcertex_b200 import flashinfer as fi
from oracle import oracle

pytestmark = pytest.mark.gpu
KV, H, D = 2, 4, 64


def rand(*shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).half()


def want_positions(keys, q_row, k):
    """[H, k] positions for one row q_row [H, D] over keys [n, KV, D]."""
    out = np.empty((H, k), dtype=np.int64)
    for h in range(H):
        ids, _ = oracle.knn(keys[:, h // (H // KV)].numpy(), q_row[h][None].numpy(), k, "ip")
        out[h] = ids[0]
    return out


def batch(k_max=256):
    """Slots 7, 3, 5 at batch positions 0, 1, 2; the last holds fewer keys than k."""
    lens = [9000, 5000, 100]
    keys = [rand(n, KV, D, seed=s) for s, n in enumerate(lens)]
    sel = fi.ExactTopK(KV, D, k_max=k_max)
    for slot, K in zip((7, 3, 5), keys):
        for s in range(0, K.shape[0], 2500):  # keys arrive in steps
            sel.append(slot, K[s : s + 2500].cuda())
    rows = torch.tensor([0, 0, 1, 2, 1, 0])
    q = rand(rows.numel(), H, D, seed=9)
    return sel, keys, rows, q, torch.tensor([7, 3, 5])


def test_ragged_transform_is_exact_per_sequence_and_head():
    sel, keys, rows, q, slots = batch()
    assert sel.length(7) == 9000 and sel.length(5) == 100 and sel.length(11) == 0
    offsets = torch.tensor([0, 1000, 2000, 3000, 4000, 5000], dtype=torch.int32)
    out = sel.ragged_transform(q.cuda(), offsets.cuda(), 128, row_to_batch=rows.cuda(), slots=slots)
    assert out.shape == (6, H, 128) and out.dtype == torch.int32
    out = out.cpu()
    for i in range(6):
        b = int(rows[i])
        if b == 2:  # 100 keys < k: all of them in order, then -1
            assert bool((out[i, :, 100:] == -1).all())
            assert bool((out[i, :, :100] - offsets[i] == torch.arange(100)).all())
        else:
            assert np.array_equal((out[i] - offsets[i]).numpy(), want_positions(keys[b], q[i], 128))


def test_page_table_transform_points_at_the_physical_keys():
    sel, keys, rows, q, slots = batch()
    ps = 16
    pages = [(K.shape[0] + ps - 1) // ps for K in keys]
    perm = torch.randperm(sum(pages), generator=torch.Generator().manual_seed(1))
    table = torch.full((3, max(pages)), -1, dtype=torch.int32)
    start = 0
    for b in range(3):
        table[b, : pages[b]] = perm[start : start + pages[b]].int()
        start += pages[b]
    out = sel.page_table_transform(q.cuda(), table.cuda(), 64, row_to_batch=rows.cuda(), slots=slots, page_size=ps).cpu()
    for i in range(6):
        b = int(rows[i])  # k = 64 is below every sequence's length: the 100-key sequence is searched too
        local = torch.from_numpy(want_positions(keys[b], q[i], 64))
        assert bool((out[i].long() == table[b, local // ps].long() * ps + local % ps).all())


def test_single_head_rows_and_default_batch_positions():
    keys = rand(12000, 1, D, seed=4)
    q = rand(8, D, seed=5)
    sel = fi.ExactTopK(1, D, k_max=64).append(0, keys.cuda())
    out = sel.ragged_transform(q.cuda(), torch.zeros(8, dtype=torch.int32), 64, row_to_batch=torch.zeros(8, dtype=torch.long))
    assert out.shape == (8, 64)
    ids, _ = oracle.knn(keys[:, 0].numpy(), q.numpy(), 64, "ip")
    assert np.array_equal(out.cpu().numpy(), ids)
    # without row_to_batch, row i reads slot i
    for s in range(1, 3):
        sel.append(s, rand(3000, 1, D, seed=10 + s).cuda())
    out = sel.select(q[:3].cuda(), 10).cpu().numpy()
    for s in range(3):
        K = keys[:, 0] if s == 0 else rand(3000, 1, D, seed=10 + s)[:, 0]
        ids, _ = oracle.knn(K.numpy(), q[s][None].numpy(), 10, "ip")
        assert np.array_equal(out[s], ids[0])


def test_released_slot_is_gone_and_its_name_starts_again():
    sel, keys, rows, q, slots = batch(k_max=32)
    sel.release(7)
    assert sel.length(7) == 0
    with pytest.raises(Exception):
        sel.select(q.cuda(), 8, row_to_batch=rows.cuda(), slots=slots)
    fresh = rand(4000, KV, D, seed=20)
    sel.append(7, fresh.cuda())
    out = sel.select(q.cuda(), 32, row_to_batch=rows.cuda(), slots=slots).cpu().numpy()
    for i in range(6):
        b = int(rows[i])
        K = fresh if b == 0 else keys[b]
        assert np.array_equal(out[i], want_positions(K, q[i], 32))


def test_top_k_one_call():
    keys = rand(20000, D, seed=6)
    q = rand(16, D, seed=7)
    values, indices = fi.top_k(q.cuda().bfloat16(), keys.cuda(), 32)
    assert values.shape == indices.shape == (16, 32) and indices.dtype == torch.int64
    ids, _ = oracle.knn(keys.numpy(), q.bfloat16().half().numpy(), 32, "ip")
    assert np.array_equal(indices.cpu().numpy(), ids)
    ip = torch.einsum("md,mkd->mk", q.bfloat16().double(), keys.double()[indices.cpu()])
    assert torch.allclose(values.cpu().double(), ip, rtol=1e-3, atol=1e-3)
