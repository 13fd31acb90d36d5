"""The multi-process path on CPU: two gloo ranks, each answering for its contiguous row shard (the shard's exact
top-k comes from the CPU oracle here, since the test has no GPU), exchange their lists with the library's all-gather
and must end with the same merged answer as a search over the whole set."""

import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from libcertex_b200 import distributed
from oracle import oracle


def _rank(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)  # the same data on every rank
        x = rng.integers(0, 256, (3001, 24)).astype(np.uint8)
        q = rng.integers(0, 256, (17, 24)).astype(np.uint8)
        lo, hi = distributed.shard_bounds(len(x), world, rank)
        ids, scores = oracle.knn(x[lo:hi], q, 9, "l2", id_base=lo)
        all_s, all_i = distributed.gather_lists(torch.from_numpy(scores), torch.from_numpy(ids))
        assert tuple(all_s.shape) == (world, 17, 9) and int(all_i[rank, 0, 0]) == int(ids[0, 0])
        merged_i, merged_s = oracle.merge(all_i.numpy(), all_s.numpy())
        want_i, want_s = oracle.knn(x, q, 9, "l2")
        assert np.array_equal(merged_i, want_i) and np.array_equal(merged_s, want_s)
        np.save(os.path.join(out_dir, f"ok{rank}.npy"), merged_i)
    finally:
        dist.destroy_process_group()


def test_two_ranks_gather_and_merge(tmp_path):
    port = 29000 + os.getpid() % 2000
    mp.spawn(_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "ok0.npy"), np.load(tmp_path / "ok1.npy")
    assert np.array_equal(a, b)
