"""Row-sharded search: several shards (on the available devices, round-robin as the reference's tests do,
cpp/tests/neighbors/ann_certex/test_shards.cu:21-24) must return exactly what one index over all vectors returns, for
every metric; the device merge must equal the oracle's merge; and, when two GPUs are present, one process per GPU
over NCCL."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from libcertex_b200 import synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("n_shards,metric,dtype", [(2, "l2", "uint8"), (3, "l2", "uint8"), (5, "ip", "int8"),
                                                   (3, "cosine", "float32"), (2, "ip", "float32")])
def test_shards_equal_one_index(n_shards, metric, dtype):
    x = synthetic.correlated(30011, 64, seed=11, dtype=dtype, unequal_norms=metric != "l2")
    q = synthetic.correlated(150, 64, seed=12, dtype=dtype)
    devices = [s % torch.cuda.device_count() for s in range(n_shards)]
    sharded = certex.ShardedIndex(64, devices, metric=metric)
    sharded.add(x)
    D, I = sharded.search(q, k=10)
    ids, scores = oracle.knn(x, q, 10, metric)
    assert np.array_equal(I, ids)


def test_device_merge_equals_oracle_merge_with_missing_entries():
    rng = np.random.default_rng(0)
    parts, nq, k = 4, 50, 16
    s = np.sort(rng.integers(0, 40, (parts, nq, k)).astype(np.float64), axis=2)  # many ties across parts
    i = rng.permutation(parts * nq * k).reshape(parts, nq, k).astype(np.int64)
    i[1, :, 10:] = -1  # a shard with fewer than k admitted vectors
    s[1, :, 10:] = np.inf
    q = torch.zeros((nq, 8), dtype=torch.float32, device="cuda")
    D, I, S = certex.merge_shards(q, torch.from_numpy(s).cuda(), torch.from_numpy(i).cuda(), "l2", return_scores=True)
    wi, ws = oracle.merge(i, s)
    assert np.array_equal(I.cpu().numpy(), wi) and np.array_equal(S.cpu().numpy(), ws)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_per_gpu_over_nccl(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(
        "import os, sys, numpy as np, torch, torch.distributed as dist\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "from libcertex_b200 import distributed, synthetic\n"
        "from oracle import oracle\n"
        "rank = int(os.environ['RANK']); torch.cuda.set_device(int(os.environ['LOCAL_RANK']))\n"
        "dist.init_process_group('nccl')\n"
        "x = synthetic.correlated(40000, 32, seed=3, dtype='uint8'); q = synthetic.correlated(100, 32, seed=4, dtype='uint8')\n"
        "idx = distributed.DistributedIndex(32).add(torch.from_numpy(x))\n"
        "D, I, S = idx.search(torch.from_numpy(q), k=10, return_scores=True)\n"
        "ids, scores = oracle.knn(x, q, 10, 'l2')\n"
        "assert np.array_equal(I.cpu().numpy(), ids) and np.array_equal(S.cpu().numpy(), scores)\n"
        "dist.barrier(); dist.destroy_process_group(); print('rank', rank, 'ok')\n"
    )
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29577", str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
