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


@pytest.mark.parametrize("dtype,metric", [("uint8", "l2"), ("float32", "l2"), ("float32", "cosine"), ("int8", "ip")])
def test_thresholds_exchanged_between_shards(dtype, metric):
    """The exchange a process group does with one all-reduce, replayed on one GPU: two shards, every shard's
    thresholds raised to the maximum over both. The merged answer stays exact and fewer pairs survive the screens."""
    from libcertex_b200 import distributed

    x = synthetic.correlated(60000, 48, seed=21, dtype=dtype, unequal_norms=metric != "l2")
    q = synthetic.correlated(300, 48, seed=22, dtype=dtype)
    xt, qt = torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda()
    shards = [certex.Index(48, metric=metric), certex.Index(48, metric=metric)]
    shards[0].add(xt[:30000])
    shards[1].add(xt[30000:])
    seen = [None, None]

    def search_all(exchange):
        lists, survivors = [], 0
        for s, index in enumerate(shards):
            def hook(keys, s=s):
                if exchange:
                    keys.copy_(torch.maximum(keys, seen[1 - s]))
                else:
                    seen[s] = keys.clone()
            with distributed.threshold_hook(hook), certex.search_stats() as st:
                _, I, S = index.search(qt, k=10, return_scores=True, id_base=30000 * s)
            assert st.dense_queries == 0
            survivors += st.survivors
            lists.append((S, I))
        S = torch.stack([l[0] for l in lists])
        I = torch.stack([l[1] for l in lists])
        _, Im, Sm = certex.merge_shards(qt, S, I, metric, return_scores=True)
        return Im.cpu().numpy(), Sm.cpu().numpy(), survivors

    ids, scores = oracle.knn(x, q, 10, metric)
    I0, S0, n0 = search_all(exchange=False)
    assert seen[0] is not None and seen[0].shape == (300,) and seen[0].dtype == torch.int32
    I1, S1, n1 = search_all(exchange=True)
    assert np.array_equal(I0, ids) and np.array_equal(S0, scores)
    assert np.array_equal(I1, ids) and np.array_equal(S1, scores)
    assert n1 < n0
    with certex.search_stats() as st:  # the hook is gone after the block
        shards[0].search(qt, k=10)
    assert st.survivors > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_per_gpu_over_nccl(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(
        "import os, sys, numpy as np, torch, torch.distributed as dist\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "import libcertex_b200 as certex\n"
        "from libcertex_b200 import distributed, synthetic\n"
        "from oracle import oracle\n"
        "rank = int(os.environ['RANK']); torch.cuda.set_device(int(os.environ['LOCAL_RANK']))\n"
        "dist.init_process_group('nccl')\n"
        "x = synthetic.correlated(40000, 32, seed=3, dtype='uint8'); q = synthetic.correlated(100, 32, seed=4, dtype='uint8')\n"
        "ids, scores = oracle.knn(x, q, 10, 'l2')\n"
        "for backend in ('native', 'torch'):\n"
        "    idx = distributed.DistributedIndex(32, share_thresholds=True, backend=backend).add(torch.from_numpy(x))\n"
        "    D, I, S = idx.search(torch.from_numpy(q), k=10, return_scores=True)\n"
        "    assert np.array_equal(I.cpu().numpy(), ids) and np.array_equal(S.cpu().numpy(), scores), backend\n"
        "    D2, I2 = idx.search(torch.from_numpy(q), k=10)\n"
        "    assert torch.equal(I2, I) and torch.equal(D2, D)\n"
        "    # candidate lists that overflow on purpose (capacity 16 for k = 10): the repair and the second exchange\n"
        "    idx.local._test_mode(2, 16)\n"
        "    D, I, S = idx.search(torch.from_numpy(q), k=10, return_scores=True)\n"
        "    assert np.array_equal(I.cpu().numpy(), ids) and np.array_equal(S.cpu().numpy(), scores), backend + ' overflow'\n"
        "xf = synthetic.correlated(40000, 96, seed=5, dtype='float32'); qf = synthetic.correlated(100, 96, seed=6, dtype='float32')\n"
        "ids, scores = oracle.knn(xf, qf, 20, 'cosine')\n"
        "for backend in ('native', 'torch'):\n"
        "    for share in (True, False):\n"
        "        fidx = distributed.DistributedIndex(96, metric='cosine', share_thresholds=share, backend=backend).add(torch.from_numpy(xf))\n"
        "        D, I, S = fidx.search(torch.from_numpy(qf), k=20, return_scores=True)\n"
        "        assert np.array_equal(I.cpu().numpy(), ids) and np.array_equal(S.cpu().numpy(), scores), (backend, share)\n"
        "# the exchange of thresholds: for k <= 64 the shards pool their k largest group values, beyond that they take the\n"
        "# maximum of their thresholds; either way exact, and fewer pairs survive the screens than without an exchange\n"
        "xu = synthetic.mixture_u8(400000, seed=9).cpu().numpy(); qu = synthetic.mixture_u8(200, seed=10).cpu().numpy()\n"
        "for k in (10, 100):\n"
        "    ids, scores = oracle.knn(xu, qu, k, 'l2')\n"
        "    kept = {}\n"
        "    for share in (False, True):\n"
        "        uidx = distributed.DistributedIndex(128, share_thresholds=share).add(torch.from_numpy(xu))\n"
        "        with certex.search_stats() as st:\n"
        "            D, I, S = uidx.search(torch.from_numpy(qu), k=k, return_scores=True)\n"
        "        assert np.array_equal(I.cpu().numpy(), ids) and np.array_equal(S.cpu().numpy(), scores), (k, share)\n"
        "        assert st.dense_queries == 0\n"
        "        kept[share] = st.survivors\n"
        "    assert kept[True] < kept[False], (k, kept)\n"
        "    if k == 10: assert kept[True] < 0.8 * kept[False], kept\n"
        "# two searches between search_begin and search_end (different queries and k), ended in order; then with candidate\n"
        "# lists that overflow on the last rank only: the second round of the first search then runs behind the second\n"
        "# search, which has reused the exchange buffers, and the other ranks write their lists there once more\n"
        "pidx = distributed.DistributedIndex(32, share_thresholds=True).add(torch.from_numpy(x))\n"
        "qa, qb = torch.from_numpy(q[:60]), torch.from_numpy(q[40:])\n"
        "want_a, want_b = oracle.knn(x, q[:60], 10, 'l2'), oracle.knn(x, q[40:], 7, 'l2')\n"
        "for overflow in (False, True):\n"
        "    if overflow and rank == dist.get_world_size() - 1: pidx.local._test_mode(2, 16)\n"
        "    ta = pidx.search_begin(qa, k=10, return_scores=True)\n"
        "    tb = pidx.search_begin(qb, k=7, return_scores=True)\n"
        "    try:\n"
        "        pidx.search_begin(qa, k=10); raise SystemExit('a third search in flight was accepted')\n"
        "    except certex.CertexError as e:\n"
        "        assert 'in flight' in str(e), str(e)\n"
        "    Da, Ia, Sa = pidx.search_end(ta)\n"
        "    Db, Ib, Sb = pidx.search_end(tb)\n"
        "    assert np.array_equal(Ia.cpu().numpy(), want_a[0]) and np.array_equal(Sa.cpu().numpy(), want_a[1]), overflow\n"
        "    assert np.array_equal(Ib.cpu().numpy(), want_b[0]) and np.array_equal(Sb.cpu().numpy(), want_b[1]), overflow\n"
        "    D1, I1 = pidx.search(qa, k=10)\n"
        "    assert torch.equal(I1, Ia) and torch.equal(D1, Da)\n"
        "# (lists still overflow) a later, larger search makes the library replace its exchange buffers while the first\n"
        "# search is still to be ended: its second round writes to the new ones\n"
        "want_all = oracle.knn(x, q, 10, 'l2')\n"
        "tb = pidx.search_begin(qb, k=7, return_scores=True)\n"
        "tc = pidx.search_begin(torch.from_numpy(q), k=10, return_scores=True)\n"
        "Db, Ib, Sb = pidx.search_end(tb)\n"
        "Dc, Ic, Sc = pidx.search_end(tc)\n"
        "assert np.array_equal(Ib.cpu().numpy(), want_b[0]) and np.array_equal(Sb.cpu().numpy(), want_b[1])\n"
        "assert np.array_equal(Ic.cpu().numpy(), want_all[0]) and np.array_equal(Sc.cpu().numpy(), want_all[1])\n"
        "# a rank whose local search fails (a host-side simulated allocation failure on rank 1, one query so that no\n"
        "# halving helps): every rank gets an error for the call instead of waiting, and the next call works\n"
        "idx = distributed.DistributedIndex(32).add(torch.from_numpy(x))\n"
        "if rank == 1: idx.local._test_mode(4, 0)\n"
        "try:\n"
        "    idx.search(torch.from_numpy(q[:1]), k=10); raise SystemExit('no error on rank %d' % rank)\n"
        "except certex.CertexError as e:\n"
        "    assert ('rank 1 failed' in str(e)) if rank == 0 else ('out of device memory' in str(e)), str(e)\n"
        "idx.local._test_mode(0, 0)\n"
        "D, I = idx.search(torch.from_numpy(q), k=10)\n"
        "assert np.array_equal(I.cpu().numpy(), oracle.knn(x, q, 10, 'l2')[0])\n"
        "dist.barrier(); dist.destroy_process_group(); print('rank', rank, 'ok')\n"
    )
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29577", str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-8000:]


def test_two_searches_in_flight_on_a_communicator_of_one_rank(tmp_path):
    """The two-call form of the sharded search on one GPU: a process group and a communicator of a single rank. Two
    searches are begun before the first is ended, once plainly and once with candidate lists that overflow, whose
    repair and second exchange then run behind the second search."""
    script = tmp_path / "one_rank.py"
    script.write_text(
        "import os, sys, numpy as np, torch, torch.distributed as dist\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "import libcertex_b200 as certex\n"
        "from libcertex_b200 import distributed, synthetic\n"
        "from oracle import oracle\n"
        "rank = 0; torch.cuda.set_device(0)\n"
        "dist.init_process_group('nccl', rank=0, world_size=1)\n"
        "x = synthetic.correlated(40000, 32, seed=3, dtype='uint8'); q = synthetic.correlated(100, 32, seed=4, dtype='uint8')\n"
        "# two searches between search_begin and search_end (different queries and k), ended in order; then with candidate\n"
        "# lists that overflow on the last rank only: the second round of the first search then runs behind the second\n"
        "# search, which has reused the exchange buffers, and the other ranks write their lists there once more\n"
        "pidx = distributed.DistributedIndex(32, share_thresholds=True).add(torch.from_numpy(x))\n"
        "qa, qb = torch.from_numpy(q[:60]), torch.from_numpy(q[40:])\n"
        "want_a, want_b = oracle.knn(x, q[:60], 10, 'l2'), oracle.knn(x, q[40:], 7, 'l2')\n"
        "for overflow in (False, True):\n"
        "    if overflow and rank == dist.get_world_size() - 1: pidx.local._test_mode(2, 16)\n"
        "    ta = pidx.search_begin(qa, k=10, return_scores=True)\n"
        "    tb = pidx.search_begin(qb, k=7, return_scores=True)\n"
        "    try:\n"
        "        pidx.search_begin(qa, k=10); raise SystemExit('a third search in flight was accepted')\n"
        "    except certex.CertexError as e:\n"
        "        assert 'in flight' in str(e), str(e)\n"
        "    Da, Ia, Sa = pidx.search_end(ta)\n"
        "    Db, Ib, Sb = pidx.search_end(tb)\n"
        "    assert np.array_equal(Ia.cpu().numpy(), want_a[0]) and np.array_equal(Sa.cpu().numpy(), want_a[1]), overflow\n"
        "    assert np.array_equal(Ib.cpu().numpy(), want_b[0]) and np.array_equal(Sb.cpu().numpy(), want_b[1]), overflow\n"
        "    D1, I1 = pidx.search(qa, k=10)\n"
        "    assert torch.equal(I1, Ia) and torch.equal(D1, Da)\n"
        "# (lists still overflow) a later, larger search makes the library replace its exchange buffers while the first\n"
        "# search is still to be ended: its second round writes to the new ones\n"
        "want_all = oracle.knn(x, q, 10, 'l2')\n"
        "tb = pidx.search_begin(qb, k=7, return_scores=True)\n"
        "tc = pidx.search_begin(torch.from_numpy(q), k=10, return_scores=True)\n"
        "Db, Ib, Sb = pidx.search_end(tb)\n"
        "Dc, Ic, Sc = pidx.search_end(tc)\n"
        "assert np.array_equal(Ib.cpu().numpy(), want_b[0]) and np.array_equal(Sb.cpu().numpy(), want_b[1])\n"
        "assert np.array_equal(Ic.cpu().numpy(), want_all[0]) and np.array_equal(Sc.cpu().numpy(), want_all[1])\n"
        "dist.destroy_process_group(); print('ok')\n"
    )
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29579")
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-8000:]
