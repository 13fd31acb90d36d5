"""Row-sharded exact k-NN with one process per GPU (torch.distributed, NCCL over NVLink / NVSwitch).

The semantics are those of the reference's sharded search (cpp/src/neighbors/certex/certex_shards.cu:56-167): contiguous
row shards, rank s owns the global ids [n s / S, n (s + 1) / S), every rank computes the exact local top-k of all
queries, and the per-rank lists are merged by (exact score, id). The reference moves the lists through host memory and
sorts on the CPU; here every rank contributes k (fp64 score, int64 id) pairs per query to one all-gather and merges the
gathered lists with a device kernel. No kernel reads another GPU's memory.
"""

import torch
import torch.distributed as dist

from .index import Index, _need, merge_shards


def shard_bounds(n, world, rank):
    """[lo, hi) of the rows of `rank` among `world` contiguous shards of n rows."""
    return n * rank // world, n * (rank + 1) // world


def gather_lists(scores, ids, group=None):
    """All-gather of per-rank answer lists: ([world, nq, k] scores, [world, nq, k] ids) on every rank."""
    world = dist.get_world_size(group)
    nq, k = scores.shape
    all_s = torch.empty((world * nq, k), dtype=scores.dtype, device=scores.device)  # rank-major concatenation
    all_i = torch.empty((world * nq, k), dtype=ids.dtype, device=ids.device)
    dist.all_gather_into_tensor(all_s, scores.contiguous(), group=group)
    dist.all_gather_into_tensor(all_i, ids.contiguous(), group=group)
    return all_s.view(world, nq, k), all_i.view(world, nq, k)


class DistributedIndex:
    """One shard per rank of the process group. add_shard() takes this rank's rows and the global id of its first
    row; search() returns the same (distances, ids) on every rank."""

    def __init__(self, dim, metric="l2", anchor_stride=16, group=None):
        self.d, self.metric, self.group = dim, metric, group
        self.local = Index(dim, metric=metric, anchor_stride=anchor_stride)
        self.first = 0

    def add_shard(self, rows, first_id):
        self.local.add(rows)
        self.first = int(first_id)
        return self

    def add(self, x):
        """x: the full set (same array on every rank); this rank keeps its contiguous shard."""
        lo, hi = shard_bounds(x.shape[0], dist.get_world_size(self.group), dist.get_rank(self.group))
        return self.add_shard(x[lo:hi], lo)

    def search(self, q, k=10, batch=2048, return_scores=False):
        _need(self.local.core is not None, "add vectors first")
        _need(k <= int(self.local.core.info().size), "every shard needs at least k vectors")
        Q = q.cuda().contiguous()
        _, I, S = self.local.search(Q, k=k, batch=batch, return_scores=True, id_base=self.first)
        all_s, all_i = gather_lists(S, I, self.group)
        return merge_shards(Q.to(self.local.dtype), all_s, all_i, self.metric, return_scores=return_scores)
