"""Row-sharded exact k-NN with one process per GPU (torch.distributed, NCCL over NVLink / NVSwitch).

The semantics are those of the reference's sharded search (cpp/src/neighbors/certex/certex_shards.cu:56-167): contiguous
row shards, rank s owns the global ids [n s / S, n (s + 1) / S), every rank computes the exact local top-k of all
queries, and the per-rank lists are merged by (exact score, id). The reference moves the lists through host memory and
sorts on the CPU; here every rank contributes k (fp64 score, int64 id) pairs per query to one all-gather and merges the
gathered lists with a device kernel. No kernel reads another GPU's memory.

Two ways of running the exchange: `backend="native"` (the default on GPUs) is one call into the library, which runs the
local search, ncclAllGather and the merge back to back on the stream over a communicator of its own and looks at the
device only once, at the end (certexB200DistributedSearch); `backend="torch"` runs the same three steps from Python
with torch.distributed's all_gather_into_tensor.
"""

import contextlib
import ctypes

import torch
import torch.distributed as dist

from . import _lib as L
from .index import Index, _need, merge_shards


class _DeviceInts:
    """int32 device memory that the library owns, seen through the CUDA array interface."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (int(n),), "typestr": "<i4", "data": (int(ptr), False), "version": 2}


@contextlib.contextmanager
def threshold_hook(fn):
    """Inside the block every unfiltered screened search of the calling thread hands `fn` its thresholds once per batch
    of queries, between the anchor pass and the screen: an int32 tensor of monotone keys (larger = tighter), one per
    query, each a score that k rows of the searched shard certainly reach. `fn` may raise them in place."""

    def call(_ctx, ptr, n, _stream):
        # the library runs on torch's current stream, which is where fn's work is enqueued
        fn(torch.as_tensor(_DeviceInts(ptr, n), device="cuda"))

    c_hook = L.ThresholdHook(call)
    L.check(L.lib().certexB200SetThresholdHook(c_hook, None))
    try:
        yield
    finally:
        L.check(L.lib().certexB200SetThresholdHook(ctypes.cast(None, L.ThresholdHook), None))


def shard_bounds(n, world, rank):
    """[lo, hi) of the rows of `rank` among `world` contiguous shards of n rows."""
    return n * rank // world, n * (rank + 1) // world


def gather_lists(scores, ids, group=None):
    """All-gather of per-rank answer lists: ([world, nq, k] scores, [world, nq, k] ids) on every rank. The fp64 scores
    travel as their int64 bit patterns next to the ids, so that one collective moves both."""
    world = dist.get_world_size(group)
    nq, k = scores.shape
    mine = torch.empty((2, nq, k), dtype=torch.int64, device=scores.device)
    mine[0] = scores.contiguous().view(torch.int64)
    mine[1] = ids
    both = torch.empty((world * 2 * nq, k), dtype=torch.int64, device=scores.device)  # rank-major concatenation
    dist.all_gather_into_tensor(both, mine.view(2 * nq, k), group=group)
    both = both.view(world, 2, nq, k)
    return both[:, 0].contiguous().view(torch.float64), both[:, 1].contiguous()


class _Ticket:
    """A sharded search between search_begin and search_end: the library's handle and the tensors it works on."""

    def __init__(self, pending, tensors, return_scores):
        self.pending, self.tensors, self.return_scores = pending, tensors, return_scores


class DistributedIndex:
    """One shard per rank of the process group. add_shard() takes this rank's rows and the global id of its first
    row; search() returns the same (distances, ids) on every rank.

    share_thresholds=True adds the reference's optional first round: between the anchor pass and the screen the ranks
    agree on thresholds. With the native backend and k <= 64 every rank contributes its k best threshold candidates per
    query and all take the k-th best of the union, which is what one index over all rows would screen with: the shards
    together then keep about as many pairs as one index would (80 per query and shard instead of 162 on the 10 M x 128
    benchmark with two shards, 41 with four). For larger k, and with backend="torch", the ranks take the maximum of
    their own thresholds (one all-reduce), which is hardly tighter than each of them. It is off by default because it
    ties the ranks together once more per batch of queries."""

    def __init__(self, dim, metric="l2", anchor_stride=16, group=None, share_thresholds=False, backend="native"):
        _need(backend in ("native", "torch"), "backend must be 'native' or 'torch'")
        self.d, self.metric, self.group, self.backend = dim, metric, group, backend
        self._comm = None  # the library's communicator over the ranks of `group` (native backend)
        self.local = Index(dim, metric=metric, anchor_stride=anchor_stride)
        self.first = 0
        self.share_thresholds = share_thresholds
        self._all_screen = {}  # k -> every rank's search for k neighbours goes through the screen

    def add_shard(self, rows, first_id):
        self.local.add(rows)
        self.first = int(first_id)
        self._all_screen.clear()
        return self

    def _shared(self, k):
        """Whether the ranks exchange thresholds for this k: the reference's first round (certex_shards.cu:136-141).
        Any k rows of one shard bound the k-th neighbour of the whole set, so every rank may screen with the tightest
        bound any rank found: the maximum of the keys, one all-reduce of n_queries int32 per batch. It needs every rank
        to reach the hook, i.e. to screen; that is agreed once per k."""
        if not self.share_thresholds or dist.get_world_size(self.group) == 1:
            return False
        if k not in self._all_screen:
            mine = ctypes.c_int32(0)
            L.check(L.lib().certexB200IndexWillScreen(self.local.core.handle, int(k), ctypes.byref(mine)))
            flag = torch.tensor([mine.value], dtype=torch.int32, device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            self._all_screen[k] = bool(flag.item())
        return self._all_screen[k]

    def add(self, x):
        """x: the full set (same array on every rank); this rank keeps its contiguous shard."""
        lo, hi = shard_bounds(x.shape[0], dist.get_world_size(self.group), dist.get_rank(self.group))
        return self.add_shard(x[lo:hi], lo)

    def __del__(self):
        if getattr(self, "_comm", None) is not None and L is not None:  # L is None while the interpreter shuts down
            L.lib().certexB200CommDestroy(self._comm)
            self._comm = None

    def _communicator(self):
        """The library's NCCL communicator over the ranks of the group: rank 0 makes the id, the process group carries
        it to the others (once)."""
        if self._comm is None:
            world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
            ident = ctypes.create_string_buffer(128)
            if rank == 0:
                L.check(L.lib().certexB200CommGetUniqueId(ident))
            box = [ident.raw]
            dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0) if self.group else 0, group=self.group)
            ident = ctypes.create_string_buffer(box[0], 128)
            comm = ctypes.c_void_p()
            L.check(L.lib().certexB200CommInitRank(ident, world, rank, ctypes.byref(comm)))
            self._comm = comm
        return self._comm

    def _search_native(self, Q, k, batch, return_scores):
        return self.search_end(self._begin_native(Q, k, batch, return_scores))

    def _begin_native(self, Q, k, batch, return_scores):
        nq = Q.shape[0]
        I = torch.empty((nq, k), dtype=torch.int64, device="cuda")
        D = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        S = torch.empty((nq, k), dtype=torch.float64, device="cuda") if return_scores else None
        sp = L.SearchParams(128, int(batch), 2)
        tensors = (L.Tensor(Q), L.Tensor(I), L.Tensor(D), None if S is None else L.Tensor(S))
        pending = ctypes.c_void_p()
        L.check(L.lib().certexB200DistributedSearchBegin(
            L.resources(), self._communicator(), ctypes.byref(sp), self.local.core.handle, tensors[0].ref, tensors[1].ref,
            tensors[2].ref, None if S is None else tensors[3].ref, self.first, 1 if self.share_thresholds else 0,
            ctypes.byref(pending)))
        return _Ticket(pending, (Q, I, D, S), return_scores)

    def search_begin(self, q, k=10, batch=2048, return_scores=False):
        """First half of search() (native backend): enqueues the local search, the exchange and the merge on the current
        stream and returns a ticket without waiting for the device. Up to two searches may be between search_begin and
        search_end; they end in the order they began, and every rank makes the same sequence of calls. A caller that
        begins the next search before it ends this one keeps the device busy while the host prepares the next call."""
        _need(self.backend == "native", "search_begin needs the native backend")
        _need(self.local.core is not None, "add vectors first")
        _need(k <= int(self.local.core.info().size), "every shard needs at least k vectors")
        return self._begin_native(q.cuda().contiguous().to(self.local.dtype), k, batch, return_scores)

    def search_end(self, ticket):
        """Second half: waits for that search (not for work enqueued behind it), lets the library repair and exchange
        again if a candidate list had overflowed on some rank, and returns what search() returns."""
        _need(ticket.pending is not None, "this search was ended already")
        pending, ticket.pending = ticket.pending, None
        L.check(L.lib().certexB200DistributedSearchEnd(pending))
        _, I, D, S = ticket.tensors
        if self.metric == "cosine":
            D = 1 - D
        return (D, I, S) if ticket.return_scores else (D, I)

    def search(self, q, k=10, batch=2048, return_scores=False):
        _need(self.local.core is not None, "add vectors first")
        _need(k <= int(self.local.core.info().size), "every shard needs at least k vectors")
        Q = q.cuda().contiguous()
        if self.backend == "native":
            return self._search_native(Q.to(self.local.dtype), k, batch, return_scores)
        if self._shared(k):
            with threshold_hook(lambda keys: dist.all_reduce(keys, op=dist.ReduceOp.MAX, group=self.group)):
                _, I, S = self.local.search(Q, k=k, batch=batch, return_scores=True, id_base=self.first)
        else:
            _, I, S = self.local.search(Q, k=k, batch=batch, return_scores=True, id_base=self.first)
        all_s, all_i = gather_lists(S, I, self.group)
        return merge_shards(Q.to(self.local.dtype), all_s, all_i, self.metric, return_scores=return_scores)
