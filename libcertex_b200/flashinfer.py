"""Exact top-k key selection for sparse attention with the call surface of the reference's certex/flashinfer.py
(`ExactTopK` 50-126, `top_k` 129-138): the positions FlashInfer's top_k_ragged_transform / top_k_page_table_transform
would return, computed from the queries and the keys instead of from a score matrix, exact by fp64 inner product with
ties to the smaller position.

The reference keeps one index per KV head and sequence slot and loops over them in Python. Here every key of every
slot and head lives in ONE labeled inner-product index (label = slot number * num_kv_heads + KV head), so that one
search call answers all rows of a batch: each (row, query head) pair is screened and scored against the keys of its
own sequence and head only. The ragged and page-table translations are elementwise device operations on the result.

Layouts follow FlashInfer (NHD): keys (n, num_kv_heads, head_dim); q (num_rows, num_qo_heads, head_dim), or
(num_rows, head_dim) for one head. Row i belongs to batch position row_to_batch[i] (default i), whose keys are those of
slot slots[row_to_batch[i]] (default the batch position). Positions beyond a sequence shorter than k are -1.
"""

import torch

from .attention import GrowingMap, _as_half_or_float
from .index import Index, _need


def _tensor(a):
    if isinstance(a, torch.Tensor):
        return a
    if hasattr(a, "__dlpack__"):
        return torch.from_dlpack(a)
    return torch.as_tensor(a, device="cuda")


class ExactTopK:
    """num_kv_heads, head_dim: the shape of the keys. k_max: the largest k a selection will ask for. capacity: the
    expected number of keys over all slots and heads together divided by num_kv_heads (reserves memory once)."""

    def __init__(self, num_kv_heads, head_dim, k_max=2048, capacity=None):
        _need(1 <= k_max <= 2048, f"k_max must be between 1 and 2048, not {k_max}")
        _need(num_kv_heads >= 1 and head_dim >= 1, "num_kv_heads and head_dim must be positive")
        self.num_kv_heads, self.head_dim, self.k_max = int(num_kv_heads), int(head_dim), int(k_max)
        self.capacity = capacity
        self.index, self.dtype = None, None
        self._map = GrowingMap(torch.int32)  # id of the index -> position of the key inside its sequence
        self._number = {}       # slot -> its number (labels number * num_kv_heads + head)
        self._next = 0          # numbers are never reused: the labels of removed rows stay theirs
        self._length = {}       # slot -> keys appended
        self._ids = {}          # slot -> list of (first id, count) ranges of the index

    # ------------------------------------------------------------------------------------------------ keys
    def append(self, slot, keys):
        """Append keys of shape (n, num_kv_heads, head_dim) to a sequence slot; positions continue."""
        K = _tensor(keys)
        _need(K.ndim == 3 and K.shape[1] == self.num_kv_heads and K.shape[2] == self.head_dim,
              f"keys must have shape (n, {self.num_kv_heads}, {self.head_dim}), not {tuple(K.shape)}")
        K = _as_half_or_float(K)
        n_new = K.shape[0]
        if n_new == 0:
            return self
        if self.index is None:
            self.dtype = K.dtype
            cap = None if self.capacity is None else int(self.capacity) * self.num_kv_heads
            self.index = Index(self.head_dim, metric="ip", capacity=cap, partition_labels="lazy")
        _need(not (self.dtype == torch.float16 and K.dtype == torch.float32),
              "these keys do not fit float16 but the selector was started with float16 keys: start it with float32 keys")
        if slot not in self._number:
            self._number[slot], self._next = self._next, self._next + 1
            self._length[slot], self._ids[slot] = 0, []
        base = self._number[slot] * self.num_kv_heads
        # head-major rows: the keys of one (slot, head) label are adjacent and in position order
        rows = K.to(self.dtype).transpose(0, 1).reshape(self.num_kv_heads * n_new, self.head_dim).contiguous()
        labels = (base + torch.arange(self.num_kv_heads, dtype=torch.int32, device="cuda")).repeat_interleave(n_new)
        first = len(self._map)
        self.index.add(rows, labels=labels)
        at = self._length[slot]
        pos = torch.arange(at, at + n_new, dtype=torch.int32, device="cuda").repeat(self.num_kv_heads)
        self._map.append(pos, reserve=0 if self.capacity is None else int(self.capacity) * self.num_kv_heads)
        self._ids[slot].append((first, self.num_kv_heads * n_new))
        self._length[slot] = at + n_new
        return self

    def release(self, slot):
        """Forget the keys of a finished sequence (their rows are removed from the index; a slot of the same name
        starts again at position 0)."""
        if slot not in self._number:
            return
        ranges = self._ids.pop(slot)
        ids = torch.cat([torch.arange(a, a + c, dtype=torch.int64, device="cuda") for a, c in ranges])
        self.index.remove(ids)
        del self._number[slot], self._length[slot]

    def length(self, slot):
        return self._length.get(slot, 0)

    # ------------------------------------------------------------------------------------------------ selection
    def select(self, q, k, row_to_batch=None, slots=None):
        """The exact top-k positions of every query row within its sequence: int32 (num_rows, num_qo_heads, k), or
        (num_rows, k) for single-head rows; all positions (ascending) then -1 where a sequence has at most k keys."""
        _need(1 <= k <= self.k_max, f"k must be between 1 and k_max={self.k_max}, not {k}")
        Q = _tensor(q)
        single = Q.ndim == 2
        if single:
            Q = Q[:, None, :]
        _need(Q.ndim == 3 and Q.shape[2] == self.head_dim and Q.shape[1] % self.num_kv_heads == 0,
              f"q must have shape (num_rows, num_qo_heads, {self.head_dim}) with num_qo_heads a multiple of "
              f"{self.num_kv_heads}, or (num_rows, {self.head_dim})")
        R, H, d = Q.shape
        group = H // self.num_kv_heads
        b = list(range(R)) if row_to_batch is None else [int(v) for v in _tensor(row_to_batch).reshape(-1).tolist()]
        _need(len(b) == R, "row_to_batch needs one entry per query row")
        slot_of = [(v if slots is None else int(slots[v])) for v in b]
        for s in set(slot_of):
            _need(s in self._length, f"slot {s} has no keys: append them first")
        number = torch.tensor([self._number[s] for s in slot_of], dtype=torch.int32, device="cuda")
        length = torch.tensor([self._length[s] for s in slot_of], dtype=torch.int32, device="cuda")
        out = torch.full((R, H, k), -1, dtype=torch.int32, device="cuda")
        # short sequences: every position is selected, as in FlashInfer
        short = length <= k
        if bool(short.any()):
            ar = torch.arange(k, dtype=torch.int32, device="cuda")
            fill = torch.where(ar[None, :] < length[short][:, None], ar[None, :], torch.full_like(ar, -1)[None, :])
            out[short] = fill[:, None, :].expand(-1, H, -1)
        rows = torch.nonzero(~short).flatten()
        if rows.numel() > 0:
            head = torch.arange(H, dtype=torch.int32, device="cuda") // group
            labels = (number[rows][:, None] * self.num_kv_heads + head[None, :]).reshape(-1).contiguous()
            Qs = _as_half_or_float(Q[rows])
            _need(not (self.dtype == torch.float16 and Qs.dtype == torch.float32),
                  "these queries do not fit float16 but the selector holds float16 keys: start it with float32 keys")
            Qs = Qs.to(self.dtype).reshape(rows.numel() * H, d).contiguous()
            _, I = self.index.search(Qs, k=k, labels=labels)
            out[rows] = self._map.values[I.clamp_(min=0)].reshape(rows.numel(), H, k)
        return out[:, 0] if single else out

    def ragged_transform(self, q, offsets, k, row_to_batch=None, slots=None):
        """flashinfer.top_k_ragged_transform from queries: the exact top-k positions plus offsets[i] for row i."""
        local = self.select(q, k, row_to_batch, slots)
        off = _tensor(offsets).to(local.device).to(torch.int32).reshape(-1, *([1] * (local.ndim - 1)))
        return torch.where(local >= 0, local + off, local)

    def page_table_transform(self, q, src_page_table, k, row_to_batch=None, slots=None, page_size=1):
        """flashinfer.top_k_page_table_transform from queries: position p of row i becomes the physical position
        src_page_table[row_to_batch[i], p // page_size] * page_size + p % page_size."""
        local = self.select(q, k, row_to_batch, slots)
        R = local.shape[0]
        b = torch.arange(R, device=local.device) if row_to_batch is None else _tensor(row_to_batch).to(local.device).long()
        b = b.reshape(-1, *([1] * (local.ndim - 1)))
        pos = local.clamp_min(0).long()
        page = _tensor(src_page_table).to(local.device)[b, pos // page_size].to(torch.int32)
        return torch.where(local >= 0, page * page_size + (pos % page_size).to(torch.int32), local)


def top_k(q, keys, k, sorted=True):
    """flashinfer.top_k(q @ keys.T, k) from queries and keys, exact: q (num_rows, head_dim), keys (n, head_dim).
    Returns (values, indices): float32 inner products, largest first, and their int64 positions, each (num_rows, k)."""
    K, Q = _tensor(keys), _tensor(q)
    _need(K.ndim == 2 and Q.ndim == 2 and Q.shape[1] == K.shape[1],
          "q must have shape (num_rows, head_dim) and keys (n, head_dim)")
    from .attention import KeyCache

    values, indices = KeyCache(1, K.shape[1], k=k).append(K[None]).topk(Q[None], k)
    return values[0], indices[0]
