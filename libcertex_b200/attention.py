"""Exact top-k over the keys of a KV cache, with the call surface of the reference's certex/attention.py
(`KeyCache` 44-106, `topk` 109-114): one inner-product index per KV head, extended by append(); grouped-query
attention maps query head h to KV head h // (n_heads / n_kv_heads). Returns what torch.topk(q @ keys.mT, k) returns,
but the k keys of every query are the exact top k by fp64 inner product, ties to the smaller key position.
"""

import torch

from .index import Index, _need


def _as_half_or_float(x):
    """float16 on the GPU, or float32 where float16 would overflow (bf16 inputs can)."""
    x = torch.as_tensor(x, device="cuda")
    h = x.to(torch.float16)
    return h if bool(torch.isfinite(h).all()) else x.to(torch.float32)


class GrowingMap:
    """A one-dimensional device tensor that is appended to: the buffer doubles when it is full, so that appending a few
    entries per decoding step does not copy the whole map every time."""

    def __init__(self, dtype):
        self.dtype, self.buf, self.n = dtype, None, 0

    def append(self, values, reserve=0):
        need = self.n + values.numel()
        if self.buf is None or need > self.buf.numel():
            grown = torch.empty((max(need, int(reserve), 2 * self.n),), dtype=self.dtype, device="cuda")
            if self.n:
                grown[: self.n] = self.buf[: self.n]
            self.buf = grown
        self.buf[self.n : need] = values
        self.n = need

    def __len__(self):
        return self.n

    @property
    def values(self):
        return self.buf[: self.n]


class KeyCache:
    """n_kv_heads, head_dim: the shape of the keys; k: the largest k searches will ask for; capacity: expected keys
    per head (reserves memory once).

    All KV heads live in one labeled inner-product index (label = KV head), so that one search call answers the
    queries of every head: each query is screened and scored against the keys of its own head only."""

    def __init__(self, n_kv_heads, head_dim, k=2048, capacity=None):
        _need(n_kv_heads >= 1 and head_dim >= 1, "n_kv_heads and head_dim must be positive")
        _need(1 <= k <= 2048, f"k must be between 1 and 2048, not {k}")
        self.n_kv_heads, self.head_dim, self.k, self.capacity = int(n_kv_heads), int(head_dim), int(k), capacity
        self.index, self.dtype, self.size = None, None, 0
        self._map = GrowingMap(torch.int64)  # id of the index -> position of the key inside its head

    def append(self, keys):
        """Append keys of shape (n_kv_heads, n, head_dim); positions continue from the keys appended before."""
        K = _as_half_or_float(keys)
        _need(K.ndim == 3 and K.shape[0] == self.n_kv_heads and K.shape[2] == self.head_dim,
              f"keys must have shape ({self.n_kv_heads}, n, {self.head_dim}), not {tuple(K.shape)}")
        n_new = K.shape[1]
        if self.index is None:
            self.dtype = K.dtype
            cap = None if self.capacity is None else int(self.capacity) * self.n_kv_heads
            # the partition by head is renewed once an eighth of the keys is newer than it: appending a few keys per
            # decoding step must not copy the whole cache
            self.index = Index(self.head_dim, metric="ip", capacity=cap, partition_labels="lazy")
        _need(not (self.dtype == torch.float16 and K.dtype == torch.float32),
              "these keys do not fit float16 but the cache was started with float16 keys: start it with float32 keys")
        heads = torch.arange(self.n_kv_heads, dtype=torch.int32, device="cuda").repeat_interleave(n_new)
        self.index.add(K.to(self.dtype).reshape(self.n_kv_heads * n_new, self.head_dim).contiguous(), labels=heads)
        pos = torch.arange(self.size, self.size + n_new, dtype=torch.int64, device="cuda").repeat(self.n_kv_heads)
        self._map.append(pos, reserve=0 if self.capacity is None else int(self.capacity) * self.n_kv_heads)
        self.size += n_new
        return self

    @property
    def _position(self):
        return self._map.values

    def topk(self, q, k=None, batch=2048):
        """q: (n_heads, m, head_dim) or (n_heads, head_dim), n_heads a multiple of n_kv_heads. Returns (scores, ids) of
        shape (n_heads, m, k) or (n_heads, k), scores descending, ids = key positions."""
        _need(self.index is not None, "the cache is empty: append keys first")
        k = self.k if k is None else int(k)
        _need(1 <= k <= min(2048, self.size), f"k must be between 1 and {min(2048, self.size)}, not {k}")
        Q = _as_half_or_float(q)
        single = Q.ndim == 2
        if single:
            Q = Q[:, None, :]
        _need(Q.ndim == 3 and Q.shape[2] == self.head_dim and Q.shape[0] % self.n_kv_heads == 0,
              f"queries must have shape (n_heads, m, {self.head_dim}) with n_heads a multiple of {self.n_kv_heads}")
        _need(not (self.dtype == torch.float16 and Q.dtype == torch.float32),
              "these queries do not fit float16 but the cache holds float16 keys: start the cache with float32 keys")
        H, m, d = Q.shape
        group = H // self.n_kv_heads
        heads = (torch.arange(H, dtype=torch.int32, device="cuda") // group).repeat_interleave(m)
        D, I = self.index.search(Q.reshape(H * m, d).to(self.dtype).contiguous(), k=k, batch=batch, labels=heads)
        ids = self._position[I.clamp_(min=0)]  # every head holds at least k keys: no entry is missing
        scores, ids = D.reshape(H, m, k), ids.reshape(H, m, k)
        return (scores[:, 0], ids[:, 0]) if single else (scores, ids)


def topk(q, keys, k):
    """One call: keys (n_kv_heads, n, head_dim), q (n_heads, m, head_dim) or (n_heads, head_dim)."""
    K = torch.as_tensor(keys)
    _need(K.ndim == 3, "keys must have shape (n_kv_heads, n, head_dim)")
    return KeyCache(K.shape[0], K.shape[2], k=k).append(K).topk(q, k)
