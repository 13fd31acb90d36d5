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


class KeyCache:
    """n_kv_heads, head_dim: the shape of the keys; k: the largest k searches will ask for; capacity: expected keys
    per head (reserves memory once)."""

    def __init__(self, n_kv_heads, head_dim, k=2048, capacity=None):
        _need(n_kv_heads >= 1 and head_dim >= 1, "n_kv_heads and head_dim must be positive")
        _need(1 <= k <= 2048, f"k must be between 1 and 2048, not {k}")
        self.n_kv_heads, self.head_dim, self.k, self.capacity = int(n_kv_heads), int(head_dim), int(k), capacity
        self.heads, self.dtype, self.size = None, None, 0

    def append(self, keys):
        """Append keys of shape (n_kv_heads, n, head_dim); ids continue from the keys appended before."""
        K = _as_half_or_float(keys)
        _need(K.ndim == 3 and K.shape[0] == self.n_kv_heads and K.shape[2] == self.head_dim,
              f"keys must have shape ({self.n_kv_heads}, n, {self.head_dim}), not {tuple(K.shape)}")
        if self.heads is None:
            self.dtype = K.dtype
            self.heads = [Index(self.head_dim, metric="ip", capacity=self.capacity) for _ in range(self.n_kv_heads)]
        for g, idx in enumerate(self.heads):
            idx.add(K[g].to(self.dtype).contiguous())
        self.size += K.shape[1]
        return self

    def topk(self, q, k=None, batch=2048):
        """q: (n_heads, m, head_dim) or (n_heads, head_dim), n_heads a multiple of n_kv_heads. Returns (scores, ids) of
        shape (n_heads, m, k) or (n_heads, k), scores descending."""
        _need(self.heads is not None, "the cache is empty: append keys first")
        k = self.k if k is None else int(k)
        _need(1 <= k <= min(2048, self.size), f"k must be between 1 and {min(2048, self.size)}, not {k}")
        Q = _as_half_or_float(q)
        single = Q.ndim == 2
        if single:
            Q = Q[:, None, :]
        _need(Q.ndim == 3 and Q.shape[2] == self.head_dim and Q.shape[0] % self.n_kv_heads == 0,
              f"queries must have shape (n_heads, m, {self.head_dim}) with n_heads a multiple of {self.n_kv_heads}")
        H, m, d = Q.shape
        group = H // self.n_kv_heads
        scores = torch.empty((H, m, k), dtype=torch.float32, device="cuda")
        ids = torch.empty((H, m, k), dtype=torch.int64, device="cuda")
        for g, idx in enumerate(self.heads):
            rows = slice(g * group, (g + 1) * group)
            D, I = idx.search(Q[rows].reshape(group * m, d).to(self.dtype), k=k, batch=batch)
            scores[rows] = D.reshape(group, m, k)
            ids[rows] = I.reshape(group, m, k)
        return (scores[:, 0], ids[:, 0]) if single else (scores, ids)


def topk(q, keys, k):
    """One call: keys (n_kv_heads, n, head_dim), q (n_heads, m, head_dim) or (n_heads, head_dim)."""
    K = torch.as_tensor(keys)
    _need(K.ndim == 3, "keys must have shape (n_kv_heads, n, head_dim)")
    return KeyCache(K.shape[0], K.shape[2], k=k).append(K).topk(q, k)
