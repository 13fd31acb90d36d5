"""libcertex_b200: a B200 (sm_100a) exact k-nearest-neighbour engine behind the API of hpdic/libcertex.

    import libcertex_b200 as certex
    D, I = certex.search(xb, xq, k=10)            # the exact 10 nearest neighbours of every query
    index = certex.Index(dim=128); index.add(xb); D, I = index.search(xq, k=10)

All arithmetic runs in the CUDA library `lib/libcertex_b200.so` (C ABI: include/certex_b200.h); there is no CPU or
PyTorch fallback.
"""

from ._lib import CertexError
from .attention import KeyCache, topk
from .index import Index, ShardedIndex, merge_shards, search, search_stats, verify

__version__ = "0.2.0"
__all__ = ["CertexError", "KeyCache", "topk", "Index", "ShardedIndex", "merge_shards", "search", "search_stats", "verify", "__version__"]
