"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations. They stand in for
the public datasets the reference measures on (BIGANN / SIFT1B prefixes), which are not available offline."""

import numpy as np
import torch

CHUNK = 1 << 20  # rows generated per call of the device generator; fixed so that shards reproduce the same rows


def mixture_centers(n_centers=1000, dim=128, seed=2):
    """Centres uniform in [20, 235] (CPU generator: identical on every rank and device)."""
    g = torch.Generator().manual_seed(seed)
    return torch.rand((n_centers, dim), generator=g) * 215.0 + 20.0


def mixture_u8(n, dim=128, n_centers=1000, sigma=18.0, seed=0, row0=0, device="cuda", centers=None):
    """Rows [row0, row0 + n) of the uint8 Gaussian mixture: centre[uniform index] + N(0, sigma^2) per dimension,
    rounded and clipped to [0, 255]. Chunk c of CHUNK rows is drawn from a generator seeded with (seed, c), so any
    row range gives the same values whichever process asks for it (on the same kind of device)."""
    if centers is None:
        centers = mixture_centers(n_centers, dim)
    centers = centers.to(device)
    out = torch.empty((n, dim), dtype=torch.uint8, device=device)
    c0, c1 = row0 // CHUNK, (row0 + n + CHUNK - 1) // CHUNK
    for c in range(c0, c1):
        g = torch.Generator(device=device).manual_seed(seed * 1_000_003 + c)
        which = torch.randint(0, centers.shape[0], (CHUNK,), generator=g, device=device)
        lo, hi = max(row0, c * CHUNK), min(row0 + n, (c + 1) * CHUNK)
        # the noise of a whole chunk is drawn in slabs to bound memory; the slab size is part of the recipe
        slab = 1 << 18
        for s0 in range(0, CHUNK, slab):
            noise = torch.randn((slab, dim), generator=g, device=device) * sigma
            a, b = max(lo, c * CHUNK + s0), min(hi, c * CHUNK + s0 + slab)
            if a < b:
                ra, rb = a - c * CHUNK, b - c * CHUNK
                rows = centers[which[ra:rb]] + noise[ra - s0 : rb - s0]
                out[a - row0 : b - row0] = rows.round_().clamp_(0, 255).to(torch.uint8)
    return out


def clustered_unit_f32(n, dim=768, n_clusters=4096, seed=0, row0=0, device="cuda"):
    """Rows [row0, row0 + n) of the filtered workload's float32 vectors: a unit-length cluster centre (Gaussian
    direction) plus noise of length about sigma, sigma log-uniform in [0.05, 0.3] per cluster and unequal over the
    dimensions (fixed per-dimension scales in [0.25, 1.75]); every row is then scaled to unit length. Chunked and
    seeded like mixture_u8."""
    g0 = torch.Generator().manual_seed(7_000_003 + n_clusters)
    centers = torch.randn((n_clusters, dim), generator=g0)
    centers /= centers.norm(dim=1, keepdim=True)
    sigma = torch.exp(torch.rand(n_clusters, generator=g0) * np.log(0.3 / 0.05) + np.log(0.05))
    scales = (torch.rand(dim, generator=g0) * 1.5 + 0.25) / np.sqrt(dim)
    centers, sigma, scales = centers.to(device), sigma.to(device), scales.to(device)
    out = torch.empty((n, dim), dtype=torch.float32, device=device)
    slab = 1 << 16
    s0, s1 = row0 // slab, (row0 + n + slab - 1) // slab
    for c in range(s0, s1):
        g = torch.Generator(device=device).manual_seed(seed * 1_000_003 + c)
        which = torch.randint(0, n_clusters, (slab,), generator=g, device=device)
        rows = centers[which] + torch.randn((slab, dim), generator=g, device=device) * scales * sigma[which, None]
        rows /= rows.norm(dim=1, keepdim=True)
        a, b = max(row0, c * slab), min(row0 + n, (c + 1) * slab)
        out[a - row0 : b - row0] = rows[a - c * slab : b - c * slab]
    return out


def gaussian_f32(n, nq, dim=128, seed=0):
    """The CPU plumbing configuration: base then queries from one numpy default_rng(seed) stream, i.i.d. N(0, 1)."""
    rng = np.random.default_rng(seed)
    xb = rng.standard_normal((n, dim), dtype=np.float32)
    xq = rng.standard_normal((nq, dim), dtype=np.float32)
    return xb, xq


def correlated(n, dim, seed=0, dtype="float32", unequal_norms=False, mix_seed=1234):
    """Correlated Gaussian rows (a fixed random mixing matrix gives a decaying spectrum), as float32 / float16, or
    scaled and clamped to int8 / uint8; the kind of data the reference's exactness tests draw."""
    mix = np.random.default_rng(mix_seed).standard_normal((dim, dim)).astype(np.float32) / np.float32(np.sqrt(dim))
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, dim)).astype(np.float32) @ mix
    if unequal_norms:
        x = x * (0.2 + 3.0 * rng.random((n, 1), dtype=np.float32))
    if dtype == "float32":
        return x
    if dtype == "float16":
        return x.astype(np.float16)
    if dtype == "int8":
        return np.clip(np.round(x * 30), -127, 127).astype(np.int8)
    return np.clip(np.round(x * 30 + 100), 0, 255).astype(np.uint8)


def keys_with_outliers(n_kv_heads=8, n=131072, head_dim=128, n_outlier=4, scale=20.0, seed=0, device="cuda"):
    """bf16 keys ~ N(0, 1) with `n_outlier` fixed channels per head scaled by `scale`."""
    g = torch.Generator(device=device).manual_seed(seed)
    k = torch.randn((n_kv_heads, n, head_dim), generator=g, device=device)
    gc = torch.Generator().manual_seed(seed + 1)
    for h in range(n_kv_heads):
        ch = torch.randperm(head_dim, generator=gc)[:n_outlier]
        k[h][:, ch.to(device)] *= scale
    return k.to(torch.bfloat16)
