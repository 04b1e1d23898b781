"""Seeded synthetic inputs shaped like the graphs the reference is run on.

The reference's datasets (ogbn-products, ogbn-papers100M, Friendster;
oppo_bench/single_node/utils/load_graph.py) are not available offline, so the
tests and the benchmark use generators with the same sizes and degree
statistics.  Everything is CSC with int64 indptr/indices, the layout the
reference stores in its ChunkTensors (oppo_bench/single_node/chunktensor.py).
"""
import numpy as np


def uniform_graph_csc(num_nodes, num_edges, seed=1):
    """Uniform-random endpoints; CSC by destination, neighbour order = stable
    sort by destination (the small parity configuration)."""
    rng = np.random.default_rng(seed)
    src = rng.integers(0, num_nodes, num_edges, dtype=np.int64)
    dst = rng.integers(0, num_nodes, num_edges, dtype=np.int64)
    order = np.argsort(dst, kind="stable")
    indices = src[order]
    indptr = np.zeros(num_nodes + 1, dtype=np.int64)
    np.cumsum(np.bincount(dst, minlength=num_nodes), out=indptr[1:])
    return indptr, indices


def distinct_seeds(num_nodes, n, seed=2):
    rng = np.random.default_rng(seed)
    return rng.choice(num_nodes, size=n, replace=False).astype(np.int64)


def chung_lu_csc(num_nodes, mean_degree, gamma, seed, device="cpu", max_degree=None, chunk=1 << 25,
                 degree_sorted=False):
    """Chung-Lu style power-law graph built directly in CSC with torch ops.

    Node v gets expected degree w_v proportional to (r_v + i0)^(-1/(gamma-1)) where
    r is a random permutation (degree independent of id), scaled to the requested
    mean; its in-degree is Poisson(w_v) and every neighbour is drawn with
    probability proportional to w.  With degree_sorted the permutation is the
    identity: node ids are ranked by expected in-degree, hottest first (the
    renumbering a cache-by-degree placement wants).
    Returns (indptr, indices) int64 tensors on `device`.
    """
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    if max_degree is None:
        max_degree = max(16.0, num_nodes ** 0.5 * mean_degree ** 0.5)
    alpha = 1.0 / (gamma - 1.0)
    if degree_sorted:
        rank = torch.arange(num_nodes, device=device, dtype=torch.float64)
    else:
        rank = torch.randperm(num_nodes, generator=g, device=device).to(torch.float64)
    # i0 bounds the largest expected degree: w_max / w_mean ~ ((N+i0)/i0)^alpha
    i0 = 1.0
    for _ in range(60):
        w = (rank + i0).pow(-alpha)
        scale = mean_degree * num_nodes / w.sum()
        if float(scale * i0 ** (-alpha)) <= max_degree:
            break
        i0 *= 1.5
    w = w * scale
    deg = torch.poisson(w.to(torch.float32), generator=g).to(torch.int64)
    indptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=device)
    torch.cumsum(deg, 0, out=indptr[1:])
    num_edges = int(indptr[-1].item())
    cdf = torch.cumsum(w, 0)
    cdf = cdf / cdf[-1]
    indices = torch.empty(num_edges, dtype=torch.int64, device=device)
    for lo in range(0, num_edges, chunk):
        hi = min(lo + chunk, num_edges)
        u = torch.rand(hi - lo, generator=g, device=device, dtype=torch.float64)
        torch.searchsorted(cdf, u, out=indices[lo:hi])
    indices.clamp_(max=num_nodes - 1)
    return indptr, indices


def train_batches(num_nodes, train_size, batch, seed=12):
    """A fixed random training set, cut into consecutive batches of a fixed
    permutation (numpy int64 [num_batches, batch])."""
    rng = np.random.default_rng(seed)
    train = rng.choice(num_nodes, size=train_size, replace=False).astype(np.int64)
    perm = rng.permutation(train)
    nb = train_size // batch
    return perm[: nb * batch].reshape(nb, batch)


def hash_of_index(e, salt=0):
    """fp32 value in [-1, 1) of flat element indices `e` (an int64 tensor)."""
    import torch
    x = (e ^ (e >> 31)) * 0x7FB5D329728EA185 + salt    # wraps modulo 2^64
    x = (x ^ (x >> 27)) * 0x1B87359352DCE729
    x = x ^ (x >> 33)
    return (x & 0xFFFFFF).to(torch.float32) * (2.0 / 16777216.0) - 1.0


def hashed_values(start, count, device="cpu", salt=0):
    """Deterministic fp32 value of every flat element index in [start, start+count):
    any chunk of a huge table can be generated (and checked) on its own without
    storing the whole table anywhere."""
    import torch
    return hash_of_index(torch.arange(start, start + count, device=device, dtype=torch.int64), salt)
