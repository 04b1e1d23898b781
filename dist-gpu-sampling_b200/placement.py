"""Placement policy around ChunkTensor: how much of each tensor goes into GPU memory, and which rows.

The reference keeps this in its benchmark glue:
  * get_available_memory: oppo_bench/single_node/utils/chunktensor_sampler.py:22-29 (python/utils.py:17-25 is
    an older variant) -- memory that may still be given to ChunkTensors, the minimum over the ranks of the group;
  * the order in which the tensors are placed when memory is short -- features, then probs, then indices,
    then indptr (oppo_bench/single_node/README.md:93; applied by creating them in that order, each taking
    min(its share, what is left): oppo_bench/single_node/chunktensor.py:57-102,
    oppo_bench/multi_node/dist_graph.py:101-185);
  * ChunkTensor puts the FIRST elements of a tensor on the GPUs and the tail in host memory
    (src/chunk_tensor.cc:57-73), so which rows are "hot" is decided by the node numbering.  The reference
    records degrees (oppo_bench/single_node/utils/load_graph.py:263) but never reorders by them;
    renumber_by_degree below is the missing step for a cache-by-degree placement.

Everything here is host-side arithmetic plus torch tensor ops; nothing launches this library's kernels.
"""


def get_available_memory(device, reserved_mem, local_group=None):
    """chunktensor_sampler.py:22-29: total device memory minus `reserved_mem`, minus what ChunkTensors hold
    already, minus 0.3 x torch's peak reserved memory; not below zero; MIN over the ranks of `local_group`
    (every rank must be able to hold its chunk).  Without an initialised process group: this rank's value."""
    import torch
    import torch.distributed as dist
    total = torch.cuda.mem_get_info(device)[1]
    avail = total - reserved_mem - torch.ops.dgs_ops._CAPI_get_current_allocated() \
        - 0.3 * torch.cuda.max_memory_reserved()
    return reduce_min_over_ranks(max(int(avail), 0), local_group)


def reduce_min_over_ranks(value, local_group=None):
    """MIN all-reduce of one integer over `local_group` (the world group when None); the value itself when
    torch.distributed is not initialised.  Works with the nccl and the gloo backend."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return int(value)
    on_gpu = dist.get_backend(local_group) == "nccl"
    t = torch.tensor([int(value)], dtype=torch.int64, device="cuda" if on_gpu else "cpu")
    dist.all_reduce(t, dist.ReduceOp.MIN, group=local_group)
    return int(t.item())


#: the order in which tensors get GPU memory when it is short (oppo_bench/single_node/README.md:93)
CACHE_PRIORITY = ("features", "probs", "indices", "indptr")


def plan_capacities(tensors, num_gpus, available_mem, priority=CACHE_PRIORITY, whole_rows=True):
    """capacity_per_gpu (bytes) for every tensor of a graph, in the reference's priority order.

    tensors: {name: (total_bytes, row_bytes, cache_rate)} -- cache_rate is the fraction of the tensor wanted in
    GPU memory summed over all GPUs (the reference's --feat-cache-rate / --graph-cache-rate).
    Names listed in `priority` are served first, in that order; other names afterwards in the order given.
    Each tensor takes min(total * rate // num_gpus, what is left of available_mem) like create_chunktensor
    (chunktensor_sampler.py:39-43), cut to whole rows (see cached_size_per_gpu) unless whole_rows is False.
    Returns {name: capacity_per_gpu}; the same arithmetic on every rank gives the same plan.
    """
    from . import cached_size_per_gpu
    order = [n for n in priority if n in tensors] + [n for n in tensors if n not in priority]
    left = max(int(available_mem), 0)
    plan = {}
    for name in order:
        total_bytes, row_bytes, rate = tensors[name]
        cap = cached_size_per_gpu(total_bytes, num_gpus, left, rate, row_bytes if whole_rows else None)
        plan[name] = cap
        left -= cap
    return plan


def renumber_by_degree(indptr, indices, by="in", edge_chunk=1 << 27, with_edge_source=True):
    """Renumber the nodes of a CSC graph by descending degree, so that the hottest rows get the smallest ids and
    land in the GPU chunks of a ChunkTensor that caches only part of a tensor.

    by="in":  degree = row length of the CSC (indptr[v+1] - indptr[v]);
    by="out": degree = how often v occurs in `indices` (how often its feature row is fetched by sampling).
    Ties keep their old order (stable).  Works on any device with torch ops; the edge array is rewritten in
    pieces of about `edge_chunk` edges, so the temporaries stay bounded for graphs with billions of edges.

    Returns (new_indptr, new_indices, old_of_new, edge_source):
      old_of_new[i] = old id of new node i   (node tensors: features_new = features[old_of_new])
      edge_source[p] = old position of new edge p   (edge tensors: probs_new = probs[edge_source]);
                       None when with_edge_source is False or the graph has more than `edge_chunk` * 8
                       edges (call permute_edge_tensor with the returned node order instead).
    Row i of the new graph holds the neighbours of old node old_of_new[i], in the old order, renamed.
    """
    import torch
    n = indptr.numel() - 1
    dev = indptr.device
    in_deg = indptr[1:] - indptr[:-1]
    if by == "in":
        key = in_deg
    elif by == "out":
        key = torch.zeros(n, dtype=torch.int64, device=dev)
        for lo in range(0, indices.numel(), edge_chunk):
            key += torch.bincount(indices[lo:lo + edge_chunk], minlength=n)[:n]
    else:
        raise ValueError("by must be 'in' or 'out'")
    old_of_new = torch.sort(key, descending=True, stable=True).indices
    new_of_old = torch.empty_like(old_of_new)
    new_of_old[old_of_new] = torch.arange(n, dtype=old_of_new.dtype, device=dev)
    new_deg = in_deg[old_of_new]
    new_indptr = torch.zeros(n + 1, dtype=indptr.dtype, device=dev)
    torch.cumsum(new_deg, 0, out=new_indptr[1:])
    e_total = int(new_indptr[-1])
    new_indices = torch.empty(e_total, dtype=indices.dtype, device=dev)
    keep_source = with_edge_source and e_total <= 8 * edge_chunk
    edge_source = torch.empty(e_total, dtype=torch.int64, device=dev) if keep_source else None
    old_begin = indptr[:-1][old_of_new]
    row = 0
    while row < n:
        # rows [row, stop) hold at most edge_chunk edges (a single longer row goes alone)
        limit = int(new_indptr[row]) + edge_chunk
        stop = int(torch.searchsorted(new_indptr, torch.tensor([limit], device=dev, dtype=new_indptr.dtype),
                                      right=True).item()) - 1
        stop = min(max(stop, row + 1), n)
        e_lo, e_hi = int(new_indptr[row]), int(new_indptr[stop])
        if e_hi > e_lo:
            seg = torch.repeat_interleave(torch.arange(row, stop, device=dev), new_deg[row:stop])
            src = old_begin[seg] + (torch.arange(e_lo, e_hi, device=dev) - new_indptr[seg])
            new_indices[e_lo:e_hi] = new_of_old[indices[src]].to(indices.dtype)
            if keep_source:
                edge_source[e_lo:e_hi] = src
            del seg, src
        row = stop
    return new_indptr, new_indices, old_of_new, edge_source


def permute_edge_tensor(values, indptr_old, new_indptr, old_of_new, edge_chunk=1 << 27):
    """Per-edge tensor (sampling weights) of the old graph brought into the edge order of the renumbered one,
    piece by piece (for graphs too large for renumber_by_degree to return edge_source)."""
    import torch
    dev = values.device
    n = old_of_new.numel()
    out = torch.empty_like(values)
    new_deg = new_indptr[1:] - new_indptr[:-1]
    old_begin = indptr_old[:-1][old_of_new]
    row = 0
    while row < n:
        limit = int(new_indptr[row]) + edge_chunk
        stop = int(torch.searchsorted(new_indptr, torch.tensor([limit], device=dev, dtype=new_indptr.dtype),
                                      right=True).item()) - 1
        stop = min(max(stop, row + 1), n)
        e_lo, e_hi = int(new_indptr[row]), int(new_indptr[stop])
        if e_hi > e_lo:
            seg = torch.repeat_interleave(torch.arange(row, stop, device=dev), new_deg[row:stop])
            src = old_begin[seg] + (torch.arange(e_lo, e_hi, device=dev) - new_indptr[seg])
            out[e_lo:e_hi] = values[src]
            del seg, src
        row = stop
    return out
