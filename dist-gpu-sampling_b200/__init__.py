"""dgs-b200: B200-native hot path of Dist-GPU-sampling.

The product is two shared libraries built in-tree by `build.py`:

  lib/libdgs_b200.so   C ABI (include/dgs_b200.h)
  lib/libdgs.so        torch.classes.dgs_classes.ChunkTensor + torch.ops.dgs_ops.*

This module only loads them and mirrors the small Python glue of the reference
(communicator bootstrap, ChunkTensor creation, the sample_blocks loop).  There
is no CPU fallback: if the libraries are missing, loading raises.

(The directory name contains a hyphen; import it with
 importlib.import_module("dist-gpu-sampling_b200") after putting the repository
 root on sys.path.)
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
_loaded = {"ops": False, "abi": None}


def abi_path():
    return os.path.join(_PKG, "lib", "libdgs_b200.so")


def binding_path():
    return os.path.join(_PKG, "lib", "libdgs.so")


def build(force=False, verbose=False):
    """Compile both libraries for sm_100a (nvcc + g++, in-tree)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("dgs_b200_build", os.path.join(_PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_all(force=force, verbose=verbose)


def load_ops():
    """torch.ops.load_library on libdgs.so -- the call a user of the reference
    makes with its libdgs.so (example/dgs_create_communicator.py:4)."""
    path = binding_path()
    if not _loaded["ops"]:
        import torch
        if not os.path.exists(path):
            raise RuntimeError(
                "dgs-b200: %s is missing; run `python __graft_entry__.py` (or build.py) first. "
                "There is no fallback path." % path)
        torch.ops.load_library(path)
        _loaded["ops"] = True
    return path


# ---------------------------------------------------------------------------
# ctypes view of the C ABI (used by the tests and by hosts without torch)
# ---------------------------------------------------------------------------
DGS_MAX_PARTS = 8
DGS_MAX_SEGMENTS = 8
DGS_MAX_HOPS = 8


class ChunkDesc(ctypes.Structure):
    _fields_ = [("total", ctypes.c_int64), ("threshold", ctypes.c_int64), ("each", ctypes.c_int64),
                ("num_parts", ctypes.c_int32), ("local_rank", ctypes.c_int32), ("esz", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("host", ctypes.c_void_p),
                ("dev", ctypes.c_void_p * DGS_MAX_PARTS)]


class Segments(ctypes.Structure):
    _fields_ = [("count", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("ptr", ctypes.c_void_p * DGS_MAX_SEGMENTS), ("len", ctypes.c_int64 * DGS_MAX_SEGMENTS)]


class Hop(ctypes.Structure):
    _fields_ = [("fanout", ctypes.c_int64), ("seed_bound", ctypes.c_int64), ("frontier_bound", ctypes.c_int64),
                ("coo_row", ctypes.c_void_p), ("coo_col", ctypes.c_void_p), ("frontier", ctypes.c_void_p)]


# name -> (restype, argtypes); every symbol include/dgs_b200.h declares
_I32, _I64, _U64, _VP, _SZ = ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_size_t
_DP, _SP = ctypes.POINTER(ChunkDesc), ctypes.POINTER(Segments)
_I64P = ctypes.POINTER(ctypes.c_int64)
_HP = ctypes.POINTER(Hop)
ABI_SIGNATURES = {
    "dgs_last_error": (ctypes.c_char_p, []),
    "dgs_device_check": (ctypes.c_int, []),
    "dgs_placement": (ctypes.c_int, [_I64, _I32, _I64, _I32, _I64P, _I64P, _I64P]),
    "dgs_comm_get_unique_id": (ctypes.c_int, [_I64P]),
    "dgs_comm_init": (ctypes.c_int, [_I64, _I64P, _I64]),
    "dgs_comm_barrier": (ctypes.c_int, []),
    "dgs_comm_rank": (ctypes.c_int, []),
    "dgs_comm_size": (ctypes.c_int, []),
    "dgs_comm_destroy": (ctypes.c_int, []),
    "dgs_store_create": (ctypes.c_int, [_I64P, _I32, _I32, _I64, ctypes.POINTER(_VP)]),
    "dgs_store_destroy": (ctypes.c_int, [_VP]),
    "dgs_store_desc": (ctypes.c_int, [_VP, _DP]),
    "dgs_store_elem_stride": (_I64, [_VP]),
    "dgs_store_load": (ctypes.c_int, [_VP, _VP, _I64]),
    "dgs_store_host_view": (ctypes.c_int, [_VP, ctypes.POINTER(_VP), _I64P]),
    "dgs_store_local_view": (ctypes.c_int, [_VP, ctypes.POINTER(_VP), _I64P]),
    "dgs_alloc_current_bytes": (_I64, []),
    "dgs_gather_rows": (ctypes.c_int, [_DP, _I32, _VP, _I32, _I64, _I64, _VP, _VP, _VP]),
    "dgs_gather_rows_counted": (ctypes.c_int, [_DP, _VP, _I32, _I64, _VP, _I64, _VP, _VP, _VP]),
    "dgs_split_index_scratch_bytes": (_SZ, [_I64]),
    "dgs_split_index": (ctypes.c_int, [_DP, _VP, _I32, _I64, _I64, _VP, _VP, _VP, _SZ, _VP]),
    "dgs_split_index_static": (ctypes.c_int, [_DP, _VP, _I32, _I64, _I64, _VP, _VP, _VP]),
    "dgs_sample_plan_bytes": (_SZ, [_I64]),
    "dgs_sample_plan": (ctypes.c_int, [_DP, _VP, _I32, _I64, _I64, _I32, _VP, _VP, _VP, _VP]),
    "dgs_sample_uniform": (ctypes.c_int, [_DP, _VP, _I32, _I64, _I64, _I32, _VP, _U64, _U64, _VP, _VP,
                                          _I64, _VP, _VP, _VP, _VP]),
    "dgs_sample_weighted": (ctypes.c_int, [_DP, _DP, _VP, _I32, _I64, _I64, _I32, _VP, _U64, _U64, _VP,
                                           _VP, _I64, _VP, _VP, _VP, _VP]),
    "dgs_relabel_table_bytes": (_SZ, [_I64]),
    "dgs_unique_first_occurrence": (ctypes.c_int, [_SP, _I32, _VP, _SZ, _VP, _VP, _VP, _VP]),
    "dgs_relabel_lookup": (ctypes.c_int, [_VP, _SZ, _I64, _SP, _I32, _VP, _VP]),
    "dgs_sample_blocks_bounds": (ctypes.c_int, [_I64, _I64P, _I32, _I64, _HP]),
    "dgs_sample_blocks_workspace_bytes": (_SZ, [_HP, _I32]),
    "dgs_sample_blocks": (ctypes.c_int, [_DP, _DP, _DP, _VP, _I32, _HP, _I32, _I32, _U64, _U64, _VP, _SZ, _VP, _VP,
                                         _VP]),
    "dgs_sample_blocks_frontier_count": (_VP, [_HP, _I32, _VP]),
    "dgs_sample_blocks_record": (ctypes.c_int, [_DP, _DP, _DP, _VP, _I32, _HP, _I32, _I32, _VP, _VP, _SZ, _VP, _VP,
                                                _VP, ctypes.POINTER(_VP)]),
    "dgs_sample_blocks_replay": (ctypes.c_int, [_VP, _VP]),
    "dgs_sample_blocks_recording_free": (None, [_VP]),
    "dgs_cache_table_slots": (_I64, [_I64]),
    "dgs_cache_build": (ctypes.c_int, [_VP, _VP, _I32, _I64, _VP, _VP, _I64, _VP, _VP]),
    "dgs_cache_fetch": (ctypes.c_int, [_VP, _I64, _DP, _VP, _I32, _I64, _I64, _VP, _VP, _I64, _VP, _VP, _VP]),
}


def load_abi():
    """ctypes handle on libdgs_b200.so with argtypes set; raises if it is missing."""
    if _loaded["abi"] is None:
        path = abi_path()
        if not os.path.exists(path):
            raise RuntimeError("dgs-b200: %s is missing; build it first. There is no fallback path." % path)
        lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in ABI_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _loaded["abi"] = lib
    return _loaded["abi"]


class AbiError(RuntimeError):
    pass


def check(rc):
    if rc != 0:
        raise AbiError("dgs error %d: %s" % (rc, load_abi().dgs_last_error().decode()))


# ---------------------------------------------------------------------------
# Python glue of the reference, without DGL
# ---------------------------------------------------------------------------
def create_dgs_communicator(group_size, local_group=None):
    """oppo_bench/single_node/utils/chunktensor_sampler.py:7-19: rank 0 of each
    group draws an NCCL unique id, broadcasts it over torch.distributed, and
    every rank joins the library's bootstrap communicator."""
    import torch
    import torch.distributed as dist
    load_ops()
    if dist.get_rank() % group_size == 0:
        broadcast_list = [torch.ops.dgs_ops._CAPI_get_unique_id()]
    else:
        broadcast_list = [None]
    dist.broadcast_object_list(broadcast_list, dist.get_rank() - dist.get_rank() % group_size, local_group)
    torch.ops.dgs_ops._CAPI_set_nccl(group_size, broadcast_list[0], dist.get_rank() % group_size)


def cached_size_per_gpu(total_bytes, num_gpus, available_mem, cache_rate=1.0, row_bytes=None):
    """Capacity rule of create_chunktensor (chunktensor_sampler.py:39-43): an equal share of the cached part,
    limited by the memory that is free.  With row_bytes the result is rounded down to whole rows, so that no
    row straddles two chunks and every row keeps the alignment of the first (the reference's rule cuts chunks
    at arbitrary bytes; the gather then has to fall back to narrower loads for the chunks after the first)."""
    cap = int(min(total_bytes * cache_rate // num_gpus, available_mem))
    if row_bytes:
        # a whole number of rows, and of 16-byte vectors when the row size allows it
        unit = row_bytes
        while unit % 16 and unit < 16 * row_bytes:
            unit += row_bytes
        cap = max(cap // unit * unit, min(cap, unit) // row_bytes * row_bytes)
    return cap


def create_chunktensor(tensor, num_gpus, available_mem, cache_rate=1.0, root_rank=0, local_group=None,
                       whole_rows=True):
    """chunktensor_sampler.py:32-60: the root rank decides the capacity, every rank
    constructs the ChunkTensor (collective), the root loads the data.  Capacities are whole rows
    (see cached_size_per_gpu); whole_rows=False gives the reference's byte-exact rule."""
    import torch
    import torch.distributed as dist
    load_ops()
    distributed = dist.is_available() and dist.is_initialized()
    rank = dist.get_rank() if distributed else 0
    if rank == root_rank:
        total = tensor.numel() * tensor.element_size()
        row_bytes = tensor.element_size() * (tensor.shape[1] if tensor.dim() == 2 else 1)
        meta = [list(tensor.shape), tensor.dtype,
                cached_size_per_gpu(total, num_gpus, available_mem, cache_rate, row_bytes if whole_rows else None)]
    else:
        meta = [None, None, None]
    if distributed:
        dist.broadcast_object_list(meta, root_rank, local_group)
    ct = torch.classes.dgs_classes.ChunkTensor(meta[0], meta[1], meta[2])
    if rank == root_rank:
        ct._CAPI_load_from_tensor(tensor)
    if distributed:
        dist.barrier(local_group)
    return ct


def sample_blocks(seeds, fanouts, indptr, indices, probs=None, replace=False, fused=False):
    """The hot loop of ChunkTensorSampler.sample_blocks
    (chunktensor_sampler.py:93-118) without the DGL block objects.

    indptr / indices / probs are ChunkTensors or plain CUDA tensors.  Returns
    (frontier, blocks, n_edges) with blocks = [(coo_row, coo_col, n_src, n_dst)]
    in layer order (outermost hop first, like the reference's blocks.insert(0, ...)).

    fused=False runs the reference's own sequence: one sampling operator and one
    _CAPI_tensor_relabel per hop.  fused=True hands the whole loop to
    _CAPI_sample_blocks*, which queues every hop without reading a size back in
    between; the results follow the same rules (and are identical wherever no
    random choice is involved).
    """
    import torch
    ops = torch.ops.dgs_ops
    chunked = not isinstance(indptr, torch.Tensor)
    if fused:
        if probs is not None:
            fn = ops._CAPI_sample_blocks_with_probs_with_chunk_tensor if chunked else ops._CAPI_sample_blocks_with_probs
            frontier, rows, cols, shape = fn(seeds, indptr, indices, probs, list(fanouts), replace)
        else:
            fn = ops._CAPI_sample_blocks_with_chunk_tensor if chunked else ops._CAPI_sample_blocks
            frontier, rows, cols, shape = fn(seeds, indptr, indices, list(fanouts), replace)
        blocks = [(rows[i], cols[i], shape[2 * i], shape[2 * i + 1]) for i in range(len(rows))]
        return frontier, blocks, sum(r.numel() for r in rows)
    blocks, n_edges = [], 0
    for fan_out in reversed(list(fanouts)):
        if probs is not None:
            fn = ops._CAPI_sample_neighbors_with_probs_with_chunk_tensor if chunked \
                else ops._CAPI_sample_neighbors_with_probs
            coo_row, coo_col = fn(seeds, indptr, indices, probs, fan_out, replace)
        else:
            fn = ops._CAPI_sample_neighbors_with_chunk_tensor if chunked else ops._CAPI_sample_neighbors
            coo_row, coo_col = fn(seeds, indptr, indices, fan_out, replace)
        n_edges += coo_row.numel()
        frontier, (coo_row, coo_col) = ops._CAPI_tensor_relabel([seeds, coo_col], [coo_row, coo_col])
        blocks.insert(0, (coo_row, coo_col, frontier.numel(), seeds.numel()))
        seeds = frontier
    return seeds, blocks, n_edges


class PipelinedSampler:
    """Mini-batches in flight: the role DGL's DataLoader plays around ChunkTensorSampler in the reference
    (oppo_bench/single_node/chunktensor.py:120-172), on torch.classes.dgs_classes.BlockPipeline.

        sampler = PipelinedSampler(indptr_ct, indices_ct, [15, 10, 5], features=feat_ct, max_seeds=1024, depth=6)
        for input_nodes, blocks, n_edges, x in sampler(seed_batches):
            ...   # blocks = [(coo_row, coo_col, n_src, n_dst)] in layer order, x = features[input_nodes]

    Up to `depth` batches are in flight, each on a stream of its own, so the small hops of one batch overlap
    with the gather of another and with the consumer of the batch before.  What a batch yields are views into
    its slot: valid until the NEXT batch is drawn from the iterator (that is when the slot is handed to a new
    batch); clone what must live longer.  With submit() / next() called by hand, a batch stays valid until
    the submit() that reuses its slot, the depth-th after its own.  indptr / indices / probs / features are ChunkTensors; seed
    batches are tensors on the GPU or in (pinned) host memory, at most max_seeds ids each.  Results follow
    the same rules as sample_blocks(): identical wherever no random choice is involved.
    Delete the sampler before the ChunkTensors it reads (their destructor is collective).
    src_nodes: the size of the id space `indices` draws from when that is larger than indptr's node count
    (a bipartite CSC); the buffers for the input nodes are sized by it.
    """

    def __init__(self, indptr, indices, fanouts, features=None, probs=None, replace=False, max_seeds=1024, depth=6,
                 src_nodes=0):
        import torch
        load_ops()
        self.depth = int(depth)
        self.pipe = torch.classes.dgs_classes.BlockPipeline(indptr, indices, probs, features, list(fanouts),
                                                            bool(replace), int(max_seeds), self.depth, int(src_nodes))

    def submit(self, seeds):
        self.pipe.submit(seeds)

    def next(self):
        frontier, rows, cols, shape, x = self.pipe.next()
        blocks = [(rows[i], cols[i], shape[2 * i], shape[2 * i + 1]) for i in range(len(rows))]
        return frontier, blocks, sum(r.numel() for r in rows), x

    def __call__(self, seed_batches):
        ahead = 0
        for seeds in seed_batches:
            self.pipe.submit(seeds)
            ahead += 1
            if ahead == self.depth:
                yield self.next()
                ahead -= 1
        while ahead:
            yield self.next()
            ahead -= 1


def block_csc(coo_row, coo_col, n_dst, rows_sorted=True):
    """CSC form of one sampled block, for a GNN layer that wants (indptr, indices) instead of COO.

    coo_row holds relabelled destination ids (positions of the seeds), coo_col relabelled source ids.
    The samplers emit edges grouped by seed position, so with a duplicate-free seed list coo_row is already
    non-decreasing and the column order is the CSC order (rows_sorted=True: no sort).  With repeated seeds
    (rows_sorted=False) the edges are first brought into destination order by a stable sort.
    Returns (indptr[n_dst + 1], indices) on coo_row's device; the DGL-free counterpart of the
    dgl.create_block call in chunktensor_sampler.py:112-116.
    """
    import torch
    if not rows_sorted:
        order = torch.sort(coo_row, stable=True).indices
        coo_row, coo_col = coo_row[order], coo_col[order]
    indptr = torch.zeros(n_dst + 1, dtype=torch.int64, device=coo_row.device)
    if coo_row.numel():
        indptr[1:] = torch.cumsum(torch.bincount(coo_row.to(torch.int64), minlength=n_dst)[:n_dst], 0)
    return indptr, coo_col


# placement policy (capacity planning in the reference's priority order, free-memory rule, renumbering by degree)
from .placement import (CACHE_PRIORITY, get_available_memory, permute_edge_tensor, plan_capacities,  # noqa: E402,F401
                        reduce_min_over_ranks, renumber_by_degree)
