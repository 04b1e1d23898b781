"""numpy/ctypes front end of the CPU oracle (oracle/dgs_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py -- never by the product package.

Every function restates the reference operator named in its docstring
(paths are inside gpzlx1/Dist-GPU-sampling).  Parity status is stated in the
header of dgs_oracle.c: placement is pinned by the README demo vector, every
deterministic operator output by vectors recorded from the reference's own
kernels on a B200 (tests/golden/reference_b200.json).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libdgs_oracle.so")
_lib = None

_i64p = ctypes.POINTER(ctypes.c_int64)


def build(force=False):
    """Compile the C restatement into oracle/_ref/ (gcc, a second or two)."""
    src = os.path.join(_HERE, "dgs_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.dgs_oracle_sample_counts.restype = ctypes.c_int64
        _lib.dgs_oracle_unique.restype = ctypes.c_int64
        _lib.dgs_oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads():
    return int(lib().dgs_oracle_num_threads())


def use_all_cores():
    """OpenMP threads = the cores this process may run on, whatever OMP_NUM_THREADS the launcher exported
    (torchrun sets it to 1 for its children).  Returns the thread count now in use."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().dgs_oracle_set_num_threads(ctypes.c_int(max(1, n)))
    return num_threads()


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def placement(total, esz, capacity_per_gpu, world):
    """ChunkTensor size rules, src/chunk_tensor.cc:53-73 -> (each, threshold, host)."""
    e, t, h = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    lib().dgs_oracle_placement(ctypes.c_int64(total), ctypes.c_int32(esz),
                               ctypes.c_int64(capacity_per_gpu), ctypes.c_int32(world),
                               ctypes.byref(e), ctypes.byref(t), ctypes.byref(h))
    return e.value, t.value, h.value


class ChunkModel:
    """Host model of one ChunkTensor: W chunk buffers + host tail.

    Mirrors ChunkTensor (src/chunk_tensor.cc:37-200): chunks are 0xFF-filled
    at creation (:108), `load` follows LoadFromTensor (:173-200), `index`
    follows _IndexMemcpyKernel through chunk_tensor_wrapper::At
    (src/cuda/index_with_chunk_tensor.cu:9-27, src/chunk_tensor.h:33-42).
    """

    def __init__(self, shape, dtype, capacity_per_gpu, world=1):
        shape = tuple(int(s) for s in shape)
        assert len(shape) in (1, 2)
        self.shape = shape
        self.dtype = np.dtype(dtype)
        self.world = int(world)
        self.total = int(np.prod(shape))
        self.D = shape[1] if len(shape) == 2 else 1
        self.esz = self.dtype.itemsize
        self.each, self.thr, self.host_n = placement(self.total, self.esz, capacity_per_gpu, world)
        self.dev = [np.full(self.each * self.esz, 0xFF, dtype=np.uint8) for _ in range(self.world)]
        self.host = np.zeros(max(self.host_n, 0) * self.esz, dtype=np.uint8)

    def _dev_array(self):
        arr = (ctypes.c_void_p * self.world)()
        for i, d in enumerate(self.dev):
            arr[i] = d.ctypes.data if d.size else None
        return arr

    def load(self, flat):
        flat = np.ascontiguousarray(flat, dtype=self.dtype).reshape(-1)
        assert flat.size == self.total
        lib().dgs_oracle_load(_p(flat), ctypes.c_int64(self.total), ctypes.c_int32(self.esz),
                              ctypes.c_int64(self.each), ctypes.c_int64(self.thr),
                              ctypes.c_int32(self.world), self._dev_array(), _p(self.host))

    def host_tensor(self):
        """GetHostTensor, src/chunk_tensor.cc:151-160 (flat view of the tail)."""
        return self.host.view(self.dtype)

    def sub_device_tensor(self, rank):
        """GetSubDeviceTensor, src/chunk_tensor.cc:162-171 (flat view of chunk `rank`)."""
        return self.dev[rank].view(self.dtype)

    def index(self, idx):
        idx = _i64(idx).reshape(-1)
        out = np.empty((idx.size, self.D), dtype=self.dtype)
        if self.each == 0:  # no GPU part: At() never divides
            each = 1
        else:
            each = self.each
        lib().dgs_oracle_index(self._dev_array(), _p(self.host), ctypes.c_int64(each),
                               ctypes.c_int64(self.thr), ctypes.c_int32(self.esz), _p(idx),
                               ctypes.c_int64(idx.size), ctypes.c_int64(self.D), _p(out))
        return out

    def split_index(self, idx, rank):
        """SplitIndexFromChunkTensorCUDA, src/cuda/index_with_chunk_tensor.cu:55-108."""
        return split_index(idx, self.D, self.each, self.thr, rank)


def split_index(idx, D, each, thr, rank):
    idx = _i64(idx).reshape(-1)
    n = idx.size
    lo, re, ho = (np.empty(n, np.int64) for _ in range(3))
    cnt = np.zeros(3, np.int64)
    lib().dgs_oracle_split_index(_p(idx), ctypes.c_int64(n), ctypes.c_int64(D),
                                 ctypes.c_int64(each), ctypes.c_int64(thr), ctypes.c_int64(rank),
                                 _p(lo), _p(re), _p(ho), _p(cnt))
    return lo[:cnt[0]].copy(), re[:cnt[1]].copy(), ho[:cnt[2]].copy()


def index_flat(flat2d, idx):
    """torch.index_select(T, 0, idx) on the flat logical tensor (timed CPU baseline)."""
    flat2d = np.ascontiguousarray(flat2d)
    idx = _i64(idx).reshape(-1)
    D = flat2d.shape[1] if flat2d.ndim == 2 else 1
    out = np.empty((idx.size, D), dtype=flat2d.dtype)
    lib().dgs_oracle_index_flat(_p(flat2d), ctypes.c_int32(flat2d.dtype.itemsize), _p(idx),
                                ctypes.c_int64(idx.size), ctypes.c_int64(D), _p(out))
    return out


def sample_counts(indptr, seeds, k, replace):
    """_GetSubIndptr + scan, src/cuda/rowwise_sampling.cu:13-40 -> (out_ptr[n+1], nnz)."""
    indptr, seeds = _i64(indptr), _i64(seeds)
    out_ptr = np.empty(seeds.size + 1, np.int64)
    nnz = lib().dgs_oracle_sample_counts(_p(indptr), _p(seeds), ctypes.c_int64(seeds.size),
                                         ctypes.c_int64(k), ctypes.c_int32(int(replace)),
                                         _p(out_ptr))
    return out_ptr, int(nnz)


def sample_uniform(indptr, indices, seeds, k, replace, rng_seed=0, want_pos=False):
    """RowWiseSamplingUniformCUDA, src/cuda/rowwise_sampling.cu:42-187."""
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    out_ptr, nnz = sample_counts(indptr, seeds, k, replace)
    row, col = np.empty(nnz, np.int64), np.empty(nnz, np.int64)
    pos = np.empty(nnz, np.int64) if want_pos else None
    lib().dgs_oracle_sample_uniform(_p(indptr), _p(indices), _p(seeds), ctypes.c_int64(seeds.size),
                                    ctypes.c_int64(k), ctypes.c_int32(int(replace)), _p(out_ptr),
                                    ctypes.c_uint64(rng_seed), _p(row), _p(col),
                                    _p(pos) if want_pos else None)
    return (row, col, pos, out_ptr) if want_pos else (row, col)


def sample_weighted(indptr, indices, probs, seeds, k, replace, rng_seed=0, want_pos=False):
    """RowWiseSamplingProbCUDA, src/cuda/rowwise_sampling_probs.cu:54-282."""
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    probs = np.ascontiguousarray(probs, dtype=np.float32)
    out_ptr, nnz = sample_counts(indptr, seeds, k, replace)
    row, col = np.empty(nnz, np.int64), np.empty(nnz, np.int64)
    pos = np.empty(nnz, np.int64) if want_pos else None
    lib().dgs_oracle_sample_weighted(_p(indptr), _p(indices), _p(probs), _p(seeds),
                                     ctypes.c_int64(seeds.size), ctypes.c_int64(k),
                                     ctypes.c_int32(int(replace)), _p(out_ptr),
                                     ctypes.c_uint64(rng_seed), _p(row), _p(col),
                                     _p(pos) if want_pos else None)
    return (row, col, pos, out_ptr) if want_pos else (row, col)


def unique(keys):
    """Unique, src/cuda/tensor_reindex.cu:82-159: distinct keys, first-occurrence order."""
    keys = _i64(keys).reshape(-1)
    out = np.empty(keys.size, np.int64)
    n = lib().dgs_oracle_unique(_p(keys), ctypes.c_int64(keys.size), _p(out))
    return out[:n].copy()


def relabel(uniq, x):
    """Relabel, src/cuda/tensor_reindex.cu:161-180: position in `uniq` or -1."""
    uniq, x = _i64(uniq), _i64(x).reshape(-1)
    out = np.empty(x.size, np.int64)
    lib().dgs_oracle_relabel(_p(uniq), ctypes.c_int64(uniq.size), _p(x), ctypes.c_int64(x.size),
                             _p(out))
    return out


def tensor_relabel(mapping, requiring):
    """TensorRelabelCUDA, src/cuda/tensor_reindex.cu:182-205."""
    u = unique(np.concatenate([_i64(m).reshape(-1) for m in mapping]) if mapping else np.empty(0, np.int64))
    return u, [relabel(u, r) for r in requiring]


def cache_fetch(cpu_data, gpu_flat, cache_keys, cache_vals, nid):
    """FetchDataCUDA, src/cuda/pagraph.cu:126-159,196-227."""
    cpu_data = np.ascontiguousarray(cpu_data)
    gpu_flat = np.ascontiguousarray(gpu_flat, dtype=cpu_data.dtype)
    D = cpu_data.shape[1]
    ck, cv, nid = _i64(cache_keys), _i64(cache_vals), _i64(nid)
    out = np.empty((nid.size, D), dtype=cpu_data.dtype)
    lib().dgs_oracle_cache_fetch(_p(cpu_data), _p(gpu_flat), ctypes.c_int32(cpu_data.dtype.itemsize),
                                 _p(ck), _p(cv), ctypes.c_int64(ck.size), _p(nid),
                                 ctypes.c_int64(nid.size), ctypes.c_int64(D), _p(out))
    return out


def sample_blocks(indptr, indices, seeds, fanouts, replace=False, probs=None, rng_seed=0):
    """The hot loop of ChunkTensorSampler.sample_blocks
    (oppo_bench/single_node/utils/chunktensor_sampler.py:93-118) without the DGL
    block object: per hop sample -> relabel([seeds, col], [row, col]).
    Returns (frontier, [(row_local, col_local, n_src, n_dst)] innermost first, total edges)."""
    seeds = _i64(seeds)
    blocks, edges = [], 0
    for hop, k in enumerate(reversed(list(fanouts))):
        if probs is None:
            row, col = sample_uniform(indptr, indices, seeds, k, replace, rng_seed + hop)
        else:
            row, col = sample_weighted(indptr, indices, probs, seeds, k, replace, rng_seed + hop)
        edges += row.size
        frontier, (r, c) = tensor_relabel([seeds, col], [row, col])
        blocks.insert(0, (r, c, frontier.size, seeds.size))
        seeds = frontier
    return seeds, blocks, edges


# --------------------------------------------------------------------------
# Checkers for stochastic rows (validity + distribution), shared by the tests.
# --------------------------------------------------------------------------
def check_sample(indptr, indices, seeds, k, replace, row, col, pos):
    """Structure every sampler output must satisfy (reference contracts:
    counts rowwise_sampling.cu:27-34; COO grouped by seed position; full rows
    in CSC order :66-72; picks are positions of the seed's row; distinct
    positions without replacement)."""
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    out_ptr, nnz = sample_counts(indptr, seeds, k, replace)
    assert row.size == nnz and col.size == nnz and pos.size == nnz, (row.size, nnz)
    cnt = np.diff(out_ptr)
    assert np.array_equal(row, np.repeat(seeds, cnt)), "coo_row must be seeds repeated by count"
    st = np.repeat(indptr[seeds], cnt)
    deg = np.repeat(indptr[seeds + 1] - indptr[seeds], cnt)
    assert np.all((pos >= 0) & (pos < deg)), "picked position outside the row"
    assert np.array_equal(col, indices[st + pos]), "coo_col must equal indices[row_start + pos]"
    if not replace:
        seg = np.repeat(np.arange(seeds.size), cnt)
        key = seg * (int(deg.max()) + 1 if nnz else 1) + pos
        assert np.unique(key).size == nnz, "duplicate position without replacement"
        full = deg <= k
        within = np.arange(nnz) - np.repeat(out_ptr[:-1], cnt)
        assert np.array_equal(pos[full], within[full]), "full rows must be copied in CSC order"
    return out_ptr
