"""Helpers for the GPU parity tests: call the C ABI with torch-owned memory."""
import ctypes

import numpy as np
import torch

from conftest import load_pkg

pkg = load_pkg()


def vp(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() else None


class Words:
    """Pinned words the kernels write sizes / status into."""

    def __init__(self):
        self.sizes = torch.zeros(8, dtype=torch.int64).pin_memory()
        self.status = torch.zeros(1, dtype=torch.int32).pin_memory()

    def take_status(self):
        torch.cuda.synchronize()
        s = int(self.status[0])
        self.status[0] = 0
        return s


def plain_desc(t):
    d = pkg.ChunkDesc()
    d.total = d.threshold = d.each = t.numel()
    d.num_parts, d.local_rank, d.esz = 1, 0, t.element_size()
    d.dev[0] = t.data_ptr()
    return d


class EmulatedChunks:
    """A multi-part ChunkTensor laid out on ONE GPU: every 'peer' chunk is a
    separate device buffer and the host tail is pinned memory, so the kernels'
    owner resolution, straddling rows and host reads are exercised without
    several GPUs.  Placement comes from the library's own dgs_placement."""

    def __init__(self, flat_np, D, capacity_per_gpu, world, rank=0):
        abi = pkg.load_abi()
        self.np = np.ascontiguousarray(flat_np).reshape(-1)
        self.D = D
        esz = self.np.dtype.itemsize
        e, t, h = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        pkg.check(abi.dgs_placement(self.np.size, esz, capacity_per_gpu, world, ctypes.byref(e),
                                    ctypes.byref(t), ctypes.byref(h)))
        self.each, self.thr, self.host_n = e.value, t.value, h.value
        raw = torch.from_numpy(self.np.view(np.uint8))
        self.parts = []
        for p in range(world):
            buf = torch.full((max(self.each * esz, 1),), 0xFF, dtype=torch.uint8, device="cuda")
            lo = p * self.each
            n = max(0, min(self.each, self.np.size - lo))
            if n > 0:
                buf[: n * esz] = raw[lo * esz:(lo + n) * esz].cuda()
            self.parts.append(buf)
        self.host = torch.zeros(max(self.host_n * esz, 1), dtype=torch.uint8).pin_memory()
        if self.host_n > 0:
            self.host[: self.host_n * esz] = raw[self.each * world * esz:]
        d = pkg.ChunkDesc()
        d.total, d.threshold, d.each = self.np.size, self.thr, self.each
        d.num_parts, d.local_rank, d.esz = world, rank, esz
        d.host = self.host.data_ptr() if self.host_n > 0 else None
        for p in range(world):
            d.dev[p] = self.parts[p].data_ptr()
        self.desc = d


def gather(desc, idx_t, D, dtype, words, cls=0):
    abi = pkg.load_abi()
    n = idx_t.numel()
    out = torch.empty((n, D), dtype=dtype, device="cuda")
    pkg.check(abi.dgs_gather_rows(ctypes.byref(desc), cls, vp(idx_t), int(idx_t.dtype == torch.int64), n, D,
                                  vp(out), vp(words.status), None))
    return out


def sample(indptr_desc, indices_desc, seeds_t, k, replace, words, probs_desc=None, rng=(1, 0)):
    """plan + sample through the C ABI; returns (row, col, pos) as numpy."""
    abi = pkg.load_abi()
    n = seeds_t.numel()
    ids64 = int(seeds_t.dtype == torch.int64)
    plan = torch.empty(abi.dgs_sample_plan_bytes(n), dtype=torch.uint8, device="cuda")
    cap = max(n * k, 1)
    row = torch.full((cap,), -7, dtype=seeds_t.dtype, device="cuda")
    col = torch.full((cap,), -7, dtype=seeds_t.dtype, device="cuda")
    pos = torch.full((cap,), -7, dtype=torch.int64, device="cuda")
    pkg.check(abi.dgs_sample_plan(ctypes.byref(indptr_desc), vp(seeds_t), ids64, n, k, int(replace), vp(plan),
                                  None, vp(words.status), None))
    if probs_desc is None:
        pkg.check(abi.dgs_sample_uniform(ctypes.byref(indices_desc), vp(seeds_t), ids64, n, k, int(replace),
                                         vp(plan), rng[0], rng[1], vp(row), vp(col), n * k,
                                         vp(words.sizes), vp(pos), vp(words.status), None))
    else:
        pkg.check(abi.dgs_sample_weighted(ctypes.byref(indices_desc), ctypes.byref(probs_desc), vp(seeds_t),
                                          ids64, n, k, int(replace), vp(plan), rng[0], rng[1],
                                          vp(row), vp(col), n * k, vp(words.sizes), vp(pos), vp(words.status),
                                          None))
    torch.cuda.synchronize()
    nnz = int(words.sizes[0])
    return row[:nnz].cpu().numpy(), col[:nnz].cpu().numpy(), pos[:nnz].cpu().numpy()


def segments(tensors):
    s = pkg.Segments()
    s.count = len(tensors)
    for i, t in enumerate(tensors):
        s.ptr[i] = t.data_ptr() if t.numel() else None
        s.len[i] = t.numel()
    return s


def unique_relabel(mapping, requiring, words):
    abi = pkg.load_abi()
    ids64 = int(mapping[0].dtype == torch.int64)
    n_keys = sum(t.numel() for t in mapping)
    tb = abi.dgs_relabel_table_bytes(n_keys)
    table = torch.empty(tb, dtype=torch.uint8, device="cuda")
    uniq = torch.empty(max(n_keys, 1), dtype=mapping[0].dtype, device="cuda")
    n_req = sum(t.numel() for t in requiring)
    out = torch.empty(max(n_req, 1), dtype=mapping[0].dtype, device="cuda")
    ks, rs = segments(mapping), segments(requiring)
    pkg.check(abi.dgs_unique_first_occurrence(ctypes.byref(ks), ids64, vp(table), tb, vp(uniq), vp(words.sizes),
                                              vp(words.status), None))
    pkg.check(abi.dgs_relabel_lookup(vp(table), tb, n_keys, ctypes.byref(rs), ids64, vp(out), None))
    torch.cuda.synchronize()
    nu = int(words.sizes[0])
    return uniq[:nu].cpu().numpy(), out[:n_req].cpu().numpy()
