"""dgs_split_index_static: the split-index entry point for hosts that are not
allowed to allocate device memory (its tile counters live in an array inside
the library instead of caller-provided scratch).

Collected last on purpose: a run that stops at the first failure has already
run every other test.  The check is against the regular entry point
(dgs_split_index with caller scratch) and against the CPU oracle: identical
ids, order and class sizes, on two calls in a row -- the second call finds the
first call's leftovers in the shared array and must not be disturbed by them --
and the device's free memory and torch's allocation count are the same before
and after the call.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_IDS = 1 << 24   # DGS_SPLIT_STATIC_MAX_IDS


def _both(pkg, desc, idx_t, D, sizes_a, sizes_b):
    """(regular, static) results for one id tensor."""
    from gpu_util import vp
    abi = pkg.load_abi()
    n = idx_t.numel()
    ids64 = int(idx_t.dtype == torch.int64)
    sb = abi.dgs_split_index_scratch_bytes(n)
    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
    ref = torch.full((max(n, 1),), -3, dtype=idx_t.dtype, device="cuda")
    got = torch.full((max(n, 1),), -5, dtype=idx_t.dtype, device="cuda")
    pkg.check(abi.dgs_split_index(ctypes.byref(desc), vp(idx_t), ids64, n, D, vp(ref), vp(sizes_a),
                                  vp(scratch), sb, None))
    torch.cuda.synchronize()
    free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    pkg.check(abi.dgs_split_index_static(ctypes.byref(desc), vp(idx_t), ids64, n, D, vp(got), vp(sizes_b), None))
    torch.cuda.synchronize()
    # the property in the entry point's name: nothing was allocated (or freed) on the device by the call
    assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == allocated_before
    return ref[:n].cpu(), sizes_a[:3].clone(), got[:n].cpu(), sizes_b[:3].clone()


def test_static_split_index_matches_regular_entry_point(pkg, oracle):
    from gpu_util import EmulatedChunks
    rng = np.random.default_rng(77)
    table = rng.standard_normal((5000, 6)).astype(np.float32)
    em = EmulatedChunks(table, 6, 4 * (6 * 1100 + 2), 3, rank=1)      # chunks + host tail, not row aligned
    cm = oracle.ChunkModel([5000, 6], np.float32, 4 * (6 * 1100 + 2), world=3)
    sizes_a = torch.zeros(8, dtype=torch.int64).pin_memory()
    sizes_b = torch.zeros(8, dtype=torch.int64).pin_memory()
    # two calls in a row with different sizes, contents and id types; then the first again
    calls = [(torch.int64, 300_001), (torch.int32, 4_097), (torch.int64, 300_001), (torch.int64, 0)]
    for dt, n in calls:
        idx_t = torch.from_numpy(rng.integers(0, 5000, size=n)).to(dt).cuda()
        ref, ca, got, cb = _both(pkg, em.desc, idx_t, 6, sizes_a, sizes_b)
        assert ca.tolist() == cb.tolist() and int(ca.sum()) == n
        assert torch.equal(ref, got)                                   # bit-exact: same ids, same order
        lo, re, ho = cm.split_index(idx_t.cpu().numpy().astype(np.int64), 1)     # and what the oracle says
        assert cb.tolist() == [lo.size, re.size, ho.size]
        assert got.tolist() == lo.tolist() + re.tolist() + ho.tolist()


def test_static_split_index_rejects_oversized_calls(pkg):
    from gpu_util import EmulatedChunks, vp
    abi = pkg.load_abi()
    em = EmulatedChunks(np.zeros((10, 4), np.float32), 4, 160, 1)
    idx = torch.zeros(16, dtype=torch.int64, device="cuda")
    out = torch.zeros(16, dtype=torch.int64, device="cuda")
    sizes = torch.full((8,), -1, dtype=torch.int64).pin_memory()
    rc = abi.dgs_split_index_static(ctypes.byref(em.desc), vp(idx), 1, MAX_IDS + 1, 4, vp(out), vp(sizes), None)
    assert rc == 5                                                      # DGS_ERR_UNSUPPORTED, nothing launched
    msg = abi.dgs_last_error().decode()
    assert str(MAX_IDS) in msg and "scratch" in msg
    torch.cuda.synchronize()
    assert sizes.tolist() == [-1] * 8
