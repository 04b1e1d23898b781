"""Row gather / split-index on the GPU against the CPU oracle (bit-exact)."""
import ctypes
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def words():
    from gpu_util import Words
    return Words()


CASES = [
    # rows, D, dtype, capacity elems per gpu, world
    (1000, 128, np.float32, 10 ** 9, 1),       # all in one chunk
    (1000, 128, np.float32, 128 * 100, 4),     # row-aligned chunks + host tail
    (1000, 100, np.float32, 100 * 77 + 36, 3), # 400-byte rows, non-row-aligned: rows straddle every boundary
    (777, 64, np.float32, 64 * 50 + 2, 8),     # 8-byte aligned bases only
    (500, 3, np.float32, 101, 2),              # 12-byte rows
    (4096, 1, np.int64, 300, 5),               # 1-D tensor -> [n, 1]
    (300, 7, np.bool_, 400, 2),                # 1-byte elements
    (64, 256, np.float32, 256 * 8, 2),         # 1 KB rows
    (5, 5000, np.float32, 6000, 2),            # rows larger than a tile
    (123, 8, np.float64, 0, 1),                # everything in the host tail
    (10, 4, np.int32, 3, 4),                   # chunks smaller than a row: a row spans several chunks
]


@pytest.mark.parametrize("rows,D,dtype,cap_elems,world", CASES)
@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_gather_matches_oracle(oracle, words, rows, D, dtype, cap_elems, world, idx_dtype):
    from gpu_util import EmulatedChunks, gather
    rng = np.random.default_rng(rows * 31 + D)
    if dtype == np.bool_:
        table = rng.integers(0, 2, size=(rows, D)).astype(np.bool_)
    elif np.issubdtype(dtype, np.integer):
        table = rng.integers(-2 ** 31, 2 ** 31 - 1, size=(rows, D)).astype(dtype)
    else:
        table = rng.standard_normal((rows, D)).astype(dtype)
    esz = table.dtype.itemsize
    cm = oracle.ChunkModel([rows, D] if D > 1 else [rows], dtype, cap_elems * esz, world=world)
    cm.load(table)
    em = EmulatedChunks(table, D, cap_elems * esz, world)
    assert (em.each, em.thr) == (cm.each, cm.thr)
    idx = np.concatenate([rng.integers(0, rows, size=3000), np.arange(rows), [0, rows - 1]])
    idx_t = torch.from_numpy(idx).to(idx_dtype).cuda()
    tdt = {np.float32: torch.float32, np.float64: torch.float64, np.int64: torch.int64,
           np.int32: torch.int32, np.bool_: torch.bool}[dtype]
    out = gather(em.desc, idx_t, D, tdt, words)
    assert words.take_status() == 0
    assert out.cpu().numpy().tobytes() == cm.index(idx).tobytes()


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_gather_with_a_device_side_row_count(pkg, words, idx_dtype):
    """dgs_gather_rows_counted: the request length is a device word (as the frontier length of a queued
    sample_blocks sequence is); rows up to min(word, bound) are gathered, nothing is written past them."""
    import ctypes
    from gpu_util import EmulatedChunks, vp
    abi = pkg.load_abi()
    rng = np.random.default_rng(12)
    rows, D = 300_000, 100
    table = rng.standard_normal((rows, D)).astype(np.float32)
    em = EmulatedChunks(table, D, 4 * (D * 70_000 + 36), 4)       # 4 chunks + host tail, straddling rows
    idx = rng.integers(0, rows, size=200_001)
    idx_t = torch.from_numpy(idx).to(idx_dtype).cuda()
    for live, bound in ((150_003, 200_001), (0, 200_001), (200_001, 200_001), (10 ** 9, 70_000), (-5, 1000)):
        n_dev = torch.tensor([live], dtype=torch.int64, device="cuda")
        out = torch.full((bound, D), -7.0, dtype=torch.float32, device="cuda")
        pkg.check(abi.dgs_gather_rows_counted(ctypes.byref(em.desc), vp(idx_t), int(idx_dtype == torch.int64), bound,
                                              vp(n_dev), D, vp(out), vp(words.status), None))
        assert words.take_status() == 0
        n = max(0, min(live, bound))
        got = out.cpu().numpy()
        assert got[:n].tobytes() == table[idx[:n]].tobytes()
        assert (got[n:] == -7.0).all()
    rc = abi.dgs_gather_rows_counted(ctypes.byref(em.desc), vp(idx_t), 1, 10, None, D, vp(out), None, None)
    assert rc == 1 and b"row count" in abi.dgs_last_error()


def test_gather_empty_and_out_of_range(words):
    from gpu_util import EmulatedChunks, gather
    table = np.arange(40 * 8, dtype=np.float32).reshape(40, 8)
    em = EmulatedChunks(table, 8, 8 * 4 * 10, 2)
    out = gather(em.desc, torch.empty(0, dtype=torch.int64, device="cuda"), 8, torch.float32, words)
    assert out.shape == (0, 8) and words.take_status() == 0
    idx = torch.tensor([3, 40, -1, 39], device="cuda")
    out = gather(em.desc, idx, 8, torch.float32, words).cpu().numpy()
    assert words.take_status() == 6                      # DGS_ERR_RANGE, no fault
    assert out[0].tolist() == table[3].tolist() and out[3].tolist() == table[39].tolist()
    assert not out[1].any() and not out[2].any()          # zero rows


def test_gather_large_is_index_select(words):
    """Size-independent property at benchmark scale: gather == torch index_select."""
    from gpu_util import plain_desc, gather
    g = torch.Generator(device="cuda").manual_seed(1)
    table = torch.randn(1_000_000, 128, device="cuda", generator=g)
    idx = torch.randint(0, 1_000_000, (3_000_000,), device="cuda", generator=g)
    out = gather(plain_desc(table), idx, 128, torch.float32, words)
    assert words.take_status() == 0
    assert torch.equal(out, table[idx])
    t100 = table[:, :100].contiguous()
    assert torch.equal(gather(plain_desc(t100), idx[:500_000], 100, torch.float32, words), t100[idx[:500_000]])


def test_gather_offsets_beyond_4_gib(words):
    """Table and result both larger than 2^32 bytes: every byte offset is 64-bit."""
    from gpu_util import plain_desc, gather
    g = torch.Generator(device="cuda").manual_seed(2)
    rows = 9_000_000                                     # x 512 B = 4.6 GB
    table = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, 128), device="cuda", generator=g, dtype=torch.int32)
    idx = torch.randint(0, rows, (rows,), device="cuda", generator=g)
    idx[-1] = rows - 1
    out = gather(plain_desc(table), idx, 128, torch.int32, words)
    assert words.take_status() == 0
    for lo in range(0, rows, 3_000_000):
        assert torch.equal(out[lo:lo + 3_000_000], table[idx[lo:lo + 3_000_000]])


def test_split_index_matches_oracle(oracle, words, pkg):
    from gpu_util import EmulatedChunks, vp
    abi = pkg.load_abi()
    rng = np.random.default_rng(4)
    table = rng.standard_normal((1000, 6)).astype(np.float32)
    for world, cap in [(3, 4 * 50 * 6 + 8), (1, 4 * 6 * 400), (4, 0)]:
        for rank in range(world):
            em = EmulatedChunks(table, 6, cap, world, rank=rank)
            for n in [0, 1, 5000, 2048 * 3 + 17]:
                idx = rng.integers(0, 1000, size=n)
                for dt in (torch.int64, torch.int32):
                    idx_t = torch.from_numpy(idx).to(dt).cuda()
                    out = torch.empty(max(n, 1), dtype=dt, device="cuda")
                    sb = abi.dgs_split_index_scratch_bytes(n)
                    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
                    pkg.check(abi.dgs_split_index(ctypes.byref(em.desc), vp(idx_t), int(dt == torch.int64), n, 6,
                                                  vp(out), vp(words.sizes), vp(scratch), sb, None))
                    torch.cuda.synchronize()
                    nl, nr, nh = (int(x) for x in words.sizes[:3])
                    lo, re, ho = oracle.split_index(idx, 6, em.each, em.thr, rank)
                    got = out.cpu().numpy()
                    assert (nl, nr, nh) == (lo.size, re.size, ho.size)
                    assert got[:nl].tolist() == lo.tolist()
                    assert got[nl:nl + nr].tolist() == re.tolist()
                    assert got[nl + nr:n].tolist() == ho.tolist()


def test_chunktensor_class_readme_demo(ops):
    """The reference's demo (example/demo.py:23-36) through the drop-in class."""
    g = json.load(open(os.path.join(GOLDEN, "readme_demo.json")))
    c = torch.classes.dgs_classes.ChunkTensor(g["shape"], torch.int64, g["capacity_per_gpu"])
    c._CAPI_load_from_tensor(torch.arange(100))
    assert c._CAPI_get_host_tensor().tolist() == g["host_tensor"]
    dev = c._CAPI_get_sub_device_tensor()
    assert dev.is_cuda and dev.tolist() == g["device_tensor"]
    assert torch.ops.dgs_ops._CAPI_get_current_allocated() == 200
    idx = torch.tensor([99, 0, 24, 25, 50], device="cuda")
    assert c._CAPI_index(idx).reshape(-1).tolist() == [99, 0, 24, 25, 50]
    lo, re, ho = c._CAPI_split_index(idx)
    assert (lo.tolist(), re.tolist(), ho.tolist()) == ([0, 24], [], [99, 25, 50])
    assert c._CAPI_local_index(lo).reshape(-1).tolist() == [0, 24]
    assert c._CAPI_host_index(ho).reshape(-1).tolist() == [99, 25, 50]
    assert c._CAPI_remote_index(re).shape == (0, 1)
    # chunks can be filled in place through the views, as the reference's benchmarks do
    c._CAPI_get_sub_device_tensor().fill_(7)
    c._CAPI_get_host_tensor().fill_(9)
    assert c._CAPI_index(idx).reshape(-1).tolist() == [9, 7, 7, 9, 9]
    del c, dev
    assert torch.ops.dgs_ops._CAPI_get_current_allocated() == 0


def test_chunktensor_class_features(ops, oracle):
    rng = np.random.default_rng(8)
    table = rng.standard_normal((5000, 100)).astype(np.float32)
    cap = 100 * 4 * 3000 + 40   # 3000.1 rows on the GPU: one row straddles into the host tail
    c = torch.classes.dgs_classes.ChunkTensor([5000, 100], torch.float32, cap)
    c._CAPI_load_from_tensor(torch.from_numpy(table))
    cm = oracle.ChunkModel([5000, 100], np.float32, cap, world=1)
    cm.load(table)
    idx = rng.integers(0, 5000, size=20000)
    out = c._CAPI_index(torch.from_numpy(idx).cuda())
    assert out.shape == (20000, 100) and out.cpu().numpy().tobytes() == cm.index(idx).tobytes()
    out32 = c._CAPI_index(torch.from_numpy(idx).int().cuda())
    assert torch.equal(out, out32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        c._CAPI_index(torch.from_numpy(idx))
    with pytest.raises(RuntimeError):
        c._CAPI_load_from_tensor(torch.zeros(5000, 100, dtype=torch.float64))
    # an out-of-range id is reported at the next call instead of faulting
    c._CAPI_index(torch.tensor([5000], device="cuda"))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="out-of-range"):
        c._CAPI_index(torch.tensor([1], device="cuda"))
    assert c._CAPI_index(torch.tensor([1], device="cuda")).cpu().numpy().tobytes() == table[1].tobytes()


def test_chunktensor_index_counted(ops):
    """_CAPI_index_counted: the row count is an int64 word on the device; rows past it are left untouched,
    a count beyond the request is clamped; 512-byte rows take the bulk-copy form, 36-byte rows the other."""
    rng = np.random.default_rng(9)
    for D in (128, 9):
        table = rng.standard_normal((6000, D)).astype(np.float32)
        c = torch.classes.dgs_classes.ChunkTensor([6000, D], torch.float32, 4 * D * 4000)   # 2 000 rows on the host
        c._CAPI_load_from_tensor(torch.from_numpy(table))
        idx = torch.from_numpy(rng.integers(0, 6000, size=5000)).cuda()
        whole = c._CAPI_index(idx)
        for live in (0, 1, 777, 5000, 9999):
            count = torch.tensor([live], dtype=torch.int64, device="cuda")
            out = c._CAPI_index_counted(idx, count)
            n = min(live, 5000)
            assert out.shape == (5000, D) and torch.equal(out[:n], whole[:n])
        with pytest.raises(RuntimeError, match="int64"):
            c._CAPI_index_counted(idx, torch.tensor([5], dtype=torch.int32, device="cuda"))
        del c

