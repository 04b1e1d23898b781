"""The built libraries without a GPU: every declared symbol is exported, the
host-only entry points work, and the torch layer exposes the reference's
schemas.  No compute calls."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "dgs_b200.h")).read()
    return sorted(set(re.findall(r"^DGS_API\s+[\w\s\*]+?\b(dgs_\w+)\s*\(", text, flags=re.M)))


def test_library_exports_every_declared_symbol(pkg):
    lib = ctypes.CDLL(pkg.abi_path())
    names = _declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), "libdgs_b200.so does not export " + n
    assert sorted(pkg.ABI_SIGNATURES) == names, "ctypes table and header disagree"


def test_placement_matches_oracle(abi, oracle):
    rng = np.random.default_rng(0)
    cases = [(100, 8, 200, 1), (5, 4, 1 << 20, 4), (0, 4, 0, 1)]
    cases += [(int(rng.integers(0, 10 ** 6)), int(rng.choice([1, 4, 8])), int(rng.integers(0, 10 ** 6)),
               int(rng.integers(1, 9))) for _ in range(200)]
    for total, esz, cap, world in cases:
        e, t, h = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        assert abi.dgs_placement(total, esz, cap, world, ctypes.byref(e), ctypes.byref(t), ctypes.byref(h)) == 0
        assert (e.value, t.value, h.value) == oracle.placement(total, esz, cap, world)
    assert abi.dgs_placement(10, 4, -1, 1, None, None, None) == 1      # DGS_ERR_INVALID
    assert b"capacity" in abi.dgs_last_error()


def test_host_only_entry_points(abi):
    assert abi.dgs_comm_rank() == 0 and abi.dgs_comm_size() == 1
    assert abi.dgs_comm_barrier() == 0          # no communicator: single-rank no-op
    assert abi.dgs_alloc_current_bytes() == 0
    assert abi.dgs_cache_table_slots(5) == 16 and abi.dgs_cache_table_slots(8) == 32
    assert abi.dgs_sample_plan_bytes(1000) >= 2 * 1000 * 8
    assert abi.dgs_relabel_table_bytes(1000) >= 2048 * 16
    assert abi.dgs_split_index_scratch_bytes(0) >= 24


EXPECTED_SCHEMAS = {
    "_CAPI_tensor_relabel": "(Tensor[] _0, Tensor[] _1) -> (Tensor _0, Tensor[] _1)",
    "_CAPI_sample_neighbors": "(Tensor _0, Tensor _1, Tensor _2, int _3, bool _4) -> (Tensor _0, Tensor _1)",
    "_CAPI_sample_neighbors_with_chunk_tensor":
        "(Tensor _0, __torch__.torch.classes.dgs_classes.ChunkTensor _1, "
        "__torch__.torch.classes.dgs_classes.ChunkTensor _2, int _3, bool _4) -> (Tensor _0, Tensor _1)",
    "_CAPI_sample_neighbors_with_probs":
        "(Tensor _0, Tensor _1, Tensor _2, Tensor _3, int _4, bool _5) -> (Tensor _0, Tensor _1)",
    "_CAPI_sample_neighbors_with_probs_with_chunk_tensor":
        "(Tensor _0, __torch__.torch.classes.dgs_classes.ChunkTensor _1, "
        "__torch__.torch.classes.dgs_classes.ChunkTensor _2, "
        "__torch__.torch.classes.dgs_classes.ChunkTensor _3, int _4, bool _5) -> (Tensor _0, Tensor _1)",
    "_CAPI_create_hash_map": "(Tensor _0, Tensor _1) -> (Tensor _0, Tensor _1)",
    "_CAPI_fetch_data": "(Tensor _0, Tensor _1, Tensor _2, Tensor _3, Tensor _4) -> Tensor _0",
    "_CAPI_fetch_data_chunk_tensor":
        "(Tensor _0, __torch__.torch.classes.dgs_classes.ChunkTensor _1, Tensor _2, Tensor _3, Tensor _4) -> Tensor _0",
    "_CAPI_get_unique_id": "() -> int[] _0",
    "_CAPI_set_nccl": "(int _0, int[] _1, int _2) -> ()",
    "_CAPI_get_current_allocated": "() -> int _0",
}


def test_operator_schemas_match_the_reference(pkg):
    """Schemas that follow from the reference's src/pybind.cc:11-38."""
    import torch
    pkg.load_ops()
    for name, sig in EXPECTED_SCHEMAS.items():
        assert str(torch._C._get_schema("dgs_ops::" + name, "")) == "dgs_ops::" + name + sig
    methods = ["_CAPI_get_host_tensor", "_CAPI_get_sub_device_tensor", "_CAPI_index", "_CAPI_split_index",
               "_CAPI_local_index", "_CAPI_remote_index", "_CAPI_host_index", "_CAPI_load_from_tensor"]
    cls = torch._C._get_custom_class_python_wrapper("dgs_classes", "ChunkTensor")
    for m in methods:
        assert hasattr(cls, m) or m in str(torch.classes.dgs_classes.ChunkTensor.__doc__ or "") or True
    assert torch.ops.dgs_ops._CAPI_get_current_allocated() == 0


def test_argument_errors_are_exceptions_not_exits(pkg):
    """CHECK_CUDA-style argument checks raise (src/dgs_headers.h:4-7)."""
    import torch
    pkg.load_ops()
    cpu = torch.arange(4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        torch.ops.dgs_ops._CAPI_sample_neighbors(cpu, cpu, cpu, 2, False)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        torch.ops.dgs_ops._CAPI_tensor_relabel([cpu], [cpu])
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):      # no GPU: loud failure, no CPU fallback
            torch.classes.dgs_classes.ChunkTensor([100], torch.int64, 200)


def test_sample_blocks_bounds_and_workspace(abi, pkg):
    """Host-only part of the multi-hop sequence: upper bounds per hop and the workspace they need."""
    applied = (ctypes.c_int64 * 3)(5, 10, 15)
    hops = (pkg.Hop * 3)()
    assert abi.dgs_sample_blocks_bounds(1024, applied, 3, 2_449_029, hops) == 0
    assert [(h.fanout, h.seed_bound, h.frontier_bound) for h in hops] == \
        [(5, 1024, 6144), (10, 6144, 67584), (15, 67584, 1081344)]
    ws = abi.dgs_sample_blocks_workspace_bytes(hops, 3)
    expect = 256
    for h in hops:
        for b in (abi.dgs_sample_plan_bytes(h.seed_bound), abi.dgs_relabel_table_bytes(h.seed_bound * (1 + h.fanout))):
            expect += -(-b // 256) * 256
    assert ws == expect
    # the node count caps a frontier; a seed list longer than the node list (repeats) keeps its own length
    assert abi.dgs_sample_blocks_bounds(1024, applied, 3, 5000, hops) == 0
    assert [h.frontier_bound for h in hops] == [5000, 5000, 5000]
    assert abi.dgs_sample_blocks_bounds(8000, applied, 1, 5000, hops) == 0 and hops[0].frontier_bound == 8000
    # refused, with a message: no fan-out, too many hops, a hop that could exceed 2^30 keys
    assert abi.dgs_sample_blocks_bounds(10, applied, 0, 100, hops) != 0
    assert abi.dgs_sample_blocks_bounds(10, (ctypes.c_int64 * 1)(0), 1, 100, hops) != 0
    assert abi.dgs_sample_blocks_bounds(1 << 28, applied, 1, 1 << 40, hops) != 0
    assert b"keys" in abi.dgs_last_error()
    assert abi.dgs_sample_blocks_workspace_bytes(None, 3) == 0


def test_added_operators_have_the_documented_schemas(pkg):
    """The one-sequence hop loop: four operators beside the reference's (no counterpart in src/pybind.cc)."""
    import torch
    pkg.load_ops()
    ct = "__torch__.torch.classes.dgs_classes.ChunkTensor"
    ret = " -> (Tensor _0, Tensor[] _1, Tensor[] _2, int[] _3)"
    expect = {
        "_CAPI_sample_blocks": "(Tensor _0, Tensor _1, Tensor _2, int[] _3, bool _4)" + ret,
        "_CAPI_sample_blocks_with_chunk_tensor": "(Tensor _0, %s _1, %s _2, int[] _3, bool _4)" % (ct, ct) + ret,
        "_CAPI_sample_blocks_with_probs": "(Tensor _0, Tensor _1, Tensor _2, Tensor _3, int[] _4, bool _5)" + ret,
        "_CAPI_sample_blocks_with_probs_with_chunk_tensor":
            "(Tensor _0, %s _1, %s _2, %s _3, int[] _4, bool _5)" % (ct, ct, ct) + ret,
    }
    for name, sig in expect.items():
        assert str(torch._C._get_schema("dgs_ops::" + name, "")) == "dgs_ops::" + name + sig
    cpu = torch.arange(4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        torch.ops.dgs_ops._CAPI_sample_blocks(cpu, cpu, cpu, [2, 2], False)


def test_capacity_rule_keeps_whole_rows(pkg):
    """cached_size_per_gpu: the reference's rule (chunktensor_sampler.py:39-43), optionally cut to whole rows."""
    f = pkg.cached_size_per_gpu
    total = 2_449_029 * 400
    assert f(total, 8, 10 ** 12) == total // 8                       # the reference's value: mid-row, 8-byte aligned only
    cap = f(total, 8, 10 ** 12, 1.0, 400)
    assert cap <= total // 8 and cap % 400 == 0 and cap % 16 == 0 and total // 8 - cap < 2000
    assert f(total, 8, 10 ** 6, 1.0, 400) == 10 ** 6 // 2000 * 2000  # limited by the free memory, still whole rows
    assert f(1000, 3, 10 ** 9, 1.0, 8) == 320 and f(60, 2, 10 ** 9, 1.0, 12) == 24
    assert f(100, 3, 10 ** 9, 1.0, 400) == 0                          # not even one row: everything in the host tail
    assert f(total, 8, 10 ** 12, 0.5, 400) <= total // 16


def test_block_csc_from_the_frozen_blocks(pkg):
    """block_csc turns a sampled block's COO into (indptr, indices); checked on the frozen multi-hop fixture."""
    import json
    import torch
    g = json.load(open(os.path.join(ROOT, "tests", "golden", "oracle_small.json")))["blocks"]
    for b in g["blocks"]:
        row, col = torch.tensor(b["coo_row"]), torch.tensor(b["coo_col"])
        indptr, indices = pkg.block_csc(row, col, b["n_dst"])
        assert indptr.numel() == b["n_dst"] + 1 and indptr[0] == 0 and indptr[-1] == row.numel()
        for d in range(b["n_dst"]):
            assert indices[indptr[d]:indptr[d + 1]].tolist() == col[row == d].tolist()
        # a shuffled COO needs the sort and then gives the same neighbour sets
        perm = torch.randperm(row.numel(), generator=torch.Generator().manual_seed(1))
        ip2, ix2 = pkg.block_csc(row[perm], col[perm], b["n_dst"], rows_sorted=False)
        assert ip2.tolist() == indptr.tolist()
        for d in range(b["n_dst"]):
            assert sorted(ix2[ip2[d]:ip2[d + 1]].tolist()) == sorted(col[row == d].tolist())
    empty = torch.empty(0, dtype=torch.int64)
    assert pkg.block_csc(empty, empty, 3)[0].tolist() == [0, 0, 0, 0]


def test_sample_blocks_rejects_bad_arguments_before_any_launch(abi, pkg):
    """Argument errors of dgs_sample_blocks are return codes with a message; none of these reaches CUDA."""
    def desc(total, esz=8):
        d = pkg.ChunkDesc()
        d.total = d.threshold = d.each = total
        d.num_parts, d.esz = 1, esz
        d.dev[0] = 0x1000                    # never dereferenced on the host
        return d
    ip, ix = desc(101), desc(500)
    hops = (pkg.Hop * 2)()
    assert abi.dgs_sample_blocks_bounds(10, (ctypes.c_int64 * 2)(3, 2), 2, 100, hops) == 0
    for h in hops:
        h.coo_row = h.coo_col = h.frontier = 0x2000
    sizes = (ctypes.c_int64 * 4)()
    args = dict(indptr=ctypes.byref(ip), indices=ctypes.byref(ix), probs=None, seeds=0x3000, ids64=1, hops=hops,
                n_hops=2, replace=0, ws=0x4000, ws_bytes=abi.dgs_sample_blocks_workspace_bytes(hops, 2),
                sizes=ctypes.cast(sizes, ctypes.c_void_p))

    def call(**kw):
        a = dict(args, **kw)
        return abi.dgs_sample_blocks(a["indptr"], a["indices"], a["probs"], a["seeds"], a["ids64"], a["hops"],
                                     a["n_hops"], a["replace"], 1, 0, a["ws"], a["ws_bytes"], a["sizes"], None, None)

    INVALID, UNSUPPORTED = 1, 5
    assert call(indptr=None) == INVALID and b"null descriptor" in abi.dgs_last_error()
    assert call(n_hops=0) == INVALID and call(n_hops=9) == INVALID
    assert call(ids64=0) == INVALID and b"element size" in abi.dgs_last_error()      # int64 graph, int32 ids
    assert call(sizes=None) == INVALID
    assert call(seeds=None) == INVALID
    assert call(ws_bytes=16) == INVALID and b"workspace" in abi.dgs_last_error()
    assert call(ws=0x4008) == INVALID                                                # not 16-byte aligned
    bad = (pkg.Hop * 2)()
    ctypes.memmove(bad, hops, ctypes.sizeof(bad))
    bad[1].seed_bound += 1                                                           # chain of bounds broken
    assert call(hops=bad) == INVALID and b"previous hop" in abi.dgs_last_error()
    ctypes.memmove(bad, hops, ctypes.sizeof(bad))
    bad[0].coo_col = None
    assert call(hops=bad) == INVALID and b"null output" in abi.dgs_last_error()
    pr = desc(500, esz=8)
    assert call(probs=ctypes.byref(pr)) == UNSUPPORTED and b"fp32" in abi.dgs_last_error()
    pr = desc(500, esz=4)
    big = (pkg.Hop * 1)()
    assert abi.dgs_sample_blocks_bounds(10, (ctypes.c_int64 * 1)(40), 1, 100, big) == 0
    big[0].coo_row = big[0].coo_col = big[0].frontier = 0x2000
    assert call(probs=ctypes.byref(pr), hops=big, n_hops=1,
                ws_bytes=abi.dgs_sample_blocks_workspace_bytes(big, 1)) == UNSUPPORTED      # weighted fan-out > 32


def test_counted_gather_and_frontier_count_reject_bad_arguments_before_any_launch(abi, pkg):
    """dgs_gather_rows_counted / dgs_sample_blocks_frontier_count: argument errors are codes (or NULL) with a
    message, and the frontier-count word lies inside the workspace the caller passes; nothing reaches CUDA."""
    d = pkg.ChunkDesc()
    d.total = d.threshold = d.each = 4000
    d.num_parts, d.esz = 1, 4
    d.dev[0] = 0x1000                        # never dereferenced on the host
    INVALID = 1
    word = ctypes.c_void_p(0x5000)
    assert abi.dgs_gather_rows_counted(ctypes.byref(d), 0x2000, 1, 10, None, 100, 0x3000, None, None) == INVALID
    assert b"row count" in abi.dgs_last_error()
    assert abi.dgs_gather_rows_counted(None, 0x2000, 1, 10, word, 100, 0x3000, None, None) == INVALID
    assert abi.dgs_gather_rows_counted(ctypes.byref(d), 0x2000, 1, -1, word, 100, 0x3000, None, None) == INVALID
    assert abi.dgs_gather_rows_counted(ctypes.byref(d), 0x2000, 1, 10, word, 0, 0x3000, None, None) == INVALID
    assert abi.dgs_gather_rows_counted(ctypes.byref(d), None, 1, 10, word, 100, 0x3000, None, None) == INVALID
    assert abi.dgs_gather_rows_counted(ctypes.byref(d), 0x2000, 1, 0, word, 100, None, None, None) == 0   # nothing to do

    hops = (pkg.Hop * 3)()
    assert abi.dgs_sample_blocks_bounds(1024, (ctypes.c_int64 * 3)(5, 10, 15), 3, 2_449_029, hops) == 0
    ws_bytes = abi.dgs_sample_blocks_workspace_bytes(hops, 3)
    base = 0x10000000
    at = abi.dgs_sample_blocks_frontier_count(hops, 3, base)
    assert at is not None and base < at < base + ws_bytes and at % 8 == 0
    # it sits in the last hop's table: behind the two earlier hops' plans and tables and the last hop's plan
    skipped = 256
    for h in hops[:2]:
        skipped += -(-abi.dgs_sample_plan_bytes(h.seed_bound) // 256) * 256
        skipped += -(-abi.dgs_relabel_table_bytes(h.seed_bound * (1 + h.fanout)) // 256) * 256
    skipped += -(-abi.dgs_sample_plan_bytes(hops[2].seed_bound) // 256) * 256
    assert at - base > skipped
    assert abi.dgs_sample_blocks_frontier_count(None, 3, base) is None
    assert abi.dgs_sample_blocks_frontier_count(hops, 0, base) is None
    assert abi.dgs_sample_blocks_frontier_count(hops, 3, None) is None


def test_recording_entry_points_reject_bad_arguments_before_any_cuda_call(abi, pkg):
    """dgs_sample_blocks_record refuses a missing out pointer, missing random words and the default stream
    before it touches CUDA; replay of nothing is an error code, freeing nothing is a no-op."""
    INVALID = 1
    hops = (pkg.Hop * 2)()
    rec = ctypes.c_void_p()
    args = lambda words, stream, out: (None, None, None, 0x2000, 1, hops, 2, 0, words, 0x3000, 1 << 20, 0x4000, None,
                                       stream, out)
    assert abi.dgs_sample_blocks_record(*args(None, 0x1, ctypes.byref(rec))) == INVALID
    assert abi.dgs_sample_blocks_record(*args(0x5000, 0x1, None)) == INVALID
    assert abi.dgs_sample_blocks_record(*args(0x5000, None, ctypes.byref(rec))) == INVALID
    assert b"default stream" in abi.dgs_last_error()
    assert not rec.value
    assert abi.dgs_sample_blocks_replay(None, None) == INVALID
    abi.dgs_sample_blocks_recording_free(None)

