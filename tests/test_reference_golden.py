"""Golden vectors recorded from the reference's own kernels on a B200
(tests/golden/reference_b200.json, made by tests/golden/make_reference_golden.py
with the library of oracle/build_reference.sh).

CPU part: the oracle reproduces them -- this is what pins the oracle to the
reference for index, split-index, relabel, full-row sampling and the cache fetch.
GPU part: this repository's operators reproduce them bit for bit.
"""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.json")


@pytest.fixture(scope="module")
def ref():
    return json.load(open(GOLDEN))


def _bits(x):
    return np.array(x, dtype=np.int32).view(np.float32)


# --------------------------------------------------------------------------- CPU: oracle == reference
def test_oracle_matches_reference_placement_and_index(oracle, ref):
    d = ref["demo"]
    cm = oracle.ChunkModel([100], np.int64, 200)
    cm.load(np.arange(100))
    assert cm.host_tensor().tolist() == d["host"] and cm.sub_device_tensor(0).tolist() == d["device"]
    # the reference also counts its device-side accessor (8 bytes per chunk pointer + a 48-byte
    # struct, src/chunk_tensor.cc:143-148,223-233); this library passes the placement by value
    assert d["allocated"] == 200 + 8 + 48
    t = ref["table"]
    table = np.array(t["table"], dtype=np.int32)
    cm = oracle.ChunkModel(table.shape, np.int32, t["capacity_per_gpu"])
    cm.load(table)
    assert cm.host_tensor().tolist() == t["host_view"] and cm.sub_device_tensor(0).tolist() == t["device_view"]
    idx = np.array(t["idx"])
    assert cm.index(idx).tolist() == t["index"] == t["index_i32"]
    assert [x.tolist() for x in cm.split_index(idx, 0)] == t["split"]
    assert cm.index(np.array(t["local_ids"])).tolist() == t["local_index"]
    assert cm.index(np.array(t["host_ids"])).tolist() == t["host_index"]
    f = ref["float_table"]
    feats = _bits(f["table_bits"])
    assert oracle.index_flat(feats, np.array(f["idx"])).view(np.int32).tolist() == f["index_bits"]


def test_oracle_matches_reference_relabel(oracle, ref):
    for name in ("relabel_i64", "relabel_i32"):
        r = ref[name]
        seeds, col = np.array(r["seeds"]), np.array(r["col"])
        u, (ro, co) = oracle.tensor_relabel([seeds, col], [np.repeat(seeds, 10), col])
        assert u.tolist() == r["frontier"] and ro.tolist() == r["row_out"] and co.tolist() == r["col_out"]
    a = ref["relabel_absent"]
    u, (q,) = oracle.tensor_relabel([np.array(a["mapping"])], [np.array(a["query"])])
    assert u.tolist() == a["frontier"] and q.tolist() == a["out"] and -1 in a["out"]


def test_oracle_matches_reference_sampling(oracle, ref):
    g = ref["full_rows"]
    indptr, indices, seeds = np.array(g["indptr"]), np.array(g["indices"]), np.array(g["seeds"])
    probs = _bits(g["probs_bits"])
    row, col = oracle.sample_uniform(indptr, indices, seeds, g["k"], False)
    for name in ("plain", "chunk", "probs", "probs_chunk"):
        assert row.tolist() == g[name]["coo_row"] and col.tolist() == g[name]["coo_col"], name
    row, col = oracle.sample_weighted(indptr, indices, probs, seeds, g["k"], False)
    assert row.tolist() == g["probs"]["coo_row"] and col.tolist() == g["probs"]["coo_col"]
    m = ref["mixed_rows"]
    indptr, seeds = np.array(m["indptr"]), np.array(m["seeds"])
    for rep in (0, 1):
        out_ptr, nnz = oracle.sample_counts(indptr, seeds, m["k"], bool(rep))
        exp = np.repeat(seeds, np.diff(out_ptr)).tolist()
        assert m["uniform_replace%d_coo_row" % rep] == exp and m["weighted_replace%d_coo_row" % rep] == exp
        assert m["uniform_replace%d_valid" % rep] and m["weighted_replace%d_valid" % rep]


def test_oracle_matches_reference_cache_fetch(oracle, ref):
    c = ref["cache"]
    cpu = _bits(c["cpu_bits"])
    gpu = _bits(c["gpu_bits"])
    out = oracle.cache_fetch(cpu, gpu, np.array(c["hot"]), np.arange(len(c["hot"])), np.array(c["nid"]))
    assert out.view(np.int32).tolist() == c["fetched_bits"]


# --------------------------------------------------------------------------- GPU: this library == reference
@pytest.mark.gpu
def test_operators_match_reference_index(ops, ref):
    import torch
    CT = torch.classes.dgs_classes.ChunkTensor
    t = ref["table"]
    table = torch.tensor(t["table"], dtype=torch.int32)
    c = CT(list(table.shape), torch.int32, t["capacity_per_gpu"])
    c._CAPI_load_from_tensor(table)
    assert c._CAPI_get_host_tensor().tolist() == t["host_view"]
    assert c._CAPI_get_sub_device_tensor().tolist() == t["device_view"]
    idx = torch.tensor(t["idx"], device="cuda")
    assert c._CAPI_index(idx).tolist() == t["index"]
    assert c._CAPI_index(idx.int()).tolist() == t["index_i32"]
    assert [x.tolist() for x in c._CAPI_split_index(idx)] == t["split"]
    assert c._CAPI_local_index(torch.tensor(t["local_ids"], device="cuda")).tolist() == t["local_index"]
    assert c._CAPI_host_index(torch.tensor(t["host_ids"], device="cuda")).tolist() == t["host_index"]
    f = ref["float_table"]
    feats = torch.from_numpy(_bits(f["table_bits"]).copy())
    cf = CT(list(feats.shape), torch.float32, feats.numel() * 4)
    cf._CAPI_load_from_tensor(feats)
    got = cf._CAPI_index(torch.tensor(f["idx"], device="cuda")).cpu().numpy().view(np.int32)
    assert got.tolist() == f["index_bits"]


@pytest.mark.gpu
def test_operators_match_reference_relabel_sampling_cache(ops, ref):
    import torch

    def dev(a, dt=torch.int64):
        return torch.tensor(a, dtype=dt, device="cuda")

    for name, dt in (("relabel_i64", torch.int64), ("relabel_i32", torch.int32)):
        r = ref[name]
        seeds, col = dev(r["seeds"], dt), dev(r["col"], dt)
        f, (ro, co) = ops._CAPI_tensor_relabel([seeds, col], [seeds.repeat_interleave(10), col])
        assert f.tolist() == r["frontier"] and ro.tolist() == r["row_out"] and co.tolist() == r["col_out"]
    a = ref["relabel_absent"]
    f, (q,) = ops._CAPI_tensor_relabel([dev(a["mapping"])], [dev(a["query"])])
    assert f.tolist() == a["frontier"] and q.tolist() == a["out"]

    g = ref["full_rows"]
    ip, ix, sd = dev(g["indptr"]), dev(g["indices"]), dev(g["seeds"])
    pr = torch.from_numpy(_bits(g["probs_bits"]).copy()).cuda()
    CT = torch.classes.dgs_classes.ChunkTensor
    c_ip, c_ix, c_pr = CT([ip.numel()], torch.int64, 8 * 20), CT([ix.numel()], torch.int64, 8 * 50), \
        CT([ix.numel()], torch.float32, 4 * 64)
    c_ip._CAPI_load_from_tensor(ip.cpu())
    c_ix._CAPI_load_from_tensor(ix.cpu())
    c_pr._CAPI_load_from_tensor(pr.cpu())
    calls = {"plain": lambda: ops._CAPI_sample_neighbors(sd, ip, ix, g["k"], False),
             "chunk": lambda: ops._CAPI_sample_neighbors_with_chunk_tensor(sd, c_ip, c_ix, g["k"], False),
             "probs": lambda: ops._CAPI_sample_neighbors_with_probs(sd, ip, ix, pr, g["k"], False),
             "probs_chunk": lambda: ops._CAPI_sample_neighbors_with_probs_with_chunk_tensor(sd, c_ip, c_ix, c_pr,
                                                                                         g["k"], False)}
    for name, fn in calls.items():
        row, col = fn()
        assert row.tolist() == g[name]["coo_row"] and col.tolist() == g[name]["coo_col"], name

    m = ref["mixed_rows"]
    ip2, sd2 = dev(m["indptr"]), dev(m["seeds"])
    ix2 = torch.arange(int(m["indptr"][-1]), device="cuda") % 60
    pr2 = torch.rand(ix2.numel(), device="cuda") + 0.1
    for rep in (False, True):
        assert ops._CAPI_sample_neighbors(sd2, ip2, ix2, m["k"], rep)[0].tolist() == m["uniform_replace%d_coo_row" % rep]
        assert ops._CAPI_sample_neighbors_with_probs(sd2, ip2, ix2, pr2, m["k"], rep)[0].tolist() == \
            m["weighted_replace%d_coo_row" % rep]

    c = ref["cache"]
    cpu = torch.from_numpy(_bits(c["cpu_bits"]).copy()).pin_memory()
    gpu = torch.from_numpy(_bits(c["gpu_bits"]).copy()).cuda()
    hk, hv = ops._CAPI_create_hash_map(dev(c["hot"]), torch.arange(len(c["hot"]), device="cuda"))
    assert hk.numel() == c["table_slots"]
    out = ops._CAPI_fetch_data(cpu, gpu, dev(c["nid"]), hk, hv)
    assert out.cpu().numpy().view(np.int32).tolist() == c["fetched_bits"]
