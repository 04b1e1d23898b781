"""Unique / relabel and the cache operators against the oracle (bit-exact)."""
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


def dev(a, dt=torch.int64):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dt).cuda()


def test_relabel_golden(words):
    from gpu_util import unique_relabel
    rl = json.load(open(os.path.join(GOLDEN, "oracle_small.json")))["relabel"]
    maps = [dev(np.array(m)) for m in rl["mapping"]]
    u, out = unique_relabel(maps, maps + [dev(np.array(rl["query"]))], words)
    assert u.tolist() == rl["unique"]
    assert out.tolist() == rl["relabelled"][0] + rl["relabelled"][1] + rl["query_out"]


@pytest.mark.parametrize("n_seed,n_col,universe", [(1, 0, 10), (100, 5000, 300), (1024, 10240, 100000),
                                                   (5000, 300000, 2000), (3, 70000, 5)])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_unique_relabel_matches_oracle(oracle, words, n_seed, n_col, universe, idt):
    from gpu_util import unique_relabel
    rng = np.random.default_rng(n_col + n_seed)
    seeds = rng.permutation(max(universe, n_seed))[:n_seed]
    col = rng.integers(0, universe, size=n_col)
    rowrep = seeds[rng.integers(0, n_seed, size=n_col)]
    u, out = unique_relabel([dev(seeds, idt), dev(col, idt)], [dev(rowrep, idt), dev(col, idt)], words)
    assert words.take_status() == 0
    eu, (er, ec) = oracle.tensor_relabel([seeds, col], [rowrep, col])
    assert u.tolist() == eu.tolist()
    assert out[:n_col].tolist() == er.tolist() and out[n_col:].tolist() == ec.tolist()


def test_relabel_large_properties(words):
    """2M keys: labels invert the unique list and the list is in first-occurrence order."""
    from gpu_util import unique_relabel
    g = torch.Generator(device="cuda").manual_seed(3)
    keys = torch.randint(0, 1 << 40, (2_000_000,), device="cuda", generator=g)
    keys[1_000_000:] = keys[:1_000_000]            # every key at least twice
    u, out = unique_relabel([keys], [keys], words)
    assert words.take_status() == 0
    k = keys.cpu().numpy()
    assert np.array_equal(u[out], k)
    _, first = np.unique(k, return_index=True)
    assert np.array_equal(u, k[np.sort(first)])


def test_relabel_absent_and_negative(words):
    from gpu_util import unique_relabel
    u, out = unique_relabel([dev([5, 3, 5])], [dev([3, 9, 5, -4])], words)
    assert u.tolist() == [5, 3] and out.tolist() == [1, -1, 0, -1]
    assert words.take_status() == 0
    u, out = unique_relabel([dev([5, -1, 3])], [dev([3])], words)     # negative keys are skipped and reported
    assert u.tolist() == [5, 3] and out.tolist() == [1] and words.take_status() == 6


def test_tensor_relabel_op(ops, oracle):
    rng = np.random.default_rng(2)
    seeds = rng.permutation(5000)[:512]
    col = rng.integers(0, 5000, size=512 * 10)
    row = np.repeat(seeds, 10)
    f, (r, c) = ops._CAPI_tensor_relabel([dev(seeds), dev(col)], [dev(row), dev(col)])
    eu, (er, ec) = oracle.tensor_relabel([seeds, col], [row, col])
    assert f.tolist() == eu.tolist() and r.tolist() == er.tolist() and c.tolist() == ec.tolist()
    assert f[:512].tolist() == seeds.tolist()
    # more tensors than the segment list holds, int32 ids, empty tensors
    many = [dev(rng.integers(0, 50, size=7), torch.int32) for _ in range(11)] + [dev([], torch.int32)]
    f, outs = ops._CAPI_tensor_relabel(many, many)
    eu, eouts = oracle.tensor_relabel([m.cpu().numpy() for m in many], [m.cpu().numpy() for m in many])
    assert f.dtype == torch.int32 and f.tolist() == eu.tolist()
    assert [o.tolist() for o in outs] == [o.tolist() for o in eouts]
    f, outs = ops._CAPI_tensor_relabel([dev([])], [dev([])])
    assert f.numel() == 0 and outs[0].numel() == 0


def test_sample_blocks_small_config(ops, oracle, synth, pkg):
    """The small parity configuration end to end: 100k nodes / 2M uniform-random
    edges, 1024 seeds, fan-out [10, 10], relabel per hop, 64-wide fp32 features."""
    indptr, indices = synth.uniform_graph_csc(100_000, 2_000_000, seed=1)
    seeds = synth.distinct_seeds(100_000, 1024, seed=2)
    feats = np.random.default_rng(3).standard_normal((100_000, 64)).astype(np.float32)
    ip, ix = dev(indptr), dev(indices)
    c_feat = torch.classes.dgs_classes.ChunkTensor([100_000, 64], torch.float32, feats.nbytes)
    c_feat._CAPI_load_from_tensor(torch.from_numpy(feats))
    torch.manual_seed(0)
    cur = dev(seeds)
    total = 0
    for hop in range(2):
        s_np = cur.cpu().numpy()
        row, col = ops._CAPI_sample_neighbors(cur, ip, ix, 10, False)
        r_np, c_np = row.cpu().numpy(), col.cpu().numpy()
        out_ptr, nnz = oracle.sample_counts(indptr, s_np, 10, False)
        assert r_np.size == nnz
        cnt = np.diff(out_ptr)
        assert np.array_equal(r_np, np.repeat(s_np, cnt))
        # full rows bit-exact; sampled rows: every (seed, col) is an edge of the graph
        full = np.repeat((indptr[s_np + 1] - indptr[s_np]) <= 10, cnt)
        within = np.arange(nnz) - np.repeat(out_ptr[:-1], cnt)
        assert np.array_equal(c_np[full], indices[np.repeat(indptr[s_np], cnt)[full] + within[full]])
        edge_keys = np.sort(np.repeat(np.arange(100_000), np.diff(indptr)) * 100_000 + indices)
        got = r_np * 100_000 + c_np
        assert np.isin(got, edge_keys).all()
        frontier, (rr, cc) = ops._CAPI_tensor_relabel([cur, col], [row, col])
        eu, (er, ec) = oracle.tensor_relabel([s_np, c_np], [r_np, c_np])
        assert frontier.tolist() == eu.tolist() and rr.tolist() == er.tolist() and cc.tolist() == ec.tolist()
        total += nnz
        cur = frontier
    x = c_feat._CAPI_index(cur)
    assert x.cpu().numpy().tobytes() == feats[cur.cpu().numpy()].tobytes()
    # the packaged loop gives the same frontier sizes for the same seed
    torch.manual_seed(0)
    fr2, blocks, n_edges = pkg.sample_blocks(dev(seeds), [10, 10], ip, ix)
    assert n_edges == total and torch.equal(fr2, cur) and len(blocks) == 2


def test_cache_ops(ops, oracle):
    rng = np.random.default_rng(23)
    n, D = 4000, 100
    cpu = rng.standard_normal((n, D)).astype(np.float32)
    hot = rng.permutation(n)[:900]
    gpu = cpu[hot] + 1000.0                              # cached copy differs, so hits are visible
    cpu_t = torch.from_numpy(cpu).pin_memory()
    for idt in (torch.int64, torch.int32):
        hk, hv = ops._CAPI_create_hash_map(dev(hot, idt), dev(np.arange(900), idt))
        assert hk.numel() == 2048 and hk.dtype == idt
        nid = rng.integers(0, n, size=30000)
        exp = oracle.cache_fetch(cpu, gpu, hot, np.arange(900), nid)
        out = ops._CAPI_fetch_data(cpu_t, torch.from_numpy(gpu).cuda(), dev(nid, idt), hk, hv)
        assert out.cpu().numpy().tobytes() == exp.tobytes()
        c_gpu = torch.classes.dgs_classes.ChunkTensor([900, D], torch.float32, 4 * D * 500 + 8)
        c_gpu._CAPI_load_from_tensor(torch.from_numpy(gpu))
        out = ops._CAPI_fetch_data_chunk_tensor(cpu_t, c_gpu, dev(nid, idt), hk, hv)
        assert out.cpu().numpy().tobytes() == exp.tobytes()
    with pytest.raises(RuntimeError, match="pinned"):
        ops._CAPI_fetch_data(torch.from_numpy(cpu), torch.from_numpy(gpu).cuda(), dev(nid), hk, hv)
