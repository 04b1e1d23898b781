"""The CPU oracle against the reference's golden vector, the frozen fixtures,
and independent numpy restatements.  No GPU."""
import json
import os

import numpy as np
import pytest
from scipy import stats

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_readme_demo_vector(oracle):
    """The reference's only golden vector (README.md:48-63): ChunkTensor([100],
    int64, 200) on one rank, loaded with arange(100)."""
    g = json.load(open(os.path.join(GOLDEN, "readme_demo.json")))
    cm = oracle.ChunkModel(g["shape"], np.int64, g["capacity_per_gpu"], world=g["world"])
    assert (cm.each, cm.thr, cm.host_n) == (25, 25, 75)
    cm.load(np.arange(100, dtype=np.int64))
    assert cm.sub_device_tensor(0).tolist() == g["device_tensor"]
    assert cm.host_tensor().tolist() == g["host_tensor"]
    assert cm.index(np.array([0, 24, 25, 99])).reshape(-1).tolist() == [0, 24, 25, 99]


def test_frozen_fixtures(oracle):
    g = json.load(open(os.path.join(GOLDEN, "oracle_small.json")))
    for c in g["placement"]:
        assert list(oracle.placement(*c["in"])) == c["out"]
    ix = g["index"]
    table = np.array(ix["table"], dtype=np.int32)
    cm = oracle.ChunkModel(table.shape, np.int32, ix["capacity_per_gpu"], world=ix["world"])
    cm.load(table)
    assert (cm.each, cm.thr) == (ix["each"], ix["threshold"])
    assert cm.index(np.array(ix["idx"])).tolist() == ix["out"]
    for r in range(ix["world"]):
        assert [x.tolist() for x in cm.split_index(np.array(ix["idx"]), r)] == ix["split"][r]
    rl = g["relabel"]
    u, (ra, rb) = oracle.tensor_relabel([np.array(m) for m in rl["mapping"]], [np.array(m) for m in rl["mapping"]])
    assert u.tolist() == rl["unique"] and [ra.tolist(), rb.tolist()] == rl["relabelled"]
    assert oracle.relabel(u, np.array(rl["query"])).tolist() == rl["query_out"]
    fr = g["full_rows"]
    row, col = oracle.sample_uniform(np.array(fr["indptr"]), np.array(fr["indices"]), np.array(fr["seeds"]), fr["k"], False)
    assert row.tolist() == fr["coo_row"] and col.tolist() == fr["coo_col"]


@pytest.mark.parametrize("total,esz,cap,world", [(100, 8, 200, 1), (100, 8, 200, 4), (5, 4, 1 << 20, 4),
                                                 (1000, 4, 0, 2), (12800, 4, 6404, 8), (0, 4, 64, 2)])
def test_placement_rules(oracle, total, esz, cap, world):
    """src/chunk_tensor.cc:53-73 restated independently in Python."""
    each = cap // esz
    thr = each * world
    if thr > total:
        thr, each = total, -(-total // world)
    assert oracle.placement(total, esz, cap, world) == (each, thr, total - thr)


@pytest.mark.parametrize("world,cap_elems,D", [(1, 10 ** 9, 8), (4, 37, 8), (3, 50, 6), (8, 16, 16), (2, 0, 4)])
def test_index_equals_flat_index_select(oracle, world, cap_elems, D):
    """At()-based gather through chunks + host tail == fancy indexing of the flat tensor,
    including rows that straddle chunk boundaries (capacity not a multiple of D)."""
    rng = np.random.default_rng(5)
    rows = 123
    table = rng.standard_normal((rows, D)).astype(np.float32)
    cm = oracle.ChunkModel(table.shape, np.float32, cap_elems * 4, world=world)
    cm.load(table)
    idx = rng.integers(0, rows, size=500)
    out = cm.index(idx)
    assert out.tobytes() == table[idx].tobytes()
    assert oracle.index_flat(table, idx).tobytes() == table[idx].tobytes()
    # 1-D tensors give [n, 1]
    v = rng.integers(0, 1 << 40, size=77).astype(np.int64)
    cm1 = oracle.ChunkModel([77], np.int64, 8 * 10, world=world)
    cm1.load(v)
    assert cm1.index(np.arange(77)).shape == (77, 1)
    assert cm1.index(np.arange(77)).reshape(-1).tolist() == v.tolist()


def test_split_index_predicates(oracle):
    """src/cuda/index_with_chunk_tensor.cu:68-76 with its integer divisions."""
    rng = np.random.default_rng(9)
    D, each, world = 6, 50, 3
    thr = each * world
    idx = rng.integers(0, 40, size=300)
    for rank in range(world):
        lo, re, ho = oracle.split_index(idx, D, each, thr, rank)
        host = idx >= thr // D
        local = (~host) & (idx >= rank * each // D) & (idx < (rank + 1) * each // D)
        assert lo.tolist() == idx[local].tolist()
        assert ho.tolist() == idx[host].tolist()
        assert re.tolist() == idx[~host & ~local].tolist()


def test_relabel_first_occurrence(oracle):
    rng = np.random.default_rng(3)
    seeds = rng.permutation(1000)[:100]
    col = rng.integers(0, 1000, size=5000)
    cat = np.concatenate([seeds, col])
    u, (r, c) = oracle.tensor_relabel([seeds, col], [np.repeat(seeds, 50), col])
    _, first = np.unique(cat, return_index=True)
    assert u.tolist() == cat[np.sort(first)].tolist()
    assert u[:100].tolist() == seeds.tolist()          # seeds keep ids 0..n-1
    assert np.array_equal(u[c], col) and np.array_equal(u[r], np.repeat(seeds, 50))
    assert oracle.relabel(u, np.array([10 ** 9, -5])).tolist() == [-1, -1]
    assert oracle.unique(np.empty(0, np.int64)).size == 0


def _small_graph(rng, n=200, max_deg=40):
    deg = rng.integers(0, max_deg, size=n)
    deg[:5] = [0, 1, 10, 11, 9]
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, size=int(indptr[-1])).astype(np.int64)
    return indptr, indices


@pytest.mark.parametrize("replace", [False, True])
def test_oracle_uniform_validity(oracle, replace):
    rng = np.random.default_rng(11)
    indptr, indices = _small_graph(rng)
    seeds = rng.integers(0, 200, size=500)
    seeds[:5] = [0, 1, 2, 3, 4]
    row, col, pos, _ = oracle.sample_uniform(indptr, indices, seeds, 10, replace, rng_seed=7, want_pos=True)
    oracle.check_sample(indptr, indices, seeds, 10, replace, row, col, pos)


def test_oracle_uniform_distribution(oracle):
    """Reservoir restatement: each position of a deg-30 row is kept with probability k/deg."""
    deg, k, trials = 30, 7, 20000
    indptr = np.array([0, deg], dtype=np.int64)
    indices = np.arange(deg, dtype=np.int64)
    seeds = np.zeros(trials, dtype=np.int64)
    _, col = oracle.sample_uniform(indptr, indices, seeds, k, False, rng_seed=123)
    counts = np.bincount(col, minlength=deg)
    assert counts.sum() == trials * k
    chi2 = ((counts - trials * k / deg) ** 2 / (trials * k / deg * (1 - k / deg))).sum()
    # inclusion counts are negatively correlated; the scaled statistic is ~chi2(deg-1)
    assert stats.chi2.sf(chi2, deg - 1) > 0.001


@pytest.mark.parametrize("replace", [False, True])
def test_oracle_weighted(oracle, replace):
    rng = np.random.default_rng(13)
    indptr, indices = _small_graph(rng)
    probs = rng.random(indices.size).astype(np.float32) + 0.01
    seeds = rng.integers(0, 200, size=300)
    row, col, pos, _ = oracle.sample_weighted(indptr, indices, probs, seeds, 8, replace, rng_seed=5, want_pos=True)
    oracle.check_sample(indptr, indices, seeds, 8, replace, row, col, pos)
    if replace:  # draws proportional to the weights
        deg, trials = 12, 30000
        w = np.arange(1, deg + 1, dtype=np.float32)
        _, c = oracle.sample_weighted(np.array([0, deg]), np.arange(deg), w, np.zeros(trials, np.int64), 1, True, rng_seed=9)
        counts = np.bincount(c, minlength=deg)
        assert stats.chisquare(counts, trials * w / w.sum()).pvalue > 0.001


def test_oracle_sample_blocks_pipeline(oracle, synth):
    indptr, indices = synth.uniform_graph_csc(2000, 40000, seed=1)
    seeds = synth.distinct_seeds(2000, 64, seed=2)
    frontier, blocks, edges = oracle.sample_blocks(indptr, indices, seeds, [10, 10])
    assert frontier[:64].tolist() == seeds.tolist()
    assert edges == sum(b[0].size for b in blocks) and len(blocks) == 2
    r, c, n_src, n_dst = blocks[-1]       # innermost hop: dst = the seeds
    assert n_dst == 64 and r.max() < 64 and c.max() < n_src


def test_cache_fetch_oracle(oracle):
    rng = np.random.default_rng(17)
    cpu = rng.standard_normal((50, 4)).astype(np.float32)
    keys = rng.permutation(50)[:20]
    gpu = cpu[keys] + 100.0
    nid = rng.integers(0, 50, size=64)
    out = oracle.cache_fetch(cpu, gpu, keys, np.arange(20), nid)
    pos = {int(k): i for i, k in enumerate(keys)}
    exp = np.stack([gpu[pos[int(x)]] if int(x) in pos else cpu[int(x)] for x in nid])
    assert out.tobytes() == exp.tobytes()


def test_oracle_reproduces_the_frozen_multi_hop_loop(oracle):
    """The sample -> relabel loop over fan-outs [6, 5, 7] on a graph whose degrees are all below 5:
    nothing is random, so frontier and blocks are one fixed answer."""
    g = json.load(open(os.path.join(GOLDEN, "oracle_small.json")))["blocks"]
    f, blocks, n_edges = oracle.sample_blocks(np.array(g["indptr"]), np.array(g["indices"]), np.array(g["seeds"]),
                                              g["fanouts"])
    assert n_edges == g["n_edges"] and f.tolist() == g["frontier"]
    for (r, c, ns, nd), e in zip(blocks, g["blocks"]):
        assert r.tolist() == e["coo_row"] and c.tolist() == e["coo_col"] and (ns, nd) == (e["n_src"], e["n_dst"])
