"""Row-wise sampling on the GPU: deterministic rows bit-exact against the
oracle, stochastic rows checked for validity and distribution."""
import itertools
import json
import os

import numpy as np
import pytest
import torch
from scipy import stats

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def words():
    from gpu_util import Words
    return Words()


def small_graph(rng, n=300, max_deg=70):
    deg = rng.integers(0, max_deg, size=n)
    deg[:8] = [0, 1, 10, 11, 9, 20, 19, 300]        # empty, full, deg = k, k + 1, hub
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, size=int(indptr[-1])).astype(np.int64)
    return indptr, indices


def to_dev(a, dt=torch.int64):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dt).cuda()


@pytest.mark.parametrize("k", [1, 3, 5, 10, 15, 16, 25, 32, 40, 100])
@pytest.mark.parametrize("replace", [False, True])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_uniform_validity(oracle, words, k, replace, idt):
    from gpu_util import plain_desc, sample
    rng = np.random.default_rng(100 + k)
    indptr, indices = small_graph(rng)
    seeds = rng.integers(0, 300, size=1000)
    seeds[:8] = np.arange(8)
    ip, ix, sd = to_dev(indptr, idt), to_dev(indices, idt), to_dev(seeds, idt)
    row, col, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, replace, words, rng=(k, 5))
    assert words.take_status() == 0
    oracle.check_sample(indptr, indices, seeds, k, replace, row.astype(np.int64), col.astype(np.int64), pos)
    # same arguments -> same sample; a different offset -> a different one
    row2, col2, pos2 = sample(plain_desc(ip), plain_desc(ix), sd, k, replace, words, rng=(k, 5))
    assert np.array_equal(pos, pos2)
    _, _, pos3 = sample(plain_desc(ip), plain_desc(ix), sd, k, replace, words, rng=(k, 6))
    if k < 100:
        assert not np.array_equal(pos, pos3)


def test_full_rows_golden(words):
    """deg <= k everywhere: the output is the frozen oracle output, bit for bit."""
    from gpu_util import plain_desc, sample
    fr = json.load(open(os.path.join(GOLDEN, "oracle_small.json")))["full_rows"]
    ip, ix, sd = (to_dev(np.array(fr[x])) for x in ("indptr", "indices", "seeds"))
    row, col, _ = sample(plain_desc(ip), plain_desc(ix), sd, fr["k"], False, words)
    assert row.tolist() == fr["coo_row"] and col.tolist() == fr["coo_col"]


def test_uniform_chunked_and_bad_seed(oracle, words):
    """indptr / indices spread over 4 emulated chunks + host tail; rows straddle chunk boundaries."""
    from gpu_util import EmulatedChunks, sample
    rng = np.random.default_rng(21)
    indptr, indices = small_graph(rng)
    ip = EmulatedChunks(indptr, 1, 8 * 61, 4)
    ix = EmulatedChunks(indices, 1, 8 * 1777, 4)
    assert ix.host_n > 0 and ip.host_n > 0
    seeds = rng.integers(0, 300, size=2000)
    for k, replace in [(10, False), (15, False), (4, True)]:
        row, col, pos = sample(ip.desc, ix.desc, to_dev(seeds), k, replace, words)
        assert words.take_status() == 0
        oracle.check_sample(indptr, indices, seeds, k, replace, row, col, pos)
    bad = seeds.copy()
    bad[7] = 300          # not a node
    bad[9] = -2
    row, col, pos = sample(ip.desc, ix.desc, to_dev(bad), 5, False, words)
    assert words.take_status() == 6      # reported, not a fault; the bad seeds contribute nothing
    good = np.delete(bad, [7, 9])
    out_ptr, nnz = oracle.sample_counts(indptr, good, 5, False)
    assert row.size == nnz


def _chi2_inclusion(pos, deg, k, trials):
    counts = np.bincount(pos, minlength=deg)
    assert counts.sum() == trials * k
    p = k / deg
    # per-position inclusion is Bernoulli(p); positions are negatively correlated, so
    # sum((c - np)^2 / (np(1-p))) * (deg-1)/deg ~ chi2(deg-1)
    stat = ((counts - trials * p) ** 2 / (trials * p * (1 - p))).sum() * (deg - 1) / deg
    return stats.chi2.sf(stat, deg - 1)


@pytest.mark.parametrize("deg,k", [(30, 7), (9, 7), (16, 15), (1000, 10), (33, 32), (200, 40)])
def test_uniform_inclusion_is_uniform(words, deg, k):
    """10^6 draws: every position of a row is included with probability k/deg
    (covers direct rejection, the complement mode and the k > 32 path)."""
    from gpu_util import plain_desc, sample
    trials = max(1, 1_000_000 // k)
    ip = to_dev(np.array([0, deg]))
    ix = to_dev(np.arange(deg))
    sd = torch.zeros(trials, dtype=torch.int64, device="cuda")
    _, col, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, False, words, rng=(42, deg))
    assert np.array_equal(col, pos)
    per_row = np.sort(pos.reshape(trials, k), axis=1)
    assert (np.diff(per_row, axis=1) > 0).all()                  # distinct within every row
    assert _chi2_inclusion(pos, deg, k, trials) > 0.01


@pytest.mark.parametrize("deg,k", [(5, 2), (6, 3), (7, 5)])
def test_uniform_subsets_are_equally_likely(words, deg, k):
    """Stronger than inclusion frequencies: all C(deg,k) subsets are equally likely."""
    from gpu_util import plain_desc, sample
    trials = 400_000
    ip, ix = to_dev(np.array([0, deg])), to_dev(np.arange(deg))
    sd = torch.zeros(trials, dtype=torch.int64, device="cuda")
    _, _, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, False, words, rng=(7, deg * 10 + k))
    code = (1 << pos.reshape(trials, k)).sum(axis=1)
    subsets = [sum(1 << i for i in c) for c in itertools.combinations(range(deg), k)]
    counts = np.array([(code == s).sum() for s in subsets])
    assert counts.sum() == trials
    assert stats.chisquare(counts).pvalue > 0.01


def test_uniform_replace_is_uniform(words):
    from gpu_util import plain_desc, sample
    deg, k, trials = 37, 4, 250_000
    ip, ix = to_dev(np.array([0, deg])), to_dev(np.arange(deg))
    sd = torch.zeros(trials, dtype=torch.int64, device="cuda")
    _, _, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, True, words, rng=(3, 3))
    assert stats.chisquare(np.bincount(pos, minlength=deg)).pvalue > 0.01


# ---------------------------------------------------------------------------
# weighted
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("k", [1, 8, 32])
@pytest.mark.parametrize("replace", [False, True])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_weighted_validity(oracle, words, k, replace, idt):
    from gpu_util import plain_desc, sample, EmulatedChunks
    rng = np.random.default_rng(200 + k)
    indptr, indices = small_graph(rng)
    probs = rng.random(indices.size).astype(np.float32)
    probs[rng.random(indices.size) < 0.1] = 0.0
    seeds = rng.integers(0, 300, size=700)
    seeds[:8] = np.arange(8)
    ip, ix, sd = to_dev(indptr, idt), to_dev(indices, idt), to_dev(seeds, idt)
    pr = torch.from_numpy(probs).cuda()
    row, col, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, replace, words, probs_desc=plain_desc(pr))
    assert words.take_status() == 0
    oracle.check_sample(indptr, indices, seeds, k, replace, row.astype(np.int64), col.astype(np.int64), pos)
    if replace:   # zero-weight edges are never drawn while the row has positive weight
        st = np.repeat(indptr[seeds], np.diff(oracle.sample_counts(indptr, seeds, k, True)[0]))
        rowsum = np.add.reduceat(np.append(probs, 0), indptr[:-1])[row] if row.size else np.array([])
        drawn_w = probs[st + pos]
        assert (drawn_w[rowsum > 0] > 0).all()
    # weights in a chunked tensor with a host tail give the same sample (same RNG stream)
    if idt == torch.int64:
        pc = EmulatedChunks(probs, 1, 4 * 999, 3)
        _, _, pos_c = sample(plain_desc(ip), plain_desc(ix), sd, k, replace, words, probs_desc=pc.desc)
        assert np.array_equal(pos, pos_c)


def test_weighted_replace_is_proportional(words):
    from gpu_util import plain_desc, sample
    deg, k, trials = 45, 5, 200_000
    w = (np.arange(deg) % 7 + 1).astype(np.float32)
    w[3] = 0.0
    ip, ix = to_dev(np.array([0, deg])), to_dev(np.arange(deg))
    sd = torch.zeros(trials, dtype=torch.int64, device="cuda")
    pr = torch.from_numpy(w).cuda()          # must outlive the call: the descriptor only holds its address
    _, _, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, True, words, probs_desc=plain_desc(pr))
    counts = np.bincount(pos, minlength=deg)
    assert counts[3] == 0
    keep = w > 0
    assert stats.chisquare(counts[keep], counts.sum() * w[keep] / w.sum()).pvalue > 0.01


def _successive_inclusion(w, k):
    """Exact inclusion probabilities of weighted sampling without replacement
    (successive draws proportional to the remaining weights), which is the
    distribution A-Res realises."""
    n = len(w)
    inc = np.zeros(n)
    for perm in itertools.permutations(range(n), k):
        p, rest = 1.0, w.sum()
        for i in perm:
            p *= w[i] / rest
            rest -= w[i]
        inc[list(perm)] += p
    return inc


@pytest.mark.parametrize("deg,k", [(6, 2), (8, 3), (5, 4)])
def test_weighted_without_replacement_matches_ares(words, deg, k):
    from gpu_util import plain_desc, sample
    trials = 300_000
    w = np.linspace(0.2, 2.0, deg).astype(np.float32)
    ip, ix = to_dev(np.array([0, deg])), to_dev(np.arange(deg))
    sd = torch.zeros(trials, dtype=torch.int64, device="cuda")
    pr = torch.from_numpy(w).cuda()
    _, _, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, False, words, probs_desc=plain_desc(pr))
    per_row = np.sort(pos.reshape(trials, k), axis=1)
    assert (np.diff(per_row, axis=1) > 0).all()
    counts = np.bincount(pos, minlength=deg)
    inc = _successive_inclusion(w.astype(np.float64), k)
    # inclusion counts of one position are Binomial(trials, inc_i): z-test per position (Bonferroni)
    z = (counts - trials * inc) / np.sqrt(trials * inc * (1 - inc))
    assert np.abs(z).max() < stats.norm.isf(0.01 / (2 * deg))


@pytest.mark.parametrize("deg,k", [(1500, 1), (3000, 8), (700, 32), (9000, 5)])
def test_weighted_long_rows(words, deg, k):
    """Rows longer than one 512-edge window (and above 4096 edges: scanned by a whole CTA).
    With equal weights every position must be
    included with probability k/deg wherever it lies in the row; with k = 1 the pick must be
    exactly proportional to the weights."""
    from gpu_util import plain_desc, sample
    trials = 300_000 // max(1, k // 4)
    ip, ix = to_dev(np.array([0, deg])), to_dev(np.arange(deg))
    sd = torch.zeros(trials, dtype=torch.int64, device="cuda")
    rng = np.random.default_rng(deg)
    if k == 1:
        w = (rng.random(deg) + 0.05).astype(np.float32)
        w[rng.random(deg) < 0.2] = 0.0
    else:
        w = np.full(deg, 0.37, dtype=np.float32)
    pr = torch.from_numpy(w).cuda()
    _, _, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, False, words, probs_desc=plain_desc(pr), rng=(11, deg))
    assert words.take_status() == 0
    per_row = np.sort(pos.reshape(trials, k), axis=1)
    assert (np.diff(per_row, axis=1) > 0).all() if k > 1 else True
    nb = 50
    edges = np.linspace(0, deg, nb + 1).astype(int)
    counts = np.histogram(pos, bins=edges)[0]
    expect = np.add.reduceat(w.astype(np.float64), edges[:-1])
    expect = expect / expect.sum() * counts.sum()
    if k == 1:
        assert (w[pos] > 0).all()
        assert stats.chisquare(counts, expect).pvalue > 0.01
    else:
        # inclusion counts of buckets are slightly negatively correlated: the statistic is conservative
        assert stats.chisquare(counts, expect).pvalue > 0.01


def test_weighted_hub_rows(oracle, words):
    """Rows longer than 4096 edges are scanned by a whole CTA: same contract (valid, distinct
    positions) and picks proportional to the weights."""
    from gpu_util import plain_desc, sample
    deg, k, trials = 10_000, 4, 20_000
    w = np.ones(deg, dtype=np.float32)
    heavy = np.arange(deg) % 10 == 3
    w[heavy] = 5.0
    indptr = np.array([0, 3, 3 + deg, 3 + deg + 5000])          # a short row, the hub, a second hub
    indices = np.arange(indptr[-1]) % 977
    probs = np.concatenate([np.ones(3, np.float32), w, np.ones(5000, np.float32)])
    ip, ix = to_dev(indptr), to_dev(indices)
    pr = torch.from_numpy(probs).cuda()
    seeds = np.ones(trials, dtype=np.int64)
    seeds[::7] = 0
    seeds[3::11] = 2
    row, col, pos = sample(plain_desc(ip), plain_desc(ix), to_dev(seeds), k, False, words, probs_desc=plain_desc(pr))
    assert words.take_status() == 0
    oracle.check_sample(indptr, indices, seeds, k, False, row, col, pos)
    hub = pos[row == 1]
    n_draws = hub.size
    share = heavy[hub].mean()
    # with k << deg, without-replacement picks are proportional to the weights to first order
    expect = 5.0 * heavy.sum() / (5.0 * heavy.sum() + (~heavy).sum())
    assert abs(share - expect) < 4 * np.sqrt(expect * (1 - expect) / n_draws) + 2e-3
    counts = np.bincount(hub // 1000, minlength=10)              # every part of the row is reached
    assert stats.chisquare(counts).pvalue > 0.001


def test_weighted_zero_weights_fill_only_leftovers(words):
    from gpu_util import plain_desc, sample
    deg, k = 40, 6
    w = np.zeros(deg, dtype=np.float32)
    w[[2, 11, 30]] = [1.0, 1e-30, 5.0]           # 3 positive weights, one tiny
    ip, ix = to_dev(np.array([0, deg])), to_dev(np.arange(deg))
    sd = torch.zeros(1000, dtype=torch.int64, device="cuda")
    pr = torch.from_numpy(w).cuda()
    _, _, pos = sample(plain_desc(ip), plain_desc(ix), sd, k, False, words, probs_desc=plain_desc(pr))
    per_row = pos.reshape(1000, k)
    for p in (2, 11, 30):
        assert (per_row == p).any(axis=1).all()   # every positive-weight edge is always kept


def test_sampling_ops_through_torch(ops, oracle):
    """The reference-facing operators (plain tensors and ChunkTensors)."""
    rng = np.random.default_rng(31)
    indptr, indices = small_graph(rng)
    probs = (rng.random(indices.size) + 0.05).astype(np.float32)
    seeds = rng.permutation(300)[:200]
    ip, ix, sd, pr = to_dev(indptr), to_dev(indices), to_dev(seeds), torch.from_numpy(probs).cuda()
    c_ip = torch.classes.dgs_classes.ChunkTensor([indptr.size], torch.int64, 8 * 100)
    c_ix = torch.classes.dgs_classes.ChunkTensor([indices.size], torch.int64, 8 * 3000)
    c_pr = torch.classes.dgs_classes.ChunkTensor([indices.size], torch.float32, 4 * 5000)
    c_ip._CAPI_load_from_tensor(torch.from_numpy(indptr))
    c_ix._CAPI_load_from_tensor(torch.from_numpy(indices))
    c_pr._CAPI_load_from_tensor(torch.from_numpy(probs))
    nbr = [np.sort(indices[indptr[v]:indptr[v + 1]]) for v in range(300)]

    def check(row, col, k, replace):
        row, col = row.cpu().numpy(), col.cpu().numpy()
        out_ptr, nnz = oracle.sample_counts(indptr, seeds, k, replace)
        assert row.size == nnz and col.size == nnz
        assert np.array_equal(row, np.repeat(seeds, np.diff(out_ptr)))
        for i, s in enumerate(seeds):
            got = np.sort(col[out_ptr[i]:out_ptr[i + 1]])
            deg = indptr[s + 1] - indptr[s]
            if not replace and deg <= k:
                assert np.array_equal(col[out_ptr[i]:out_ptr[i + 1]], indices[indptr[s]:indptr[s + 1]])
            if not replace:   # multiset inclusion
                u, c = np.unique(got, return_counts=True)
                un, cn = np.unique(nbr[s], return_counts=True)
                assert np.isin(u, un).all() and (c <= cn[np.searchsorted(un, u)]).all()
            else:
                assert np.isin(got, nbr[s]).all()

    torch.manual_seed(5)
    for k, replace in [(10, False), (3, True)]:
        check(*ops._CAPI_sample_neighbors(sd, ip, ix, k, replace), k, replace)
        check(*ops._CAPI_sample_neighbors_with_chunk_tensor(sd, c_ip, c_ix, k, replace), k, replace)
        check(*ops._CAPI_sample_neighbors_with_probs(sd, ip, ix, pr, k, replace), k, replace)
        check(*ops._CAPI_sample_neighbors_with_probs_with_chunk_tensor(sd, c_ip, c_ix, c_pr, k, replace), k, replace)
    # torch.manual_seed controls the sample
    torch.manual_seed(77)
    a = ops._CAPI_sample_neighbors(sd, ip, ix, 10, False)[1]
    b = ops._CAPI_sample_neighbors(sd, ip, ix, 10, False)[1]
    torch.manual_seed(77)
    c = ops._CAPI_sample_neighbors(sd, ip, ix, 10, False)[1]
    assert torch.equal(a, c) and not torch.equal(a, b)
    # empty seeds, k = 0
    e = ops._CAPI_sample_neighbors(sd[:0], ip, ix, 10, False)
    assert e[0].numel() == 0 and e[1].numel() == 0
    z = ops._CAPI_sample_neighbors(sd, ip, ix, 0, False)
    assert z[0].numel() == 0
    with pytest.raises(RuntimeError, match="32"):
        ops._CAPI_sample_neighbors_with_probs(sd, ip, ix, pr, 33, False)
    with pytest.raises(RuntimeError, match="id type"):
        ops._CAPI_sample_neighbors(sd.int(), ip, ix, 5, False)
