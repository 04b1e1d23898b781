"""Placement policy on the CPU: capacity planning in the reference's priority order
(oppo_bench/single_node/README.md:93, chunktensor.py:57-102) and renumbering by degree."""
import numpy as np
import torch


def test_plan_capacities_serves_features_then_probs_then_indices_then_indptr(pkg):
    t = {"indptr": (800, 8, 1.0), "indices": (80_000, 8, 1.0), "probs": (40_000, 4, 1.0),
         "features": (400_000, 400, 0.5), "labels": (800, 8, 1.0)}
    # plenty of memory: everyone gets total * rate // gpus, cut to whole rows
    plan = pkg.plan_capacities(t, 2, 10 ** 9)
    assert plan == {"features": 100_000, "probs": 20_000, "indices": 40_000, "indptr": 400, "labels": 400}
    assert list(plan) == ["features", "probs", "indices", "indptr", "labels"]
    # short memory: features first, probs next, indices get (whole 16-byte units of) the rest,
    # indptr the crumbs, tensors outside the priority list nothing
    plan = pkg.plan_capacities(t, 2, 100_000 + 20_000 + 1_000)
    assert plan["features"] == 100_000 and plan["probs"] == 20_000 and plan["indices"] == 1_000 // 16 * 16
    assert plan["indptr"] == 8 and plan["labels"] == 0
    # not even the features fit: whole rows of them first, what is left trickles down the list
    plan = pkg.plan_capacities(t, 2, 1_000)
    assert plan == {"features": 800, "probs": 192, "indices": 8, "indptr": 0, "labels": 0}
    # the reference's byte-exact rule
    assert pkg.plan_capacities(t, 2, 1_000, whole_rows=False)["features"] == 1_000
    assert sum(pkg.plan_capacities(t, 2, 123_457).values()) <= 123_457


def _graph(rng, n, max_deg):
    deg = rng.integers(0, max_deg, size=n)
    deg[:3] = [max_deg * 3, 0, max_deg * 2]
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, size=int(indptr[-1])).astype(np.int64)
    return indptr, indices


def test_renumber_by_degree_is_a_relabelling_of_the_same_graph(pkg):
    rng = np.random.default_rng(3)
    indptr, indices = _graph(rng, 700, 20)
    probs = rng.random(indices.size).astype(np.float32)
    for by in ("in", "out"):
        for chunk in (1 << 27, 97):                         # one piece, and many small pieces
            ni, nx, old_of_new, src = pkg.renumber_by_degree(torch.from_numpy(indptr), torch.from_numpy(indices),
                                                             by=by, edge_chunk=chunk)
            ni, nx, old_of_new = ni.numpy(), nx.numpy(), old_of_new.numpy()
            assert sorted(old_of_new.tolist()) == list(range(700))
            key = np.diff(indptr) if by == "in" else np.bincount(indices, minlength=700)
            assert (np.diff(key[old_of_new]) <= 0).all()                      # hottest first
            ties = np.flatnonzero(np.diff(key[old_of_new]) == 0)
            assert (old_of_new[ties] < old_of_new[ties + 1]).all()            # stable
            assert ni[-1] == indices.size
            for i in (0, 1, 2, 350, 699):                                     # row i = old row old_of_new[i], renamed
                v = old_of_new[i]
                assert old_of_new[nx[ni[i]:ni[i + 1]]].tolist() == indices[indptr[v]:indptr[v + 1]].tolist()
            # the same multiset of (dst, src) edges in old ids
            new_dst = np.repeat(np.arange(700), np.diff(ni))
            a = np.sort(old_of_new[new_dst] * 700 + old_of_new[nx])
            b = np.sort(np.repeat(np.arange(700), np.diff(indptr)) * 700 + indices)
            assert np.array_equal(a, b)
            if src is not None:
                assert np.array_equal(indices[src.numpy()], old_of_new[nx])
                p2 = pkg.permute_edge_tensor(torch.from_numpy(probs), torch.from_numpy(indptr), torch.from_numpy(ni),
                                             torch.from_numpy(old_of_new), edge_chunk=chunk)
                assert np.array_equal(p2.numpy(), probs[src.numpy()])
