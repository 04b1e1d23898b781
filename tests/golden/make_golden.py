"""Writes tests/golden/*.json.

readme_demo.json restates the only golden vector the reference holds: the
expected output of example/demo.py printed in README.md:48-63
(ChunkTensor([100], int64, capacity_per_gpu=200) loaded with arange(100) on one
rank -> device part 0..24, host part 25..99).

oracle_small.json is produced by the pinned CPU oracle (oracle/dgs_oracle.c) on
seeded inputs; it freezes the oracle's deterministic outputs (placement, index,
split-index, relabel, full-row sampling, the multi-hop loop) so that a later change of the oracle
cannot silently move the target the CUDA path is compared against.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle as o  # noqa: E402


def main():
    with open(os.path.join(HERE, "readme_demo.json"), "w") as f:
        json.dump({"source": "README.md:48-63 / example/demo.py:24-36 of the reference",
                   "shape": [100], "dtype": "int64", "capacity_per_gpu": 200, "world": 1,
                   "loaded": "arange(100)",
                   "device_tensor": list(range(25)), "host_tensor": list(range(25, 100))}, f)

    rng = np.random.default_rng(20240607)
    cases = {}
    # placement: (total, esz, capacity, world) -> (each, threshold, host)
    pl = []
    for total, esz, cap, world in [(100, 8, 200, 1), (100, 8, 200, 4), (5, 4, 1 << 20, 4), (1000, 4, 0, 2),
                                   (12800, 4, 6400, 8), (12800, 4, 6404, 8), (7, 1, 3, 2),
                                   (111059956 * 128, 4, 111059956 * 128 * 4 // 8, 8)]:
        pl.append({"in": [total, esz, cap, world], "out": list(o.placement(total, esz, cap, world))})
    cases["placement"] = pl

    # index + split on a [37, 6] int32 table over 3 ranks with a non-row-aligned capacity
    table = rng.integers(-1000, 1000, size=(37, 6)).astype(np.int32)
    cm = o.ChunkModel(table.shape, np.int32, capacity_per_gpu=4 * 50, world=3)
    cm.load(table)
    idx = rng.integers(0, 37, size=64).astype(np.int64)
    cases["index"] = {"table": table.tolist(), "capacity_per_gpu": 200, "world": 3, "idx": idx.tolist(),
                      "each": cm.each, "threshold": cm.thr, "out": cm.index(idx).tolist(),
                      "split": [[x.tolist() for x in cm.split_index(idx, r)] for r in range(3)]}

    # relabel
    a = rng.integers(0, 40, size=30).astype(np.int64)
    b = rng.integers(0, 60, size=50).astype(np.int64)
    u, (ra, rb) = o.tensor_relabel([a, b], [a, b])
    q = rng.integers(0, 80, size=20).astype(np.int64)
    cases["relabel"] = {"mapping": [a.tolist(), b.tolist()], "unique": u.tolist(),
                        "relabelled": [ra.tolist(), rb.tolist()], "query": q.tolist(),
                        "query_out": o.relabel(u, q).tolist()}

    # full-row sampling: every row has deg <= k, so the output is deterministic
    deg = rng.integers(0, 6, size=20)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, 20, size=int(indptr[-1])).astype(np.int64)
    seeds = rng.permutation(20)[:12].astype(np.int64)
    row, col = o.sample_uniform(indptr, indices, seeds, 5, False)
    cases["full_rows"] = {"indptr": indptr.tolist(), "indices": indices.tolist(), "seeds": seeds.tolist(),
                          "k": 5, "coo_row": row.tolist(), "coo_col": col.tolist()}
    # the multi-hop loop (sample -> relabel per fan-out, last fan-out first) where nothing is random:
    # every degree is below every fan-out
    deg = rng.integers(0, 5, size=300)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, 300, size=int(indptr[-1])).astype(np.int64)
    seeds = rng.permutation(300)[:24].astype(np.int64)
    frontier, blocks, n_edges = o.sample_blocks(indptr, indices, seeds, [6, 5, 7])
    cases["blocks"] = {"indptr": indptr.tolist(), "indices": indices.tolist(), "seeds": seeds.tolist(),
                       "fanouts": [6, 5, 7], "frontier": frontier.tolist(), "n_edges": int(n_edges),
                       "blocks": [{"coo_row": r.tolist(), "coo_col": c.tolist(), "n_src": int(ns), "n_dst": int(nd)}
                                  for r, c, ns, nd in blocks]}
    with open(os.path.join(HERE, "oracle_small.json"), "w") as f:
        json.dump(cases, f)
    print("wrote golden fixtures")


if __name__ == "__main__":
    main()
