"""The hot path at the size the benchmark is quoted on (Products-shaped: 2,449,029 nodes, ~123.7 M edges, 100
features, 1,024 seeds, fan-outs [15, 10, 5]) -- too large for the CPU oracle to replay edge by edge in a test, so
the results are checked on the device through size-independent properties, for all three ways through the
library: per hop the edge count is sum(min(deg, k)), the rows are the seeds repeated by their counts, every
(row, col) is an edge of the graph, rows with deg <= k come out whole and in CSC order, the seeds lead the
frontier and the frontier has no repeats; every gathered feature row equals the generator's values; and the
three ways agree with each other on everything that is not a random choice (sizes of the first hop's block,
the leading part of the frontier)."""
import importlib
import os
import sys
import types

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_products_shaped_step_has_the_contract_properties(ops, pkg):
    sys.path.insert(0, ROOT)
    bench = importlib.import_module("bench")
    args = types.SimpleNamespace(workload="products", scale=0.0, batch=1024, weighted=False)
    env = bench.Env()
    env.world, env.rank, env.local_rank = 1, 0, 0
    env.dev = torch.device("cuda", 0)
    env.barrier = torch.cuda.synchronize
    env.clocks = None
    w = bench.workload("products", args)
    wl = bench.setup_workload(env, args, w, False)
    fan = w["fanouts"]
    batches = [wl.dev_batches[wl.my[i]] for i in range(3)]
    torch.manual_seed(5)
    sampler = pkg.PipelinedSampler(wl.c_indptr, wl.c_indices, fan, features=wl.c_feats, max_seeds=1024, depth=3)
    firsts = []
    for (fr, blocks, n_edges, x), seeds in zip(sampler(batches), batches):
        info = bench.verify_batch(env, pkg, wl, seeds, fr, blocks, x)
        assert info["edges_checked"] == n_edges and info["rows_checked"] == fr.numel() and info["hops"] == 3
        assert 600_000 < n_edges < 1_100_000 and 300_000 < fr.numel() < 600_000        # the benchmark's step
        firsts.append((blocks[-1][0].numel(), blocks[-1][3], fr[:1024].clone()))
    del sampler
    for fused in (True, False):                      # one batch at a time: _CAPI_sample_blocks*, then the per-hop operators
        for i, seeds in enumerate(batches):
            fr, blocks, n_edges = pkg.sample_blocks(seeds, fan, wl.c_indptr, wl.c_indices, fused=fused)
            x = wl.c_feats._CAPI_index(fr)
            bench.verify_batch(env, pkg, wl, seeds, fr, blocks, x)
            # not random: how many edges the first hop draws (sum of min(deg, 5) over the seeds), and that the
            # seeds open the frontier in their own order
            assert (blocks[-1][0].numel(), blocks[-1][3]) == firsts[i][:2]
            assert torch.equal(fr[:1024], firsts[i][2]) and torch.equal(fr[:1024], seeds)
    bench.teardown_workload(env, wl)
