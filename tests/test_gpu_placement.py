"""Placement helpers on the GPU: the free-memory rule, and a graph renumbered by degree still samples the
same edges (compared where nothing is random: fan-outs above every degree)."""
import numpy as np
import pytest
import torch

from test_gpu_blocks import to_dev

pytestmark = pytest.mark.gpu


def test_get_available_memory_follows_the_reference_rule(ops, pkg):
    total = torch.cuda.mem_get_info(0)[1]
    held = ops._CAPI_get_current_allocated()
    got = pkg.get_available_memory(0, 3 << 30)
    want = total - (3 << 30) - held - 0.3 * torch.cuda.max_memory_reserved()
    assert abs(got - max(int(want), 0)) <= 1
    assert pkg.get_available_memory(0, total * 2) == 0           # never negative
    ct = torch.classes.dgs_classes.ChunkTensor([1 << 20], torch.int64, 8 << 20)      # 8 MiB held by a ChunkTensor
    assert pkg.get_available_memory(0, 3 << 30) <= got - (8 << 20) + 1
    del ct


@pytest.mark.parametrize("by", ["in", "out"])
def test_renumbered_graph_samples_the_same_edges(ops, oracle, pkg, by):
    rng = np.random.default_rng(31)
    deg = rng.integers(0, 9, size=3000)
    deg[:2] = [30, 25]
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, 3000, size=int(indptr[-1])).astype(np.int64)
    ni, nx, old_of_new, src = pkg.renumber_by_degree(to_dev(indptr), to_dev(indices), by=by)
    new_of_old = torch.empty_like(old_of_new)
    new_of_old[old_of_new] = torch.arange(3000, device="cuda")
    seeds_old = to_dev(rng.permutation(3000)[:500])
    fan = [31, 32]                                             # above every degree: whole rows, nothing random
    f_old, b_old, e_old = pkg.sample_blocks(seeds_old, fan, to_dev(indptr), to_dev(indices), fused=True)
    f_new, b_new, e_new = pkg.sample_blocks(new_of_old[seeds_old], fan, ni, nx, fused=True)
    assert e_old == e_new
    # same frontier and, hop by hop, the same edges once the new ids are mapped back
    assert torch.equal(old_of_new[f_new], f_old)
    for (r0, c0, ns0, nd0), (r1, c1, ns1, nd1) in zip(b_old, b_new):
        assert (ns0, nd0) == (ns1, nd1) and torch.equal(r0, r1) and torch.equal(c0, c1)
    # hot rows first: degrees never increase along the new numbering
    key = (ni[1:] - ni[:-1]) if by == "in" else torch.bincount(nx, minlength=3000)
    assert bool((key[1:] <= key[:-1]).all())
