"""Multi-hop sample + relabel queued as one sequence (_CAPI_sample_blocks*,
dgs_sample_blocks): every hop must satisfy the same contracts as the per-hop
operators -- counts, grouping by seed, whole rows in CSC order, picks out of the
seed's row without repeats, first-occurrence numbering -- and must be identical
to the oracle wherever no random choice is involved.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def to_dev(a, dt=torch.int64):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dt).cuda()


def graph(rng, n, max_deg, hubs=()):
    deg = rng.integers(0, max_deg, size=n)
    for i, d in enumerate(hubs):
        deg[i] = d
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, size=int(indptr[-1])).astype(np.int64)
    return indptr, indices


def check_hops(oracle, indptr, indices, seeds0, fanouts, replace, frontier, blocks):
    """blocks in layer order (outermost hop first); hop h of the application is blocks[H-1-h]."""
    final = frontier.cpu().numpy().astype(np.int64)
    assert np.unique(final).size == final.size, "frontier has repeats"
    H = len(fanouts)
    applied = list(reversed(fanouts))
    seeds = np.asarray(seeds0, dtype=np.int64)
    total = 0
    for h in range(H):
        row_l, col_l, n_src, n_dst = blocks[H - 1 - h]
        row_l, col_l = row_l.cpu().numpy().astype(np.int64), col_l.cpu().numpy().astype(np.int64)
        k = applied[h]
        assert n_dst == seeds.size
        fr = final[:n_src]
        out_ptr, nnz = oracle.sample_counts(indptr, seeds, k, replace)
        assert row_l.size == nnz and col_l.size == nnz, (h, row_l.size, nnz)
        total += nnz
        cnt = np.diff(out_ptr)
        row_g, col_g = fr[row_l], fr[col_l]
        assert np.array_equal(row_g, np.repeat(seeds, cnt)), "rows must be the seeds repeated by their counts"
        # relabel: first-occurrence unique of (seeds ++ cols), rows/cols are positions in it
        u, (r2, c2) = oracle.tensor_relabel([seeds, col_g], [row_g, col_g])
        assert np.array_equal(u, fr) and np.array_equal(r2, row_l) and np.array_equal(c2, col_l)
        # every pick is an edge of its seed; whole rows in CSC order; no position used twice
        for p in range(seeds.size):
            lo, hi = indptr[seeds[p]], indptr[seeds[p] + 1]
            got = col_g[out_ptr[p]:out_ptr[p + 1]]
            nb = indices[lo:hi]
            if not replace and hi - lo <= k:
                assert np.array_equal(got, nb), "whole row expected in CSC order"
            elif got.size:
                vals, c = np.unique(got, return_counts=True)
                nv, nc = np.unique(nb, return_counts=True)
                at = np.searchsorted(nv, vals)
                assert np.all(at < nv.size) and np.array_equal(nv[np.minimum(at, nv.size - 1)], vals), "pick is no edge"
                if not replace:
                    assert np.all(c <= nc[at]), "a neighbour position was used twice"
        seeds = fr
    return total


@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_blocks_without_random_choice_equal_the_oracle(ops, oracle, pkg, idt):
    rng = np.random.default_rng(5)
    indptr, indices = graph(rng, 4000, 6)                 # every degree <= 5 <= each fan-out
    seeds = rng.permutation(4000)[:300]
    fanouts = [7, 5, 6]
    of, ob, oe = oracle.sample_blocks(indptr, indices, seeds, fanouts)
    f, blocks, ne = pkg.sample_blocks(to_dev(seeds, idt), fanouts, to_dev(indptr, idt), to_dev(indices, idt),
                                      fused=True)
    assert ne == oe and f.dtype == idt and np.array_equal(f.cpu().numpy(), of)
    for (r, c, ns, nd), (orow, ocol, ons, ond) in zip(blocks, ob):
        assert (ns, nd) == (ons, ond)
        assert np.array_equal(r.cpu().numpy(), orow) and np.array_equal(c.cpu().numpy(), ocol)
    # and the per-hop operator sequence gives the same
    f2, blocks2, ne2 = pkg.sample_blocks(to_dev(seeds, idt), fanouts, to_dev(indptr, idt), to_dev(indices, idt))
    assert ne2 == ne and torch.equal(f2, f)
    for a, b in zip(blocks, blocks2):
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and a[2:] == b[2:]


@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
@pytest.mark.parametrize("fused", [True, False])
def test_blocks_match_the_frozen_fixture(ops, pkg, idt, fused):
    """tests/golden/oracle_small.json "blocks": the loop's one possible answer when no row is longer than a
    fan-out, through the one-sequence operators and through the per-hop operators."""
    import json
    import os
    g = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_small.json")))["blocks"]
    f, blocks, n_edges = pkg.sample_blocks(to_dev(np.array(g["seeds"]), idt), g["fanouts"],
                                           to_dev(np.array(g["indptr"]), idt), to_dev(np.array(g["indices"]), idt),
                                           fused=fused)
    assert n_edges == g["n_edges"] and f.dtype == idt and f.tolist() == g["frontier"]
    assert len(blocks) == len(g["blocks"])
    for (r, c, ns, nd), e in zip(blocks, g["blocks"]):
        assert r.tolist() == e["coo_row"] and c.tolist() == e["coo_col"] and (ns, nd) == (e["n_src"], e["n_dst"])


@pytest.mark.parametrize("fanouts,replace", [([15, 10, 5], False), ([10, 10], False), ([3, 4], True), ([40, 2], False)])
def test_blocks_uniform_valid(ops, oracle, pkg, fanouts, replace):
    rng = np.random.default_rng(11)
    indptr, indices = graph(rng, 20000, 40, hubs=(0, 1, 500, 3000))
    seeds = rng.permutation(20000)[:512]
    seeds[:4] = [0, 1, 2, 3]
    torch.manual_seed(3)
    f, blocks, ne = pkg.sample_blocks(to_dev(seeds), fanouts, to_dev(indptr), to_dev(indices), replace=replace,
                                      fused=True)
    assert ne == check_hops(oracle, indptr, indices, seeds, fanouts, replace, f, blocks)
    # another call draws other samples; the same torch seed reproduces the first
    f2, _, _ = pkg.sample_blocks(to_dev(seeds), fanouts, to_dev(indptr), to_dev(indices), replace=replace, fused=True)
    torch.manual_seed(3)
    f3, blocks3, _ = pkg.sample_blocks(to_dev(seeds), fanouts, to_dev(indptr), to_dev(indices), replace=replace,
                                       fused=True)
    assert torch.equal(f3, f) and all(torch.equal(a[1], b[1]) for a, b in zip(blocks, blocks3))
    assert f2.numel() != f.numel() or not torch.equal(f2, f)


def test_blocks_repeated_seeds_are_numbered_by_first_occurrence(ops, oracle, pkg):
    rng = np.random.default_rng(12)
    indptr, indices = graph(rng, 3000, 30)
    seeds = rng.integers(0, 3000, size=400)
    seeds[100:200] = seeds[:100]                          # repeats
    f, blocks, ne = pkg.sample_blocks(to_dev(seeds), [8, 4], to_dev(indptr), to_dev(indices), fused=True)
    assert ne == check_hops(oracle, indptr, indices, seeds, [8, 4], False, f, blocks)


@pytest.mark.parametrize("replace", [False, True])
def test_blocks_weighted_valid(ops, oracle, pkg, replace):
    rng = np.random.default_rng(13)
    indptr, indices = graph(rng, 8000, 60, hubs=(5000,))
    probs = (rng.random(indices.size) + 0.05).astype(np.float32)
    seeds = rng.permutation(8000)[:256]
    seeds[0] = 0
    f, blocks, ne = pkg.sample_blocks(to_dev(seeds), [10, 10], to_dev(indptr), to_dev(indices),
                                      probs=torch.from_numpy(probs).cuda(), replace=replace, fused=True)
    assert ne == check_hops(oracle, indptr, indices, seeds, [10, 10], replace, f, blocks)


def test_blocks_over_chunk_tensors_with_a_host_tail(ops, oracle, pkg):
    rng = np.random.default_rng(14)
    indptr, indices = graph(rng, 6000, 30)
    CT = torch.classes.dgs_classes.ChunkTensor
    c_ip = CT([indptr.size], torch.int64, 8 * 4001)       # both straddle device chunk and host tail
    c_ix = CT([indices.size], torch.int64, 8 * (indices.size // 2 + 3))
    c_ip._CAPI_load_from_tensor(torch.from_numpy(indptr))
    c_ix._CAPI_load_from_tensor(torch.from_numpy(indices))
    seeds = rng.permutation(6000)[:300]
    f, blocks, ne = pkg.sample_blocks(to_dev(seeds), [5, 6, 4], c_ip, c_ix, fused=True)
    assert ne == check_hops(oracle, indptr, indices, seeds, [5, 6, 4], False, f, blocks)


def test_blocks_edge_cases(ops, oracle, pkg):
    rng = np.random.default_rng(15)
    indptr, indices = graph(rng, 500, 12)
    ip, ix = to_dev(indptr), to_dev(indices)
    # no seeds
    f, blocks, ne = pkg.sample_blocks(torch.empty(0, dtype=torch.int64, device="cuda"), [3, 2], ip, ix, fused=True)
    assert f.numel() == 0 and ne == 0 and all(b[0].numel() == 0 and b[2:] == (0, 0) for b in blocks)
    # a zero fan-out: nothing sampled on that hop, the frontier is the seed list
    seeds = rng.permutation(500)[:50]
    f, blocks, ne = pkg.sample_blocks(to_dev(seeds), [0, 4], ip, ix, fused=True)
    assert ne == check_hops(oracle, indptr, indices, seeds, [0, 4], False, f, blocks)
    # seeds of isolated nodes only
    iso = np.flatnonzero(np.diff(indptr) == 0)[:5]
    if iso.size:
        f, blocks, ne = pkg.sample_blocks(to_dev(iso), [4, 4], ip, ix, fused=True)
        assert ne == 0 and f.cpu().tolist() == iso.tolist()
    # an id outside the graph is reported, not trapped
    bad = to_dev(np.array([1, 2, 500000, 3]))
    with pytest.raises(RuntimeError, match="out-of-range"):
        pkg.sample_blocks(bad, [3, 3], ip, ix, fused=True)
        torch.cuda.synchronize()
        ops._CAPI_tensor_relabel([bad[:2]], [bad[:2]])   # the next operator call notices at the latest
    torch.cuda.synchronize()
    # the library stays usable afterwards
    f, blocks, ne = pkg.sample_blocks(to_dev(seeds), [3], ip, ix, fused=True)
    assert ne == check_hops(oracle, indptr, indices, seeds, [3], False, f, blocks)


def test_blocks_through_the_c_abi(oracle, pkg):
    """dgs_sample_blocks called directly: bounds, workspace, one launch sequence, sizes in a pinned array."""
    from gpu_util import plain_desc, vp
    abi = pkg.load_abi()
    rng = np.random.default_rng(16)
    indptr, indices = graph(rng, 5000, 25)
    seeds = rng.permutation(5000)[:200]
    ip, ix, sd = to_dev(indptr), to_dev(indices), to_dev(seeds)
    fanouts = [5, 10]                                    # reference order; applied 10 then 5
    applied = (ctypes.c_int64 * 2)(10, 5)
    hops = (pkg.Hop * 2)()
    pkg.check(abi.dgs_sample_blocks_bounds(200, applied, 2, 5000, hops))
    assert hops[0].seed_bound == 200 and hops[0].frontier_bound == 2200
    assert hops[1].seed_bound == 2200 and hops[1].frontier_bound == 5000        # capped by the node count
    wsb = abi.dgs_sample_blocks_workspace_bytes(hops, 2)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    bufs = []
    for h in range(2):
        cap = hops[h].seed_bound * hops[h].fanout
        r, c = torch.full((cap,), -7, device="cuda"), torch.full((cap,), -7, device="cuda")
        fr = torch.full((hops[h].frontier_bound,), -7, device="cuda")
        hops[h].coo_row, hops[h].coo_col, hops[h].frontier = vp(r), vp(c), vp(fr)
        bufs.append((r, c, fr))
    sizes = torch.zeros(4, dtype=torch.int64).pin_memory()
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    pkg.check(abi.dgs_sample_blocks(ctypes.byref(plain_desc(ip)), ctypes.byref(plain_desc(ix)), None, vp(sd), 1,
                                    hops, 2, 0, 7, 0, vp(ws), wsb, vp(sizes), vp(status), None))
    torch.cuda.synchronize()
    assert status.item() == 0
    nnz0, nu0, nnz1, nu1 = sizes.tolist()
    blocks = [(bufs[1][0][:nnz1], bufs[1][1][:nnz1], nu1, nu0), (bufs[0][0][:nnz0], bufs[0][1][:nnz0], nu0, 200)]
    assert nnz0 + nnz1 == check_hops(oracle, indptr, indices, seeds, fanouts, False, bufs[1][2][:nu1], blocks)
    # nothing is written past the reported sizes
    assert bool((bufs[0][0][nnz0:] == -7).all()) and bool((bufs[1][2][nu1:] == -7).all())


@pytest.mark.parametrize("weighted", [False, True])
def test_blocks_over_emulated_multi_gpu_chunks(oracle, pkg, weighted):
    """dgs_sample_blocks through the C ABI over indptr / indices / weights split into four device parts plus a
    host tail, with chunk boundaries that fall at odd element offsets -- the layout of a multi-GPU run."""
    from gpu_util import EmulatedChunks, vp
    abi = pkg.load_abi()
    rng = np.random.default_rng(17)
    indptr, indices = graph(rng, 9000, 30, hubs=(0, 700))
    probs = (rng.random(indices.size) + 0.05).astype(np.float32)
    e_ip = EmulatedChunks(indptr, 1, 8 * 1801, 4, rank=2)                 # 4 x 1801 elements, rest on the host
    e_ix = EmulatedChunks(indices, 1, 8 * (indices.size // 5 + 3), 4, rank=1)
    e_pr = EmulatedChunks(probs, 1, 4 * (indices.size // 5 + 3), 4, rank=1)
    assert e_ip.host_n > 0 and e_ix.host_n > 0
    seeds = rng.permutation(9000)[:400]
    seeds[:2] = [0, 1]
    sd = to_dev(seeds)
    for fanouts in ([5, 10], [31, 32]):                                   # stochastic rows / (almost) whole rows
        H = len(fanouts)
        applied = (ctypes.c_int64 * H)(*reversed(fanouts))
        hops = (pkg.Hop * H)()
        pkg.check(abi.dgs_sample_blocks_bounds(seeds.size, applied, H, 9000, hops))
        wsb = abi.dgs_sample_blocks_workspace_bytes(hops, H)
        ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
        bufs = []
        for h in range(H):
            cap = hops[h].seed_bound * hops[h].fanout
            r, c = torch.full((cap,), -7, device="cuda"), torch.full((cap,), -7, device="cuda")
            fr = torch.full((hops[h].frontier_bound,), -7, device="cuda")
            hops[h].coo_row, hops[h].coo_col, hops[h].frontier = vp(r), vp(c), vp(fr)
            bufs.append((r, c, fr))
        sizes = torch.zeros(2 * H, dtype=torch.int64).pin_memory()
        status = torch.zeros(1, dtype=torch.int32).pin_memory()
        pkg.check(abi.dgs_sample_blocks(ctypes.byref(e_ip.desc), ctypes.byref(e_ix.desc),
                                        ctypes.byref(e_pr.desc) if weighted else None, vp(sd), 1, hops, H, 0, 11, 0,
                                        vp(ws), wsb, vp(sizes), vp(status), None))
        # the frontier length is also where dgs_sample_blocks_frontier_count says it is
        n_dev = abi.dgs_sample_blocks_frontier_count(hops, H, vp(ws))
        torch.cuda.synchronize()
        assert status.item() == 0
        sz = sizes.tolist()
        assert ws.data_ptr() <= n_dev < ws.data_ptr() + wsb
        word = ws[n_dev - ws.data_ptr(): n_dev - ws.data_ptr() + 8].view(torch.int64).item()
        assert word == sz[2 * H - 1]
        blocks, n_dst = [], seeds.size
        for h in range(H):
            blocks.insert(0, (bufs[h][0][:sz[2 * h]], bufs[h][1][:sz[2 * h]], sz[2 * h + 1], n_dst))
            n_dst = sz[2 * h + 1]
        total = check_hops(oracle, indptr, indices, seeds, fanouts, False, bufs[H - 1][2][:n_dst], blocks)
        assert total == sum(sz[0::2])


@pytest.mark.parametrize("weighted", [False, True])
def test_recorded_sequence_replays_bit_for_bit(oracle, pkg, weighted):
    """dgs_sample_blocks_record / _replay: a replay gives exactly what dgs_sample_blocks gives for the same
    (seed, offset), for every new pair written to the pinned words and every new seed list written to the
    seeds buffer, without recording again."""
    from gpu_util import plain_desc, vp
    abi = pkg.load_abi()
    rng = np.random.default_rng(23)
    indptr, indices = graph(rng, 6000, 40, hubs=(0, 900))
    probs = (rng.random(indices.size) + 0.05).astype(np.float32)
    ip, ix, pr = to_dev(indptr), to_dev(indices), torch.from_numpy(probs).cuda()
    d_ip, d_ix, d_pr = plain_desc(ip), plain_desc(ix), plain_desc(pr)
    fanouts, n_seeds, H = [5, 10, 15], 300, 3
    applied = (ctypes.c_int64 * H)(*reversed(fanouts))

    def buffers():
        hops = (pkg.Hop * H)()
        pkg.check(abi.dgs_sample_blocks_bounds(n_seeds, applied, H, 6000, hops))
        wsb = abi.dgs_sample_blocks_workspace_bytes(hops, H)
        ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
        bufs = []
        for h in range(H):
            cap = hops[h].seed_bound * hops[h].fanout
            r, c = torch.full((cap,), -7, device="cuda"), torch.full((cap,), -7, device="cuda")
            fr = torch.full((hops[h].frontier_bound,), -7, device="cuda")
            hops[h].coo_row, hops[h].coo_col, hops[h].frontier = vp(r), vp(c), vp(fr)
            bufs.append((r, c, fr))
        sizes = torch.zeros(2 * H, dtype=torch.int64).pin_memory()
        status = torch.zeros(1, dtype=torch.int32).pin_memory()
        return hops, wsb, ws, bufs, sizes, status

    def snapshot(bufs, sizes):
        sz = sizes.tolist()
        return sz, [(b[0][:sz[2 * h]].clone(), b[1][:sz[2 * h]].clone(), b[2][:sz[2 * h + 1]].clone())
                    for h, b in enumerate(bufs)]

    seeds_dev = torch.empty(n_seeds, dtype=torch.int64, device="cuda")
    rng_words = torch.zeros(2, dtype=torch.int64).pin_memory()
    hops_r, wsb, ws_r, bufs_r, sizes_r, status_r = buffers()
    hops_d, _, ws_d, bufs_d, sizes_d, status_d = buffers()
    stream = torch.cuda.Stream()
    rec = ctypes.c_void_p()
    pkg.check(abi.dgs_sample_blocks_record(ctypes.byref(d_ip), ctypes.byref(d_ix), ctypes.byref(d_pr) if weighted else None,
                                           vp(seeds_dev), 1, hops_r, H, 0, vp(rng_words), vp(ws_r), wsb, vp(sizes_r),
                                           vp(status_r), ctypes.c_void_p(stream.cuda_stream), ctypes.byref(rec)))
    assert rec.value
    torch.cuda.synchronize()
    assert bool((bufs_r[0][0] == -7).all())                      # recording ran nothing
    try:
        for trial, (seed, offset) in enumerate([(7, 0), (7, 4), (123456789, 1 << 40), (7, 0)]):
            seeds = rng.permutation(6000)[:n_seeds]
            seeds_dev.copy_(to_dev(seeds))
            rng_words[0], rng_words[1] = seed, offset
            torch.cuda.synchronize()
            pkg.check(abi.dgs_sample_blocks_replay(rec, ctypes.c_void_p(stream.cuda_stream)))
            pkg.check(abi.dgs_sample_blocks(ctypes.byref(d_ip), ctypes.byref(d_ix), ctypes.byref(d_pr) if weighted else None,
                                            vp(seeds_dev), 1, hops_d, H, 0, seed, offset, vp(ws_d), wsb, vp(sizes_d),
                                            vp(status_d), None))
            torch.cuda.synchronize()
            assert status_r.item() == 0 and status_d.item() == 0
            sz_r, out_r = snapshot(bufs_r, sizes_r)
            sz_d, out_d = snapshot(bufs_d, sizes_d)
            assert sz_r == sz_d and sz_r[0] > 0
            for (a, b, c), (x, y, z) in zip(out_r, out_d):
                assert torch.equal(a, x) and torch.equal(b, y) and torch.equal(c, z)
            if trial == 0:
                blocks, n_dst = [], n_seeds
                for h in range(H):
                    blocks.insert(0, (out_r[h][0], out_r[h][1], sz_r[2 * h + 1], n_dst))
                    n_dst = sz_r[2 * h + 1]
                assert sum(sz_r[0::2]) == check_hops(oracle, indptr, indices, seeds, fanouts, False, out_r[H - 1][2],
                                                     blocks)
    finally:
        abi.dgs_sample_blocks_recording_free(rec)
