"""Several mini-batches in flight: torch.classes.dgs_classes.BlockPipeline (PipelinedSampler) and the
per-call pinned words of the operators.  Every batch must come out exactly as the one-at-a-time path
gives it -- bit for bit against the oracle wherever no random choice is involved, by the validity rules
of test_gpu_blocks.check_hops otherwise -- whatever else is running on other streams.
"""
import threading

import numpy as np
import pytest
import torch

from test_gpu_blocks import check_hops, graph, to_dev

pytestmark = pytest.mark.gpu


def chunked(a, frac=1.0):
    t = torch.from_numpy(np.ascontiguousarray(a))
    row = a.itemsize * (a.shape[1] if a.ndim == 2 else 1)
    cap = int(a.nbytes * frac) // row * row
    ct = torch.classes.dgs_classes.ChunkTensor(list(t.shape), t.dtype, cap)
    ct._CAPI_load_from_tensor(t)
    return ct


@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
@pytest.mark.parametrize("depth", [1, 3])
def test_pipeline_without_random_choice_equals_the_oracle(ops, oracle, pkg, idt, depth):
    rng = np.random.default_rng(21)
    indptr, indices = graph(rng, 5000, 6)                     # every degree <= 5 <= each fan-out
    feats = rng.standard_normal((5000, 25)).astype(np.float32)
    npdt = np.int64 if idt == torch.int64 else np.int32
    c_ip, c_ix = chunked(indptr.astype(npdt)), chunked(indices.astype(npdt), 0.6)     # host tail included
    c_ft = chunked(feats, 0.5)
    fanouts = [6, 7, 5]
    batches = [rng.permutation(5000)[:n] for n in (200, 200, 37, 200, 1, 200, 150)]
    sampler = pkg.PipelinedSampler(c_ip, c_ix, fanouts, features=c_ft, max_seeds=200, depth=depth)
    seen = 0
    for (f, blocks, ne, x), seeds in zip(sampler(to_dev(b, idt) for b in batches), batches):
        of, ob, oe = oracle.sample_blocks(indptr, indices, seeds, fanouts)
        assert ne == oe and f.dtype == idt and np.array_equal(f.cpu().numpy(), of)
        for (r, c, ns, nd), (orow, ocol, ons, ond) in zip(blocks, ob):
            assert (ns, nd) == (ons, ond)
            assert np.array_equal(r.cpu().numpy(), orow) and np.array_equal(c.cpu().numpy(), ocol)
        assert x.shape == (of.size, 25) and x.cpu().numpy().tobytes() == feats[of].tobytes()
        seen += 1
    assert seen == len(batches)
    del sampler


def test_pipeline_stochastic_batches_are_valid_and_results_outlive_later_submits(ops, oracle, pkg):
    rng = np.random.default_rng(22)
    indptr, indices = graph(rng, 20000, 40, hubs=(0, 1, 500, 3000))
    feats = rng.standard_normal((20000, 16)).astype(np.float32)
    c_ip, c_ix, c_ft = chunked(indptr), chunked(indices), chunked(feats)
    fanouts = [15, 10, 5]
    batches = [rng.permutation(20000)[:512] for _ in range(6)]
    batches[1][:4] = [0, 1, 2, 3]
    pinned = [torch.from_numpy(b).pin_memory() for b in batches]            # seeds straight from host memory
    depth = 3
    sampler = pkg.PipelinedSampler(c_ip, c_ix, fanouts, features=c_ft, max_seeds=512, depth=depth)
    torch.manual_seed(7)
    held = []
    # by hand: a batch handed out by next() stays intact, whatever the other slots are running, until the
    # submit() that takes its slot again (the depth-th after its own)
    for i in range(depth):
        sampler.submit(pinned[i])
    for i in range(len(batches)):
        f, blocks, ne, x = sampler.next()
        held.append((f, blocks, ne, x, f.clone(), x.clone()))
        assert ne == check_hops(oracle, indptr, indices, batches[i], fanouts, False, f, blocks)
        assert x.cpu().numpy().tobytes() == feats[f.cpu().numpy()].tobytes()
        torch.cuda.synchronize()                  # let the younger batches run to completion
        assert torch.equal(f, held[-1][4]) and torch.equal(x, held[-1][5])
        if i + depth < len(batches):
            sampler.submit(pinned[i + depth])     # from here on batch i's views belong to batch i + depth
    # same torch seed -> same batches again; another seed -> other samples
    torch.manual_seed(7)
    again = [(f.clone(), ne) for f, _, ne, _ in sampler(pinned)]
    assert all(torch.equal(a[0], h[4]) and a[1] == h[2] for a, h in zip(again, held))
    other = [f.clone() for f, _, _, _ in sampler(pinned)]
    assert any(o.numel() != h[4].numel() or not torch.equal(o, h[4]) for o, h in zip(other, held))
    del sampler


@pytest.mark.parametrize("weighted", [False, True])
def test_replayed_batches_equal_the_one_at_a_time_operator_bit_for_bit(ops, pkg, weighted):
    """From a slot's second batch of the same size on, the sampling sequence is a replayed recording; under
    the same torch seed it must give exactly what _CAPI_sample_blocks* gives launch by launch."""
    rng = np.random.default_rng(29)
    indptr, indices = graph(rng, 15000, 50, hubs=(0, 7, 900))
    probs = (rng.random(indices.size) + 0.05).astype(np.float32)
    c_ip, c_ix, c_pr = chunked(indptr), chunked(indices, 0.8), chunked(probs, 0.8)
    fanouts = [10, 10, 5]
    batches = [to_dev(rng.permutation(15000)[:n]) for n in (384, 384, 384, 384, 100, 100, 100, 384, 384)]
    sampler = pkg.PipelinedSampler(c_ip, c_ix, fanouts, probs=c_pr if weighted else None, max_seeds=384, depth=2)
    torch.manual_seed(31)
    piped = [(f.clone(), [(r.clone(), c.clone(), a, b) for r, c, a, b in blocks], ne)
             for f, blocks, ne, _ in sampler(batches)]
    assert sampler.pipe.recorded_slots() == 2
    torch.manual_seed(31)
    for (f, blocks, ne), seeds in zip(piped, batches):
        f2, blocks2, ne2 = pkg.sample_blocks(seeds, fanouts, c_ip, c_ix, probs=c_pr if weighted else None, fused=True)
        assert ne == ne2 and ne > 0 and torch.equal(f, f2)
        for (r, c, a, b), (r2, c2, a2, b2) in zip(blocks, blocks2):
            assert (a, b) == (a2, b2) and torch.equal(r, r2) and torch.equal(c, c2)
    del sampler


@pytest.mark.parametrize("weighted,replace", [(True, False), (True, True), (False, True)])
def test_pipeline_weighted_replace_and_without_features(ops, oracle, pkg, weighted, replace):
    rng = np.random.default_rng(23)
    indptr, indices = graph(rng, 8000, 60, hubs=(5000,))
    probs = (rng.random(indices.size) + 0.05).astype(np.float32)
    c_ip, c_ix, c_pr = chunked(indptr), chunked(indices, 0.7), chunked(probs, 0.7)
    batches = [rng.permutation(8000)[:256] for _ in range(4)]
    sampler = pkg.PipelinedSampler(c_ip, c_ix, [10, 10], probs=c_pr if weighted else None, replace=replace,
                                   max_seeds=256, depth=2)
    for (f, blocks, ne, x), seeds in zip(sampler(to_dev(b) for b in batches), batches):
        assert x.numel() == 0
        assert ne == check_hops(oracle, indptr, indices, seeds, [10, 10], replace, f, blocks)
    del sampler


def test_pipeline_edge_cases_and_errors(ops, oracle, pkg):
    rng = np.random.default_rng(24)
    indptr, indices = graph(rng, 500, 12)
    feats = rng.standard_normal((500, 8)).astype(np.float32)
    c_ip, c_ix, c_ft = chunked(indptr), chunked(indices), chunked(feats)
    sampler = pkg.PipelinedSampler(c_ip, c_ix, [3, 2], features=c_ft, max_seeds=64, depth=2)
    with pytest.raises(RuntimeError, match="nothing was submitted"):
        sampler.next()
    sampler.submit(torch.empty(0, dtype=torch.int64, device="cuda"))          # no seeds
    seeds = rng.permutation(500)[:50]
    sampler.submit(to_dev(seeds))
    with pytest.raises(RuntimeError, match="call next"):
        sampler.submit(to_dev(seeds))
    f, blocks, ne, x = sampler.next()
    assert f.numel() == 0 and ne == 0 and x.shape[0] == 0 and all(b[2:] == (0, 0) for b in blocks)
    f, blocks, ne, x = sampler.next()
    assert ne == check_hops(oracle, indptr, indices, seeds, [3, 2], False, f, blocks)
    with pytest.raises(RuntimeError, match="built for 64"):
        sampler.submit(torch.zeros(65, dtype=torch.int64, device="cuda"))
    with pytest.raises(RuntimeError, match="one id type"):
        sampler.submit(torch.zeros(4, dtype=torch.int32, device="cuda"))
    # an id outside the graph is reported for its batch, not trapped; the pipeline stays usable
    sampler.submit(to_dev(np.array([1, 2, 500000, 3])))
    sampler.submit(to_dev(seeds))
    with pytest.raises(RuntimeError, match="out-of-range"):
        sampler.next()
    f, blocks, ne, x = sampler.next()
    assert ne == check_hops(oracle, indptr, indices, seeds, [3, 2], False, f, blocks)
    with pytest.raises(RuntimeError, match="fan-outs must be >= 1"):
        pkg.PipelinedSampler(c_ip, c_ix, [3, 0], max_seeds=64)
    del sampler


def test_bipartite_graph_whose_column_ids_exceed_the_row_count(ops, oracle, pkg):
    """A CSC with 400 rows whose neighbour ids live in [0, 9000): one hop finds far more distinct ids than
    indptr has rows.  The one-sequence operator notices the outgrown frontier and gives the per-hop result;
    the pipeline needs the id space stated (src_nodes) and says so otherwise."""
    rng = np.random.default_rng(41)
    deg = rng.integers(5, 60, size=400)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, 9000, size=int(indptr[-1])).astype(np.int64)
    indices[:400] = np.arange(400)                         # some ids inside the row space as well
    seeds = rng.permutation(400)[:300]
    fanouts = [20]

    def check(f, blocks, ne):
        (r, c, n_src, n_dst), = blocks
        fr = f.cpu().numpy()
        assert n_dst == 300 and n_src == fr.size and fr.size > 400 and np.unique(fr).size == fr.size
        assert np.array_equal(fr[:300], seeds)
        cnt = np.minimum(deg[seeds], 20)
        assert ne == cnt.sum() and np.array_equal(fr[r.cpu().numpy()], np.repeat(seeds, cnt))
        cols = fr[c.cpu().numpy()]
        at = 0
        for s_, k_ in zip(seeds, cnt):
            row = indices[indptr[s_]:indptr[s_ + 1]]
            assert np.isin(cols[at:at + k_], row).all()
            at += k_
        assert fr.max() >= 400

    ip, ix, sd = to_dev(indptr), to_dev(indices), to_dev(seeds)
    f, blocks, ne = pkg.sample_blocks(sd, fanouts, ip, ix, fused=True)
    check(f, blocks, ne)
    # the next call is not blamed for the cut-off frontier of the first attempt
    f, blocks, ne = pkg.sample_blocks(sd, fanouts, ip, ix, fused=True)
    check(f, blocks, ne)

    c_ip, c_ix = chunked(indptr), chunked(indices)
    sampler = pkg.PipelinedSampler(c_ip, c_ix, fanouts, max_seeds=300, depth=2, src_nodes=9000)
    for f, blocks, ne, _ in sampler([sd, sd, sd]):
        check(f, blocks, ne)
    del sampler
    sampler = pkg.PipelinedSampler(c_ip, c_ix, fanouts, max_seeds=300, depth=2)
    sampler.submit(sd)
    with pytest.raises(RuntimeError, match="src_nodes"):
        sampler.next()
    sampler.submit(to_dev(np.arange(5)))                   # the pipeline stays usable
    f, blocks, ne, _ = sampler.next()
    assert ne == int(np.minimum(deg[:5], 20).sum())
    del sampler


def test_two_operator_calls_in_flight_on_two_streams(ops, oracle, pkg):
    """Two host threads, each on its own stream, call _CAPI_sample_blocks and the per-hop operators at the
    same time: each call leases its own pinned size / status words, so neither sees the other's sizes."""
    rng = np.random.default_rng(25)
    indptr, indices = graph(rng, 6000, 6)                      # no random choice with these fan-outs
    ip, ix = to_dev(indptr), to_dev(indices)
    fanouts = [6, 7, 5]
    jobs = [[rng.permutation(6000)[:n] for n in sizes] for sizes in ((300, 17, 250, 99) * 6, (41, 280, 5, 160) * 6)]
    want = [[oracle.sample_blocks(indptr, indices, s, fanouts) for s in js] for js in jobs]
    errors = []
    start = threading.Barrier(2)

    def worker(t):
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                sd = [to_dev(s) for s in jobs[t]]
                stream.synchronize()
                start.wait()
                for i, s in enumerate(sd):
                    f, blocks, ne = pkg.sample_blocks(s, fanouts, ip, ix, fused=(i % 2 == 0))
                    of, ob, oe = want[t][i]
                    assert ne == oe and np.array_equal(f.cpu().numpy(), of), (t, i)
                    for (r, c, ns, nd), (orow, ocol, ons, ond) in zip(blocks, ob):
                        assert (ns, nd) == (ons, ond)
                        assert np.array_equal(r.cpu().numpy(), orow) and np.array_equal(c.cpu().numpy(), ocol)
        except BaseException as e:      # noqa: BLE001 -- reported to the main thread
            errors.append(e)
            try:
                start.abort()
            except Exception:
                pass

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors


def test_deferred_status_names_the_operator_that_caused_it(ops, pkg):
    """_CAPI_index never waits for its kernel: a bad id gives a zero row, and the error surfaces at the
    next operator call on the device, naming _CAPI_index."""
    table = np.arange(40 * 8, dtype=np.float32).reshape(40, 8)
    ct = chunked(table)
    out = ct._CAPI_index(torch.tensor([3, 40, 39], device="cuda"))
    torch.cuda.synchronize()
    assert out[1].abs().sum().item() == 0 and out[2].cpu().numpy().tobytes() == table[39].tobytes()
    with pytest.raises(RuntimeError, match="earlier _CAPI_index call reported an out-of-range id"):
        ct._CAPI_index(torch.tensor([1], device="cuda"))
    out = ct._CAPI_index(torch.tensor([1], device="cuda"))          # reported once; the library stays usable
    assert out.cpu().numpy().tobytes() == table[1].tobytes()
