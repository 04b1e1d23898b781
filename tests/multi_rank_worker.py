"""Worker run under torchrun by test_gpu_multi.py: one process per GPU.

Every rank builds the same seeded data, so each can check what it reads from
its own chunk, from peer chunks (cudaIpc mappings over NVLink) and from the
shared host tail against the CPU oracle.  Prints "RANK r OK" on success.
"""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import oracle as o  # noqa: E402
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_gpu_blocks import check_hops  # noqa: E402


def main():
    pkg = importlib.import_module("dist-gpu-sampling_b200")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    pkg.load_ops()
    pkg.create_dgs_communicator(world)
    ops = torch.ops.dgs_ops
    rng = np.random.default_rng(5)          # same stream on every rank

    # ---- a mismatching constructor call fails on every rank, nobody hangs ----
    try:
        torch.classes.dgs_classes.ChunkTensor([100, 4], torch.float32, 160 + 16 * rank)
        raise SystemExit("rank %d: mismatching metadata was accepted" % rank)
    except RuntimeError as e:
        assert "differs" in str(e) or "rejected" in str(e), str(e)

    # ---- a rank that cannot pin the host tail fails the constructor on EVERY rank (all-host tensor: no
    # device chunk, so no handle exchange carries the failure); injected on the host, nothing faults ----
    os.environ["DGS_TEST_REFUSE_HOST_REGISTER"] = str(world - 1)
    try:
        torch.classes.dgs_classes.ChunkTensor([4096], torch.int64, 0)
        raise SystemExit("rank %d: a tensor whose host tail one rank could not pin was accepted" % rank)
    except RuntimeError as e:
        assert "failed on rank %d" % (world - 1) in str(e) or "cudaHostRegister" in str(e), str(e)
    del os.environ["DGS_TEST_REFUSE_HOST_REGISTER"]
    ok = torch.classes.dgs_classes.ChunkTensor([4096], torch.int64, 0)        # and the group is still in step
    assert ok._CAPI_get_host_tensor().numel() == 4096
    del ok

    # ---- feature table: chunks on every GPU + host tail, rows straddle boundaries ----
    rows, D = 6000, 100
    table = rng.standard_normal((rows, D)).astype(np.float32)
    cap = 4 * (D * (rows // (world + 1)) + 36)            # not row aligned; ~1/(world+1) of the rows on the host
    ct = pkg.create_chunktensor(torch.from_numpy(table), world, cap, cache_rate=1.0, whole_rows=False)
    cm = o.ChunkModel([rows, D], np.float32, min(cap, table.nbytes // world), world=world)
    cm.load(table)
    assert cm.host_n > 0
    sub = ct._CAPI_get_sub_device_tensor().cpu().numpy()
    assert sub.tobytes() == cm.sub_device_tensor(rank).tobytes(), "local chunk differs"
    assert ct._CAPI_get_host_tensor().numpy().tobytes() == cm.host_tensor().tobytes(), "host tail differs"
    idx = np.concatenate([rng.integers(0, rows, size=20000), np.arange(rows)])
    idx_t = torch.from_numpy(idx).to(dev)
    out = ct._CAPI_index(idx_t)
    assert out.cpu().numpy().tobytes() == table[idx].tobytes(), "index differs from index_select"
    lo, re, ho = ct._CAPI_split_index(idx_t)
    elo, ere, eho = cm.split_index(idx, rank)
    assert lo.tolist() == elo.tolist() and re.tolist() == ere.tolist() and ho.tolist() == eho.tolist()
    assert re.numel() > 0
    for part, fn in ((lo, ct._CAPI_local_index), (re, ct._CAPI_remote_index), (ho, ct._CAPI_host_index)):
        assert fn(part).cpu().numpy().tobytes() == table[part.cpu().numpy()].tobytes()
    del fn, part                                   # bound methods keep the ChunkTensor alive

    # ---- graph in ChunkTensors over all ranks: sample + relabel per rank ----
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    indptr, indices = synth.uniform_graph_csc(20000, 300000, seed=1)
    probs = np.random.default_rng(6).random(indices.size).astype(np.float32) + 0.01
    big = 1 << 40
    c_ip = pkg.create_chunktensor(torch.from_numpy(indptr), world, big)
    c_ix = pkg.create_chunktensor(torch.from_numpy(indices), world, big, cache_rate=0.8)
    c_pr = pkg.create_chunktensor(torch.from_numpy(probs), world, big, cache_rate=0.8)
    seeds = np.random.default_rng(100 + rank).permutation(20000)[:2048]      # each rank its own batch
    sd = torch.from_numpy(seeds).to(dev)
    edge_keys = np.repeat(np.arange(20000), np.diff(indptr)) * 20000 + indices
    torch.manual_seed(rank)
    for weighted in (False, True):
        cur, cur_np = sd, seeds
        for k in (10, 5):
            if weighted:
                row, col = ops._CAPI_sample_neighbors_with_probs_with_chunk_tensor(cur, c_ip, c_ix, c_pr, k, False)
            else:
                row, col = ops._CAPI_sample_neighbors_with_chunk_tensor(cur, c_ip, c_ix, k, False)
            r_np, c_np = row.cpu().numpy(), col.cpu().numpy()
            out_ptr, nnz = o.sample_counts(indptr, cur_np, k, False)
            assert r_np.size == nnz and np.array_equal(r_np, np.repeat(cur_np, np.diff(out_ptr)))
            assert np.isin(r_np * 20000 + c_np, edge_keys).all(), "sampled a non-edge"
            frontier, (rr, cc) = ops._CAPI_tensor_relabel([cur, col], [row, col])
            eu, (er, ec) = o.tensor_relabel([cur_np, c_np], [r_np, c_np])
            assert frontier.tolist() == eu.tolist() and rr.tolist() == er.tolist() and cc.tolist() == ec.tolist()
            cur, cur_np = frontier, eu
    # ---- the whole hop loop as ONE queued sequence over the same multi-rank ChunkTensors, and with several
    # batches in flight (the path the benchmark times at N > 1) ----
    for weighted in (False, True):
        pr = c_pr if weighted else None
        f, blocks, ne = pkg.sample_blocks(sd, [10, 5], c_ip, c_ix, probs=pr, fused=True)
        assert ne == check_hops(o, indptr, indices, seeds, [10, 5], False, f, blocks), "fused blocks invalid"
    # no random choice: a graph whose degrees are all below the fan-outs -> bit for bit the oracle's loop
    rng2 = np.random.default_rng(9)
    deg = rng2.integers(0, 6, size=6000)
    ip2 = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    ix2 = rng2.integers(0, 6000, size=int(ip2[-1])).astype(np.int64)
    pr2 = (rng2.random(ix2.size) + 0.01).astype(np.float32)
    ft2 = rng2.standard_normal((6000, 100)).astype(np.float32)
    c_ip2 = pkg.create_chunktensor(torch.from_numpy(ip2), world, big)
    c_ix2 = pkg.create_chunktensor(torch.from_numpy(ix2), world, big, cache_rate=0.8)
    c_pr2 = pkg.create_chunktensor(torch.from_numpy(pr2), world, big, cache_rate=0.8)
    c_ft2 = pkg.create_chunktensor(torch.from_numpy(ft2), world, big, cache_rate=0.8)
    fan2 = [6, 7, 5]
    batches = [np.random.default_rng(200 + 10 * rank + b).permutation(6000)[:n] for b, n in enumerate((300, 300, 41, 300))]
    for weighted in (False, True):
        pr = c_pr2 if weighted else None
        for b in batches:
            of, ob, oe = o.sample_blocks(ip2, ix2, b, fan2)
            f, blocks, ne = pkg.sample_blocks(torch.from_numpy(b).to(dev), fan2, c_ip2, c_ix2, probs=pr, fused=True)
            assert ne == oe and f.tolist() == of.tolist(), "fused blocks differ from the oracle"
            for (r, c, ns, nd), (orow, ocol, ons, ond) in zip(blocks, ob):
                assert (ns, nd) == (ons, ond) and r.tolist() == orow.tolist() and c.tolist() == ocol.tolist()
        sampler = pkg.PipelinedSampler(c_ip2, c_ix2, fan2, features=c_ft2, probs=pr, max_seeds=300, depth=3)
        for (f, blocks, ne, x), b in zip(sampler(torch.from_numpy(b).to(dev) for b in batches), batches):
            of, ob, oe = o.sample_blocks(ip2, ix2, b, fan2)
            assert ne == oe and f.tolist() == of.tolist(), "pipelined blocks differ from the oracle"
            for (r, c, ns, nd), (orow, ocol, ons, ond) in zip(blocks, ob):
                assert (ns, nd) == (ons, ond) and r.tolist() == orow.tolist() and c.tolist() == ocol.tolist()
            assert x.cpu().numpy().tobytes() == ft2[of].tobytes(), "pipelined features differ"
        del sampler
    # stochastic batches in flight over the big graph
    sampler = pkg.PipelinedSampler(c_ip, c_ix, [10, 5], max_seeds=2048, depth=2)
    many = [np.random.default_rng(300 + 10 * rank + b).permutation(20000)[:2048] for b in range(3)]
    for (f, blocks, ne, x), b in zip(sampler(torch.from_numpy(b).to(dev) for b in many), many):
        assert ne == check_hops(o, indptr, indices, b, [10, 5], False, f, blocks), "pipelined blocks invalid"
    del sampler
    assert torch.ops.dgs_ops._CAPI_get_current_allocated() > 0
    torch.cuda.synchronize()
    dist.barrier()
    del pr                                 # (a second name for one of the ChunkTensors)
    del c_ip2, c_ix2, c_pr2, c_ft2
    del ct, c_ip, c_ix, c_pr, sub          # collective teardown, same order everywhere
    assert torch.ops.dgs_ops._CAPI_get_current_allocated() == 0
    dist.barrier()
    print("RANK %d OK" % rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
