"""Host-side logic of the multi-rank path on CPU: two gloo ranks agree on the
placement, see complementary location classes, and shard the seed batches."""
import os
import subprocess
import sys
import textwrap

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

WORKER = textwrap.dedent('''
    import ctypes, importlib, os, sys
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, %r)
    from oracle import oracle as o
    pkg = importlib.import_module("dist-gpu-sampling_b200")
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    abi = pkg.load_abi()

    # root decides the capacity (create_chunktensor's rule) and broadcasts it
    table_bytes = 6000 * 100 * 4
    meta = [[6000, 100], "float32", pkg.cached_size_per_gpu(table_bytes, world, 10 ** 6, 0.7)] if rank == 0 else [None] * 3
    dist.broadcast_object_list(meta, 0)
    e, t, h = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    assert abi.dgs_placement(6000 * 100, 4, meta[2], world, ctypes.byref(e), ctypes.byref(t), ctypes.byref(h)) == 0
    mine = (e.value, t.value, h.value)
    assert mine == o.placement(6000 * 100, 4, meta[2], world)
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    assert all(x == mine for x in everyone), everyone

    # every id is local on exactly one rank or host on all of them
    idx = np.random.default_rng(0).integers(0, 6000, size=5000)
    lo, re, ho = o.split_index(idx, 100, mine[0], mine[1], rank)
    parts = [None] * world
    dist.all_gather_object(parts, (lo.tolist(), ho.tolist()))
    local_sets = [set(p[0]) for p in parts]
    assert all(p[1] == parts[0][1] for p in parts)
    for a in range(world):
        for b in range(a + 1, world):
            assert not (local_sets[a] & local_sets[b])
    assert set().union(*local_sets) | set(parts[0][1]) == set(idx.tolist())

    # seed batches: disjoint across ranks, same train set everywhere
    batches = synth.train_batches(50000, 8192, 256)
    mine_b = [b for b in range(batches.shape[0]) if b %% world == rank]
    allb = [None] * world
    dist.all_gather_object(allb, mine_b)
    flat = sorted(sum(allb, []))
    assert flat == list(range(batches.shape[0]))
    # free memory differs per rank: the group plans with the minimum, and every rank derives the same plan
    avail = pkg.reduce_min_over_ranks(10 ** 9 + rank * 12345)
    assert avail == 10 ** 9
    graph = {"indptr": (8 * 10 ** 6, 8, 1.0), "indices": (8 * 10 ** 8, 8, 0.8), "features": (4 * 10 ** 9, 400, 0.5)}
    plan = pkg.plan_capacities(graph, world, avail)
    plans = [None] * world
    dist.all_gather_object(plans, plan)
    assert all(p == plan for p in plans)
    assert plan["features"] == 10 ** 9 // 400 * 400 and plan["indices"] == 0 and plan["indptr"] == 0
    print("GLOO RANK %%d OK" %% rank, flush=True)
    dist.destroy_process_group()
''')


def test_two_gloo_ranks_agree(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29431", str(script)]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-3000:]
    assert "GLOO RANK 0 OK" in r.stdout and "GLOO RANK 1 OK" in r.stdout
