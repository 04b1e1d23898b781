"""Benchmark of the hot path: 3-hop neighbour sampling + relabel + feature gather.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--workload products|papers100m|friendster|small] [--batch 1024] [--weighted] [--scale F]
                  [--api blocks|per-hop]

One step = one mini-batch per rank:
  frontier, blocks = sample_blocks(seeds, [15, 10, 5])      # sample + relabel, fan-outs applied last to first
  x = features._CAPI_index(frontier)
The hop loop runs through `_CAPI_sample_blocks_with_chunk_tensor` (all hops queued as one
launch sequence, one size read-back per step; `--api blocks`, the default) or through the
reference's own operator sequence, `_CAPI_sample_neighbors_with_chunk_tensor` +
`_CAPI_tensor_relabel` per hop (`--api per-hop`).  Whichever is not the headline is timed
over the same K steps in the same run and reported as `other_api`.  The graph is
a Products-shaped synthetic graph (2,449,029 nodes, ~123.7 M edges, Chung-Lu
power law, 100 fp32 features per node) whose indptr / indices / features live in
ChunkTensors split evenly over the N GPUs of the node (weak scaling: every rank
samples its own 1,024-seed batches).  `--workload papers100m` is the
Papers100M-shaped configuration (111 M nodes, ~1.6 B edges, 128 features: 70 GB,
which fits one B200 or is split over N).  `--workload friendster` is the
Friendster-shaped hybrid configuration: fan-out [10, 10], 256 features, node ids
ranked by in-degree, 40 % of features and indices in the pinned host tail; it
runs at a quarter of the node count by default (`--scale 1` for the full 65.6 M
nodes / 3.6 B edges, which pins ~38 GB of host memory).  `--weighted` samples with
per-edge weights.

Printed JSON (rank 0, one line):
  value      sampled edges/s of the whole job, device-timed, seeds resident in HBM;
             the timed step is sample + relabel + gather
  e2e        same metric with the seeds coming from pinned host memory and a
             device->host read of the result inside the timed region
  roofline   the gather kernel: algorithmic bytes / CUDA-event time of back-to-back launches on the
             last frontiers vs measured HBM peak (the in-step figure is given beside it)
  cpu_baseline  the CPU oracle (port of the reference algorithm) on a bounded sample

`--impl reference` times that CPU port alone on all host threads (the reference
project has no CPU implementation of its own and its DGL baseline is not
installable here).
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # nodes, mean degree, power-law exponent, feature width, training-set size, fan-outs,
    # fraction of features/indices kept on the GPUs (the rest is the pinned host tail),
    # node ids ranked by in-degree (hot rows first -> they land in the GPU chunks)
    "products": dict(nodes=2_449_029, mean_deg=50.5, gamma=2.1, dim=100, train=196_615, fanouts=[15, 10, 5],
                     gpu_frac=1.0, degree_sorted=False),
    "papers100m": dict(nodes=111_059_956, mean_deg=14.5, gamma=2.3, dim=128, train=1_207_179,
                       fanouts=[15, 10, 5], gpu_frac=1.0, degree_sorted=False),
    "friendster": dict(nodes=65_608_366, mean_deg=55.0, gamma=2.2, dim=256, train=1_000_000, fanouts=[10, 10],
                       gpu_frac=0.6, degree_sorted=True),
    "small": dict(nodes=100_000, mean_deg=20.0, gamma=2.1, dim=64, train=20_000, fanouts=[15, 10, 5],
                  gpu_frac=1.0, degree_sorted=False),
}


def workload(args):
    """Workload parameters with --scale applied to the node count (edges follow: the mean degree is fixed)."""
    w = dict(WORKLOADS[args.workload])
    scale = args.scale if args.scale > 0 else (0.25 if args.workload == "friendster" else 1.0)
    w["scale"] = scale
    w["nodes"] = max(1000, int(w["nodes"] * scale))
    w["train"] = max(args.batch, min(w["train"], w["nodes"] // 2))
    return w
# kernels of this library launched per operator call (memsets are not kernels)
LAUNCHES_SAMPLE = 2   # plan (+ tile scan in its last CTA), sample
LAUNCHES_RELABEL = 4  # insert, count (+ tile scan in its last CTA), number, lookup
LAUNCHES_GATHER = 1
PRIME_STEPS = 32      # untimed steps during setup, before the warm-up steps, that populate the caching allocator
API_NAMES = {True: "_CAPI_sample_blocks* (all hops queued as one sequence, one size read-back per step)",
             False: "reference operator sequence: _CAPI_sample_neighbors* + _CAPI_tensor_relabel per hop"}
LAUNCHES_HOP_FUSED = 5  # plan (+ table clear + previous hop's lookup), sample, insert, count, number
LAUNCHES_STEP_FUSED = 2  # init words, last hop's lookup
# DRAM bytes per gathered row (read + write) from the ncu capture summarised in
# profiles/; None until a capture exists for the benchmarked row width
NCU_TRAFFIC_BYTES_PER_ROW = {100: 861.2}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="products", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--scale", type=float, default=0.0,
                    help="node-count factor; 0 = 1.0 (friendster: 0.25, so that the pinned tail stays ~10 GB)")
    ap.add_argument("--weighted", action="store_true",
                    help="sample with per-edge fp32 U(0,1) weights (the weighted operator) instead of uniformly")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--api", default="blocks", choices=["blocks", "per-hop"],
                    help="blocks: each step's hops go through _CAPI_sample_blocks* (one queued sequence, one size "
                         "read-back); per-hop: the reference's operator sequence, one sampling and one relabel "
                         "operator per hop.  The other one is timed too and reported beside the headline.")
    return ap.parse_args()


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self, lo=0, hi=None):
        """Summary of the samples [lo, hi) taken while the timed region ran
        (all samples if that window is empty because the region was too short)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        window = self.rows[lo:hi] if hi is not None and hi > lo else self.rows
        all_rows, self.rows = self.rows, window
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i] == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "samples_total": len(all_rows)}


def build_graph(w, device):
    """Same seeded graph on every rank (generated on `device`)."""
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    indptr, indices = synth.chung_lu_csc(w["nodes"], w["mean_deg"], w["gamma"], seed=11, device=device,
                                         degree_sorted=w["degree_sorted"])
    return indptr, indices


def edge_weights(start, count, device):
    """Per-edge sampling weight in (0, 1] as a function of the edge index."""
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    return synth.hashed_values(start, count, device=device, salt=17) * 0.5 + 0.5000001


def feature_values(start, count, device):
    """Feature table element values as a function of the flat element index, so
    every rank can fill its own chunk in place and nobody holds the table twice."""
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    return synth.hashed_values(start, count, device=device, salt=3)


def make_features(nodes, dim, device):
    import torch
    out = torch.empty(nodes * dim, dtype=torch.float32, device=device)
    step = 1 << 26
    for lo in range(0, out.numel(), step):
        n = min(step, out.numel() - lo)
        out[lo:lo + n] = feature_values(lo, n, device)
    return out.view(nodes, dim)


def config_dict(args, w, n_edges_graph, world):
    nodes, dim = w["nodes"], w["dim"]
    op = "sample_neighbors_with_probs_with_chunk_tensor" if args.weighted else "sample_neighbors_with_chunk_tensor"
    tail = "no host tail" if w["gpu_frac"] >= 1.0 else \
        "%.0f %% of features and indices in the pinned host tail, node ids ranked by in-degree" % (100 * (1 - w["gpu_frac"]))
    return {"workload": "%s-shaped synthetic%s: %d nodes, %d edges (Chung-Lu gamma=%.1f), CSC int64, "
                        "features [%d,%d] fp32" % (args.workload, "" if w["scale"] == 1.0 else " at scale %.2f" % w["scale"],
                                                   nodes, n_edges_graph, w["gamma"], nodes, dim),
            "fanouts": w["fanouts"], "batch_per_rank": args.batch, "global_batch": args.batch * world,
            "train_set": w["train"], "replace": False, "weighted": bool(args.weighted),
            "step": "sample_blocks over %d hops = %d x (%s + tensor_relabel), then features._CAPI_index(input_nodes)"
                    % (len(w["fanouts"]), len(w["fanouts"]), op),
            "storage": "indptr/indices/features in ChunkTensors split evenly over %d GPU(s), %s" % (world, tail),
            "setup": "caching allocator primed (one large block, %d untimed steps) before the warm-up steps" % PRIME_STEPS,
            "l2": "inputs larger than L2 (indices %.2f GB, features %.2f GB); a new seed batch every step"
                  % (n_edges_graph * 8 / 1e9, nodes * dim * 4 / 1e9)}


# ---------------------------------------------------------------------------
# CPU arm (oracle port): used by --impl reference and by the cpu_baseline leg
# ---------------------------------------------------------------------------
def cpu_step(o, indptr, indices, feats, seeds, fanouts):
    frontier, blocks, edges = o.sample_blocks(indptr, indices, seeds, fanouts)
    x = o.index_flat(feats, frontier)
    return edges, frontier.size, x


def run_cpu(args, fanouts, indptr, indices, feats, batches, steps, warmup, budget_s=None):
    from oracle import oracle as o
    o.build()
    for b in range(warmup):
        cpu_step(o, indptr, indices, feats, batches[b % len(batches)], fanouts)
    edges, t0, done = 0, time.perf_counter(), 0
    for b in range(steps):
        e, _, _ = cpu_step(o, indptr, indices, feats, batches[(warmup + b) % len(batches)], fanouts)
        edges += e
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return edges / dt, dt / done * 1e3, done, o.num_threads()


def main_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    w = workload(args)
    nodes, dim, train = w["nodes"], w["dim"], w["train"]
    indptr, indices = build_graph(w, dev)
    n_edges_graph = int(indices.numel())
    feats = make_features(nodes, dim, dev).cpu().numpy()
    indptr, indices = indptr.cpu().numpy(), indices.cpu().numpy()
    batches = synth.train_batches(nodes, train, args.batch)
    value, ms, done, threads = run_cpu(args, w["fanouts"], indptr, indices, feats, batches, args.steps, args.warmup)
    line = {"impl": "reference", "metric": "sampled_edges_per_s", "value": value, "unit": "edges/s",
            "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64",
            "data": "synthetic", "config": config_dict(args, w, n_edges_graph, args.gpus),
            "cpu_baseline": {"value": value, "unit": "edges/s", "cores": threads, "kind": "port",
                             "sample": "%d batches of %d seeds (one per step), CPU restatement of the reference's "
                                       "sample->relabel loop + index_select, OpenMP over seeds" % (done, args.batch)},
            "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def main_ours(args):
    import torch
    import torch.distributed as dist
    pkg = importlib.import_module("dist-gpu-sampling_b200")
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    pkg.load_ops()
    if world > 1:
        pkg.create_dgs_communicator(world)
    ops = torch.ops.dgs_ops

    # ---- data: same graph on every rank, each rank keeps its own chunk ----
    w = workload(args)
    nodes, dim, train, fanouts = w["nodes"], w["dim"], w["train"], w["fanouts"]
    indptr, indices = build_graph(w, dev)
    n_edges_graph = int(indices.numel())
    fill = 1 << 26

    def chunk_capacity(nbytes, frac=1.0):
        cap = -(-int(nbytes * frac) // world)
        return -(-cap // 16) * 16

    def fill_chunk(ct, total, values):
        """values(start, count) -> device tensor of the flat elements [start, start+count)."""
        sub = ct._CAPI_get_sub_device_tensor()
        lo0 = rank * sub.numel()
        for lo in range(0, max(0, min(sub.numel(), total - lo0)), fill):
            n = min(fill, sub.numel() - lo, total - lo0 - lo)
            sub[lo:lo + n] = values(lo0 + lo, n)
        host = ct._CAPI_get_host_tensor()
        if rank == 0 and host.numel():           # the pinned tail is shared: one rank writes it
            thr = total - host.numel()
            for lo in range(0, host.numel(), fill):
                n = min(fill, host.numel() - lo)
                host[lo:lo + n].copy_(values(thr + lo, n))
        return ct

    def to_chunk(t, frac=1.0):
        flat = t.reshape(-1)
        ct = torch.classes.dgs_classes.ChunkTensor(list(t.shape), t.dtype,
                                                   chunk_capacity(flat.numel() * t.element_size(), frac))
        return fill_chunk(ct, flat.numel(), lambda start, count: flat[start:start + count])

    c_indptr = to_chunk(indptr)
    c_indices = to_chunk(indices, w["gpu_frac"])
    c_probs = None
    if args.weighted:
        c_probs = torch.classes.dgs_classes.ChunkTensor([n_edges_graph], torch.float32, chunk_capacity(n_edges_graph * 4))
        fill_chunk(c_probs, n_edges_graph, lambda start, count: edge_weights(start, count, dev))
    # features: every rank fills its own chunk in place
    c_feats = torch.classes.dgs_classes.ChunkTensor([nodes, dim], torch.float32,
                                                    chunk_capacity(nodes * dim * 4, w["gpu_frac"]))
    fill_chunk(c_feats, nodes * dim, lambda start, count: feature_values(start, count, dev))
    host_graph = None
    if rank == 0 and not args.no_cpu_baseline and world == 1 and args.workload in ("products", "small") \
            and not args.weighted:
        host_graph = (indptr.cpu().numpy(), indices.cpu().numpy(), make_features(nodes, dim, dev).cpu().numpy())
    del indptr, indices
    torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()

    batches_np = synth.train_batches(nodes, train, args.batch)
    nb = batches_np.shape[0]
    my = [b for b in range(nb) if b % world == rank]           # disjoint batches per rank
    host_batches = torch.from_numpy(batches_np).pin_memory()
    dev_batches = host_batches.to(dev)
    torch.manual_seed(1234 + rank)

    has_blocks = hasattr(torch.ops.dgs_ops, "_CAPI_sample_blocks")     # absent from the reference's own library
    main_fused = args.api == "blocks" and has_blocks

    def step(seeds, fused=None):
        frontier, blocks, n_edges = pkg.sample_blocks(seeds, fanouts, c_indptr, c_indices, probs=c_probs,
                                                      fused=main_fused if fused is None else fused)
        return frontier, n_edges

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    clocks = ClockSampler(local_rank)
    if rank == 0:
        clocks.start()
    # ---- setup: fill torch's caching allocator (frontier sizes differ from batch to batch, so the first
    # steps of a process still call cudaMalloc), then the W warm-up steps ----
    # one block that covers a step's largest outputs, freed at once: the allocator then carves the steps'
    # buffers out of it instead of growing the pool one cudaMalloc at a time
    n_bound = args.batch
    for k in reversed(fanouts):
        n_bound = min(n_bound * (1 + k), nodes)
    prime = torch.empty(int(2 * n_bound * (dim * 4 + 64)) + (256 << 20), dtype=torch.uint8, device=dev)
    del prime
    for s in range(PRIME_STEPS):
        fr, _ = step(dev_batches[my[(len(my) - 1 - s) % len(my)]])
        c_feats._CAPI_index(fr)
    for s in range(args.warmup):
        fr, _ = step(dev_batches[my[s % len(my)]])
        c_feats._CAPI_index(fr)

    # ---- timed: K steps, seeds resident on the device ----
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    n_before = len(clocks.rows)
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    edges = rows = 0
    kept = []
    t_begin.record()
    for s in range(args.steps):
        seeds = dev_batches[my[(args.warmup + s) % len(my)]]
        ev[s][0].record()
        fr, e = step(seeds)
        ev[s][1].record()
        x = c_feats._CAPI_index(fr)
        ev[s][2].record()
        edges += e
        rows += fr.numel()
        if s >= args.steps - 8:
            kept.append(fr)                      # frontiers for the kernel-timing pass below
    t_end.record()
    barrier()
    n_after = len(clocks.rows)
    total_ms = t_begin.elapsed_time(t_end)
    sample_ms = sum(a.elapsed_time(b) for a, b, _ in ev)
    gather_ms = sum(b.elapsed_time(c) for _, b, c in ev)

    # ---- end to end: seeds from pinned host memory, result read back ----
    def e2e_step(s):
        seeds = host_batches[my[(args.warmup + s) % len(my)]].to(dev, non_blocking=True)
        fr, e = step(seeds)
        x = c_feats._CAPI_index(fr)
        chk = torch.stack([x.sum(), fr.sum().to(torch.float32)]).cpu()   # the step's result leaves the device
        return e, chk.numel() * 4 + 8 * (2 * len(fanouts))               # + the sizes the sampling call reads back

    for s in range(min(args.warmup, 5)):       # the first host->device / device->host round trips are not typical
        e2e_step(s)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e2e_edges, d2h = 0, 0
    e0.record()
    for s in range(args.steps):
        e, d2h = e2e_step(s)
        e2e_edges += e
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clock_info = clocks.stop(n_before, n_after) if rank == 0 else None

    # ---- the same K steps through the other API, for the record ----
    other_ms, other_edges = 0.0, 0
    if has_blocks:
        for s in range(min(args.warmup, 5)):
            fr, _ = step(dev_batches[my[s % len(my)]], fused=not main_fused)
            c_feats._CAPI_index(fr)
        barrier()
        o0 = torch.cuda.Event(enable_timing=True)
        o1 = torch.cuda.Event(enable_timing=True)
        o0.record()
        for s in range(args.steps):
            fr, e = step(dev_batches[my[(args.warmup + s) % len(my)]], fused=not main_fused)
            x = c_feats._CAPI_index(fr)
            other_edges += e
        o1.record()
        barrier()
        other_ms = o0.elapsed_time(o1)

    # ---- the gather kernel on its own: back-to-back launches over the last frontiers, so that the events
    # bracket the kernel and not the host's launch gap (inside a step the host is still busy returning
    # from the relabel operator when the GPU reaches the gather) ----
    barrier()
    n_k = max(16, min(args.steps, 64))
    kev = [torch.cuda.Event(enable_timing=True) for _ in range(n_k + 1)]
    for i in range(3):
        c_feats._CAPI_index(kept[i % len(kept)])
    kev[0].record()
    k_rows = 0
    for i in range(n_k):
        c_feats._CAPI_index(kept[i % len(kept)])
        kev[i + 1].record()
        k_rows += kept[i % len(kept)].numel()
    torch.cuda.synchronize()
    k_ms = sum(kev[i].elapsed_time(kev[i + 1]) for i in range(n_k))
    del kept

    # ---- reduce over ranks: max time, summed work ----
    stats = torch.tensor([total_ms, sample_ms, gather_ms, e2e_ms, other_ms], dtype=torch.float64, device=dev)
    work = torch.tensor([edges, rows, e2e_edges, other_edges], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    total_ms, sample_ms, gather_ms, e2e_ms, other_ms = stats.tolist()
    edges_all, rows_all, e2e_edges_all, other_edges_all = work.tolist()

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        row_alg_bytes = 8 + 2 * dim * 4
        rows_per_launch = k_rows / n_k
        gather_ms_launch = k_ms / n_k
        achieved = rows_per_launch * row_alg_bytes / (gather_ms_launch * 1e-3) / 1e9
        in_step = (rows / args.steps) * row_alg_bytes / (gather_ms / args.steps * 1e-3) / 1e9
        per_row = NCU_TRAFFIC_BYTES_PER_ROW.get(dim)
        line = {
            "library": os.environ.get("DGS_OPS_LIBRARY") or "dist-gpu-sampling_b200/lib/libdgs.so",
            "metric": "sampled_edges_per_s", "value": edges_all / (total_ms * 1e-3), "unit": "edges/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64",
            "data": "synthetic", "config": config_dict(args, w, n_edges_graph, world),
            "breakdown": {"sample_relabel_ms_per_step": sample_ms / args.steps,
                          "gather_ms_per_step": gather_ms / args.steps,
                          "sampling_only_edges_per_s": edges_all / (sample_ms * 1e-3),
                          "edges_per_step_per_rank": edges / args.steps,
                          "input_nodes_per_step_per_rank": rows / args.steps,
                          "gather_payload_gbs_all_ranks": rows_all * dim * 4 / (gather_ms * 1e-3) / 1e9},
            "e2e": {"value": e2e_edges_all / (e2e_ms * 1e-3), "unit": "edges/s",
                    "h2d_bytes_per_step": args.batch * 8, "d2h_bytes_per_step": d2h},
            "gpu_launches": args.steps * ((LAUNCHES_STEP_FUSED + len(fanouts) * LAUNCHES_HOP_FUSED if main_fused else
                                           len(fanouts) * (LAUNCHES_SAMPLE + LAUNCHES_RELABEL)) + LAUNCHES_GATHER),
            "api": API_NAMES[main_fused],
            "other_api": {"api": API_NAMES[not main_fused], "value": other_edges_all / (other_ms * 1e-3),
                          "unit": "edges/s", "ms_per_step": other_ms / args.steps} if other_ms > 0 else None,
            "roofline": {"kernel": "gather_rows_kernel (features._CAPI_index)", "bound": "hbm",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind,
                         "algorithmic_bytes_per_row": row_alg_bytes,
                         "rows_per_launch": rows_per_launch, "ms_per_launch": gather_ms_launch,
                         "launches_timed": n_k,
                         "timing": "CUDA events around %d back-to-back launches on the frontiers of the last "
                                   "timed steps (rank 0)" % n_k,
                         "frac_inside_step": in_step / peak,
                         "traffic": per_row * rows_per_launch if per_row else None},
            "clocks": clock_info,
        }
        if host_graph is not None:
            v, ms, done, threads = run_cpu(args, fanouts, host_graph[0], host_graph[1], host_graph[2], batches_np,
                                           steps=10 ** 6, warmup=1, budget_s=args.cpu_seconds)
            line["cpu_baseline"] = {"value": v, "unit": "edges/s", "cores": threads, "kind": "port",
                                    "sample": "%d batches of %d seeds in %.1f s (same graph and step)"
                                              % (done, args.batch, done * ms / 1e3)}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    del c_indptr, c_indices, c_feats, c_probs     # collective teardown, same order on every rank
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        main_reference(a)
    else:
        main_ours(a)
