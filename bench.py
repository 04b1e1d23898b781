"""Benchmark of the hot path: 3-hop neighbour sampling + relabel + feature gather.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--workload products|papers100m|friendster|small] [--batch 1024] [--weighted] [--scale F]
                  [--api pipeline|blocks|per-hop] [--depth D] [--consumer-stream high|default]

One step = one mini-batch per rank:
  frontier, blocks = sample_blocks(seeds, [15, 10, 5])      # sample + relabel, fan-outs applied last to first
  x = features._CAPI_index(frontier)
Three ways through the library, all timed in the same run over the same K batches:
  pipeline  (headline) torch.classes.dgs_classes.BlockPipeline: `--depth` batches in flight, each on its own
            stream; a batch's hops are queued as one launch sequence and its feature gather directly behind it
            (row count taken from the device), so nothing is read back while a batch runs
  blocks    one batch at a time: _CAPI_sample_blocks_with_chunk_tensor, then features._CAPI_index
  per-hop   the reference's own operator sequence, one batch at a time: _CAPI_sample_neighbors_with_chunk_tensor
            + _CAPI_tensor_relabel per hop, then features._CAPI_index
The graph is a Products-shaped synthetic graph (2,449,029 nodes, ~123.7 M edges, Chung-Lu power law, 100 fp32
features per node) whose indptr / indices / features live in ChunkTensors split evenly over the N GPUs of the
node (weak scaling: every rank samples its own 1,024-seed batches; no collective on the data path).
`--workload papers100m` is the Papers100M-shaped configuration (111 M nodes, ~1.6 B edges, 128 features: 70 GB,
which fits one B200 or is split over N); unless `--no-extra-configs` is given it is also measured, briefly, at
the end of a default (Products) run and reported under `configs`.  `--workload friendster` is the
Friendster-shaped hybrid configuration: fan-out [10, 10], 256 features, node ids ranked by in-degree, 40 % of
features and indices in the pinned host tail; it runs at a quarter of the node count by default (`--scale 1`
for the full 65.6 M nodes / 3.6 B edges, which pins ~38 GB of host memory).  `--weighted` samples with per-edge
weights.

Printed JSON (rank 0, one line):
  value        sampled edges/s of the whole job, device-timed, seeds resident in HBM; step = sample + relabel + gather
  e2e          same metric with every batch's seeds coming from pinned host memory and a device->host read of the
               step's checksum inside the timed region (the result itself stays on the device, as in the
               reference's API); the consumer -- two reduction kernels and the copy -- runs on a high-priority
               stream, `--consumer-stream default` puts it on a default-priority one; e2e_full_d2h: the variant that copies input nodes, blocks and features to
               pinned host buffers every step
  roofline     the gather kernel (`pipeline_form`: the same through the call the pipeline makes): bytes of the binding class / CUDA-event time of back-to-back launches on the
               last frontiers, against that class's peak -- local HBM at N = 1, NVLink at N > 1 -- with the
               per-class bytes and the time-weighted bound t_min = max(B_hbm/BW_hbm, B_nvl/BW_nvl, B_host/BW_host)
  verified     one untimed batch checked on the device: counts = min(deg, k), every (row, col) an edge of the
               graph, gathered rows = the generator's values
  cpu_baseline the CPU oracle (port of the reference algorithm) on a bounded sample, all host threads
  ref_gpu_baseline  the reference's own kernels compiled for this GPU, same step, in a subprocess (N = 1 only;
               "unavailable" when that library was not built)

`--impl reference` times the CPU port alone on all host threads (the reference project has no CPU
implementation of its own and its DGL baseline is not installable here); under torchrun only rank 0 works.
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

# kernels of this library launched per operator call (memsets and copies are not kernels)
LAUNCHES_SAMPLE = 2      # plan (+ tile scan in its last CTA), sample
LAUNCHES_RELABEL = 4     # insert, count (+ tile scan in its last CTA), number, lookup
LAUNCHES_GATHER = 1
LAUNCHES_HOP_FUSED = 5   # plan (+ table clear + previous hop's lookup), sample, insert, count, number
LAUNCHES_STEP_FUSED = 2  # init words, last hop's lookup
PRIME_STEPS = 8          # untimed one-at-a-time steps that populate torch's caching allocator
API_NAMES = {
    "pipeline": "BlockPipeline: %d batches in flight, each = one queued sample_blocks sequence + device-counted gather",
    "blocks": "_CAPI_sample_blocks* (all hops queued as one sequence, one size read-back per step), then _CAPI_index",
    "per-hop": "reference operator sequence: _CAPI_sample_neighbors* + _CAPI_tensor_relabel per hop, then _CAPI_index",
}
# DRAM bytes per gathered row (read + write) measured with ncu for this row width; None where no capture exists
NCU_TRAFFIC_BYTES_PER_ROW = {100: 861.2}
NVLINK_FALLBACK_GBS = 770.0   # this pool's measured peer copy, used only when the run cannot measure one


def workload(name, args):
    """Workload parameters with --scale applied to the node count (edges follow: the mean degree is fixed)."""
    w = dict(WORKLOADS[name])
    scale = args.scale if args.scale > 0 else (0.25 if name == "friendster" else 1.0)
    w["name"] = name
    w["scale"] = scale
    w["nodes"] = max(1000, int(w["nodes"] * scale))
    w["train"] = max(args.batch, min(w["train"], w["nodes"] // 2))
    return w


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
    ap.add_argument("--api", default="pipeline", choices=["pipeline", "blocks", "per-hop"],
                    help="which of the three ways through the library is the headline `value`; the other two are "
                         "timed too and reported under other_api")
    ap.add_argument("--depth", type=int, default=6, help="batches in flight in the pipeline")
    ap.add_argument("--consumer-stream", default="high", choices=["high", "default"],
                    help="priority of the stream the e2e consumer (checksum kernels, copies) runs on")
    ap.add_argument("--no-extra-configs", action="store_true",
                    help="skip the short Papers100M-shaped measurement at the end of a default run")
    ap.add_argument("--extra-steps", type=int, default=200, help="timed steps of that extra measurement")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip the reference-kernels-on-this-GPU leg")
    ap.add_argument("--ref-gpu-worker", action="store_true", help=argparse.SUPPRESS)
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
    """Same seeded graph on every rank (generated on `device`).  Workloads that keep part of their tensors in the
    host tail get their node ids ranked by in-degree with the library's own renumbering step (hot rows first, so
    that they land in the GPU chunks) -- what a user with a real graph would call before creating ChunkTensors."""
    pkg = importlib.import_module("dist-gpu-sampling_b200")
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    indptr, indices = synth.chung_lu_csc(w["nodes"], w["mean_deg"], w["gamma"], seed=11, device=device)
    if w["degree_sorted"]:
        indptr, indices, _, _ = pkg.renumber_by_degree(indptr, indices, by="in", with_edge_source=False)
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
                        "features [%d,%d] fp32" % (w["name"], "" if w["scale"] == 1.0 else " at scale %.2f" % w["scale"],
                                                   nodes, n_edges_graph, w["gamma"], nodes, dim),
            "fanouts": w["fanouts"], "batch_per_rank": args.batch, "global_batch": args.batch * world,
            "train_set": w["train"], "replace": False, "weighted": bool(args.weighted),
            "step": "sample_blocks over %d hops = %d x (%s + tensor_relabel), then features._CAPI_index(input_nodes)"
                    % (len(w["fanouts"]), len(w["fanouts"]), op),
            "storage": "indptr/indices/features in ChunkTensors split evenly over %d GPU(s) in whole rows "
                       "(the up to N-1 rows that do not divide evenly sit in the host tail), %s" % (world, tail),
            "l2": "inputs larger than L2 (indices %.2f GB, features %.2f GB); a new seed batch every step"
                  % (n_edges_graph * 8 / 1e9, nodes * dim * 4 / 1e9)}


# ---------------------------------------------------------------------------
# CPU arm (oracle port): used by --impl reference and by the cpu_baseline leg
# ---------------------------------------------------------------------------
def cpu_step(o, indptr, indices, feats, seeds, fanouts):
    frontier, blocks, edges = o.sample_blocks(indptr, indices, seeds, fanouts)
    x = o.index_flat(feats, frontier)
    return edges, frontier.size, x


def run_cpu(fanouts, indptr, indices, feats, batches, steps, warmup, budget_s=None):
    import torch
    from oracle import oracle as o
    o.build()
    threads = o.use_all_cores()          # not the OMP_NUM_THREADS=1 a launcher may have exported
    torch.set_num_threads(threads)
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
    return edges / dt, dt / done * 1e3, done, threads


def main_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    w = workload(args.workload, args)
    nodes, dim, train = w["nodes"], w["dim"], w["train"]
    indptr, indices = build_graph(w, dev)
    n_edges_graph = int(indices.numel())
    feats = make_features(nodes, dim, dev).cpu().numpy()
    indptr, indices = indptr.cpu().numpy(), indices.cpu().numpy()
    batches = synth.train_batches(nodes, train, args.batch)
    value, ms, done, threads = run_cpu(w["fanouts"], indptr, indices, feats, batches, args.steps, args.warmup)
    line = {"impl": "reference", "metric": "sampled_edges_per_s", "value": value, "unit": "edges/s",
            "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64",
            "data": "synthetic", "config": config_dict(args, w, n_edges_graph, args.gpus),
            "cpu_baseline": {"value": value, "unit": "edges/s", "cores": threads, "kind": "port",
                             "sample": "%d batches of %d seeds (one per step), CPU restatement of the reference's "
                                       "sample->relabel loop + index_select, OpenMP over seeds" % (done, args.batch),
                             "note": "one host's figure: at --gpus N > 1 the CPU arm still runs once, on rank 0, "
                                     "with all of the host's cores; it is not a per-rank number"},
            "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# the reference's own kernels on this GPU (a build of its sources; subprocess of the N = 1 run)
# ---------------------------------------------------------------------------
def ref_gpu_library():
    return os.path.join(ROOT, "oracle", "_ref", "libdgs_reference.so")


def main_ref_gpu_worker(args):
    """Runs in a process of its own, which loads the reference's operator library instead of this package's
    (same operator names, so the per-hop step below is the reference's own call sequence,
    oppo_bench/single_node/utils/chunktensor_sampler.py:93-118 + chunktensor.py:147-150)."""
    import torch
    pkg = importlib.import_module("dist-gpu-sampling_b200")      # Python glue only; its libraries are not loaded
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    torch.ops.load_library(ref_gpu_library())
    ops = torch.ops.dgs_ops
    ops._CAPI_set_nccl(1, ops._CAPI_get_unique_id(), 0)          # its ChunkTensor constructor wants a communicator
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    w = workload(args.workload, args)
    nodes, dim, fanouts = w["nodes"], w["dim"], w["fanouts"]
    indptr, indices = build_graph(w, dev)
    CT = torch.classes.dgs_classes.ChunkTensor

    def to_chunk(t):
        ct = CT(list(t.shape), t.dtype, t.numel() * t.element_size())
        ct._CAPI_get_sub_device_tensor()[:t.numel()] = t.reshape(-1)
        return ct

    c_indptr, c_indices = to_chunk(indptr), to_chunk(indices)
    c_feats = to_chunk(make_features(nodes, dim, dev))
    del indptr, indices
    batches = torch.from_numpy(synth.train_batches(nodes, w["train"], args.batch)).to(dev)

    def step(i):
        fr, _, e = pkg.sample_blocks(batches[i % batches.shape[0]], fanouts, c_indptr, c_indices, fused=False)
        c_feats._CAPI_index(fr)
        return e
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    edges = 0
    t0.record()
    for i in range(args.steps):
        edges += step(args.warmup + i)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    print("REFGPU " + json.dumps({"value": edges / (ms * 1e-3), "unit": "edges/s", "ms_per_step": ms / args.steps,
                                  "steps": args.steps, "warmup": args.warmup,
                                  "what": "the reference's CUDA sources compiled unmodified for sm_100a, its own "
                                          "operator sequence (sample + relabel per hop, then _CAPI_index), same "
                                          "graph, batches and step as `value`"}), flush=True)


def run_ref_gpu(args, steps):
    if not os.path.exists(ref_gpu_library()):
        return {"unavailable": "the reference's kernels were not built for this GPU (oracle/_ref/ has no "
                               "reference library; oracle/build_reference.sh builds it where the sources are)"}
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS")}
    cmd = [sys.executable, os.path.abspath(__file__), "--ref-gpu-worker", "--workload", args.workload,
           "--batch", str(args.batch), "--steps", str(steps), "--warmup", "10"]
    if args.scale > 0:
        cmd += ["--scale", str(args.scale)]
    try:
        r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    except Exception as e:      # noqa: BLE001
        return {"unavailable": "the reference-kernel subprocess did not finish: %r" % (e,)}
    for ln in r.stdout.splitlines():
        if ln.startswith("REFGPU "):
            return json.loads(ln[7:])
    return {"unavailable": "the reference-kernel subprocess failed (exit %d): %s" % (r.returncode, r.stdout[-300:])}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class Env:
    pass


def measure_link_peaks(env):
    """Peak of each link a gather can be bound by, measured here with plain copies (best of several):
    pinned host -> device, and peer GPU -> this GPU where there is a peer.  Rank 0 measures, the others wait."""
    import torch
    dev, world = env.dev, env.world
    peaks = {"host_gbs": None, "nvlink_gbs": None, "nvlink_kind": "none (one GPU)"}
    if env.rank == 0:
        n = 1 << 28
        dst = torch.empty(n, dtype=torch.uint8, device=dev)
        src = torch.empty(n, dtype=torch.uint8).pin_memory()
        best = 1e30
        for _ in range(6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b))
        peaks["host_gbs"] = n / best / 1e6
        del src
        if world > 1:
            try:
                peer = torch.device("cuda", (env.local_rank + 1) % world)
                psrc = torch.empty(n, dtype=torch.uint8, device=peer)
                dst.copy_(psrc)
                torch.cuda.synchronize(dev)
                torch.cuda.synchronize(peer)
                best = 1e30
                for _ in range(6):
                    t0 = time.perf_counter()
                    for _ in range(8):
                        dst.copy_(psrc)
                    torch.cuda.synchronize(peer)
                    torch.cuda.synchronize(dev)
                    best = min(best, (time.perf_counter() - t0) / 8)
                peaks["nvlink_gbs"] = n / best / 1e9
                peaks["nvlink_kind"] = "measured: peer copy of 256 MiB, best of 6"
                del psrc
            except Exception as e:      # noqa: BLE001
                peaks["nvlink_gbs"] = NVLINK_FALLBACK_GBS
                peaks["nvlink_kind"] = "fallback (peer copy failed here: %r)" % (e,)
        del dst
        torch.cuda.empty_cache()
    env.barrier()
    return peaks


def setup_workload(env, args, w, want_host_graph):
    """ChunkTensors of one workload, filled in place; returns an object with everything a measurement needs."""
    import torch
    import torch.distributed as dist
    pkg = importlib.import_module("dist-gpu-sampling_b200")
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    dev, world, rank = env.dev, env.world, env.rank
    nodes, dim = w["nodes"], w["dim"]
    indptr, indices = build_graph(w, dev)
    n_edges_graph = int(indices.numel())
    fill = 1 << 26

    def chunk_capacity(nbytes, row_bytes, frac=1.0):
        """An equal share per GPU, cut to whole rows (the package's create_chunktensor rule): with a capacity
        that is not a whole number of rows the reference's placement arithmetic (src/chunk_tensor.cc:57-68) puts
        the rows of every later chunk off the 16-byte grid and the gather has to fall back to narrow loads.  The
        rows that do not divide evenly (at most world - 1 of them) end up in the host tail."""
        if world == 1 and frac >= 1.0:
            return nbytes
        return pkg.cached_size_per_gpu(nbytes, world, 1 << 62, frac, row_bytes)

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
        row_bytes = t.element_size() * (t.shape[1] if t.dim() == 2 else 1)
        ct = torch.classes.dgs_classes.ChunkTensor(list(t.shape), t.dtype,
                                                   chunk_capacity(flat.numel() * t.element_size(), row_bytes, frac))
        return fill_chunk(ct, flat.numel(), lambda start, count: flat[start:start + count])

    wl = Env()
    wl.w, wl.n_edges_graph = w, n_edges_graph
    wl.c_indptr = to_chunk(indptr)
    wl.c_indices = to_chunk(indices, w["gpu_frac"])
    wl.c_probs = None
    if args.weighted:
        wl.c_probs = torch.classes.dgs_classes.ChunkTensor([n_edges_graph], torch.float32,
                                                           chunk_capacity(n_edges_graph * 4, 4))
        fill_chunk(wl.c_probs, n_edges_graph, lambda start, count: edge_weights(start, count, dev))
    # features: every rank fills its own chunk in place
    wl.c_feats = torch.classes.dgs_classes.ChunkTensor([nodes, dim], torch.float32,
                                                       chunk_capacity(nodes * dim * 4, dim * 4, w["gpu_frac"]))
    fill_chunk(wl.c_feats, nodes * dim, lambda start, count: feature_values(start, count, dev))
    wl.host_graph = None
    if want_host_graph:
        wl.host_graph = (indptr.cpu().numpy(), indices.cpu().numpy(), make_features(nodes, dim, dev).cpu().numpy())
    del indptr, indices
    torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
    wl.batches_np = synth.train_batches(nodes, w["train"], args.batch)
    nb = wl.batches_np.shape[0]
    wl.my = [b for b in range(nb) if b % world == rank]           # disjoint batches per rank
    wl.host_batches = torch.from_numpy(wl.batches_np).pin_memory()
    wl.dev_batches = wl.host_batches.to(dev)
    return wl


def teardown_workload(env, wl):
    import torch
    # collective teardown, same order on every rank
    wl.c_indptr = wl.c_indices = wl.c_feats = wl.c_probs = None
    torch.cuda.empty_cache()
    env.barrier()


def verify_batch(env, pkg, wl, seeds, frontier, blocks, x, max_adjacency=40_000_000):
    """One batch checked on the device against the graph in the ChunkTensors and the feature generator.
    Returns a dict of what was checked; raises AssertionError on the first violation."""
    import torch
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    w = wl.w
    nodes, dim = w["nodes"], w["dim"]
    applied = list(reversed(w["fanouts"]))
    H = len(applied)
    cur = seeds
    checked_edges = checked_rows = 0
    for h in range(H):
        row_l, col_l, n_src, n_dst = blocks[H - 1 - h]
        k = applied[h]
        assert n_dst == cur.numel(), "block %d: n_dst" % h
        fr = frontier[:n_src]
        lo = wl.c_indptr._CAPI_index(cur).view(-1)
        hi = wl.c_indptr._CAPI_index(cur + 1).view(-1)
        deg = hi - lo
        cnt = torch.clamp(deg, max=k)
        assert int(cnt.sum()) == row_l.numel() == col_l.numel(), "block %d: edge count is not sum(min(deg, k))" % h
        row_g, col_g = fr[row_l], fr[col_l]
        assert torch.equal(row_g, torch.repeat_interleave(cur, cnt)), "block %d: rows are not the seeds repeated" % h
        assert torch.equal(fr[:n_dst], cur), "block %d: the seeds do not lead the frontier" % h
        # every (row, col) is an edge: compare with the seeds' full adjacency (a bounded share of the seeds)
        csum = torch.cumsum(deg, 0)
        take = int(torch.searchsorted(csum, torch.tensor([max_adjacency], device=csum.device)).item())
        take = max(1, min(take, cur.numel()))
        n_adj = int(csum[take - 1])
        seg = torch.repeat_interleave(torch.arange(take, device=cur.device), deg[:take])
        start = csum[:take] - deg[:take]
        pos = lo[:take][seg] + (torch.arange(n_adj, device=cur.device) - start[seg])
        nb = wl.c_indices._CAPI_index(pos).view(-1)
        adj_keys = seg * nodes + nb
        n_out = int(cnt[:take].sum())
        out_seg = torch.repeat_interleave(torch.arange(take, device=cur.device), cnt[:take])
        out_keys = out_seg * nodes + col_g[:n_out]
        assert bool(torch.isin(out_keys, adj_keys).all()), "block %d: a sampled (row, col) is not an edge" % h
        # whole rows (deg <= k) come out in CSC order
        whole = (deg[:take] <= k)[out_seg]
        whole_adj = (deg[:take] <= k)[seg]
        assert torch.equal(out_keys[whole], adj_keys[whole_adj]), "block %d: a whole row is not in CSC order" % h
        checked_edges += n_out
        del seg, pos, nb, adj_keys, out_keys, out_seg
        cur = fr
    assert torch.equal(cur, frontier) and torch.unique(frontier).numel() == frontier.numel(), "frontier has repeats"
    # gathered rows = the generator's values
    step = max(1, (1 << 24) // dim)
    for lo_r in range(0, frontier.numel(), step):
        ids = frontier[lo_r:lo_r + step]
        flat = (ids[:, None] * dim + torch.arange(dim, device=ids.device)[None, :]).reshape(-1)
        assert torch.equal(x[lo_r:lo_r + step].reshape(-1), synth.hash_of_index(flat, 3)), "a gathered row differs"
        checked_rows += ids.numel()
    return {"edges_checked": checked_edges, "rows_checked": checked_rows, "hops": H}


def measure_workload(env, args, pkg, wl, steps, warmup, full):
    """All timed passes over one workload.  `full`: also the serial APIs' breakdown, e2e variants, the gather
    kernel on its own and the verification (the short extra configuration skips some of these)."""
    import torch
    import torch.distributed as dist
    dev, world, rank = env.dev, env.world, env.rank
    w = wl.w
    fanouts, dim, nodes = w["fanouts"], w["dim"], w["nodes"]
    H = len(fanouts)
    my, dev_batches, host_batches = wl.my, wl.dev_batches, wl.host_batches
    res = {}

    sampler = pkg.PipelinedSampler(wl.c_indptr, wl.c_indices, fanouts, features=wl.c_feats, probs=wl.c_probs,
                                   max_seeds=args.batch, depth=args.depth)

    def batch_ids(first, count):
        return [my[(first + s) % len(my)] for s in range(count)]

    def serial_step(seeds, api):
        frontier, blocks, n_edges = pkg.sample_blocks(seeds, fanouts, wl.c_indptr, wl.c_indices, probs=wl.c_probs,
                                                      fused=(api == "blocks"))
        return frontier, blocks, n_edges

    def timed_pipeline(seed_source, ids, consume=None):
        """K batches through the pipeline; CUDA events on the current stream, which every next() orders
        after the slot it hands out."""
        env.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        edges = rows = 0
        t0.record()
        for fr, blocks, e, x in sampler(seed_source[b] for b in ids):
            edges += e
            rows += fr.numel()
            if consume is not None:
                consume(fr, blocks, x)
        t1.record()
        env.barrier()
        return t0.elapsed_time(t1), edges, rows

    def timed_serial(api, ids, breakdown=False):
        env.barrier()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in ids] if breakdown else None
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        edges = rows = 0
        t0.record()
        for s, b in enumerate(ids):
            if breakdown:
                ev[s][0].record()
            fr, _, e = serial_step(dev_batches[b], api)
            if breakdown:
                ev[s][1].record()
            wl.c_feats._CAPI_index(fr)
            if breakdown:
                ev[s][2].record()
            edges += e
            rows += fr.numel()
        t1.record()
        env.barrier()
        out = {"ms": t0.elapsed_time(t1), "edges": edges, "rows": rows}
        if breakdown:
            out["sample_ms"] = sum(a.elapsed_time(b) for a, b, _ in ev)
            out["gather_ms"] = sum(b.elapsed_time(c) for _, b, c in ev)
        return out

    # The e2e loops (submit, next, and the consumer of a batch) run on a HIGH-priority stream unless
    # --consumer-stream default is given: see below.  The `value` pass has no consumer kernels and runs on
    # torch's default stream (measured the same either way).
    consumer_stream = torch.cuda.Stream(device=dev, priority=-1 if args.consumer_stream == "high" else 0)

    # ---- warm-up: W steps through every path that is timed below ----
    n_warm = max(warmup, 3)
    timed_pipeline(dev_batches, batch_ids(len(my) - n_warm, n_warm))
    # one large block allocated and freed, then a few one-at-a-time steps: the serial paths allocate their
    # outputs per call, and frontier sizes differ from batch to batch
    n_bound = args.batch
    for k in reversed(fanouts):
        n_bound = min(n_bound * (1 + k), nodes)
    prime = torch.empty(int(2 * n_bound * (dim * 4 + 64)) + (256 << 20), dtype=torch.uint8, device=dev)
    del prime
    for api in ("blocks", "per-hop"):
        for b in batch_ids(len(my) - PRIME_STEPS, PRIME_STEPS if full else 3):
            fr, _, _ = serial_step(dev_batches[b], api)
            wl.c_feats._CAPI_index(fr)

    ids = batch_ids(warmup, steps)
    # ---- timed: K steps, seeds resident on the device ----
    kept = []

    def keep(fr, blocks, x):
        if len(kept) < 8:
            kept.append(fr.clone())              # (a batch's tensors are views of its slot)
    # The one-batch-at-a-time APIs are timed first and the headline pass last, directly behind its own W
    # warm-up steps: with a short run (K = 20 is 3 ms of device time) the first timed pass would otherwise
    # also measure the GPU coming out of idle.
    blocks_t = timed_serial("blocks", ids, breakdown=True)
    perhop_t = timed_serial("per-hop", ids) if full else None
    timed_pipeline(dev_batches, batch_ids(len(my) - n_warm, n_warm))
    clocks_lo = len(env.clocks.rows) if env.clocks else 0
    pipe_ms, pipe_edges, pipe_rows = timed_pipeline(dev_batches, ids, keep)
    clocks_hi = len(env.clocks.rows) if env.clocks else 0
    res["clock_window"] = (clocks_lo, clocks_hi)
    res["pipeline"] = {"ms": pipe_ms, "edges": pipe_edges, "rows": pipe_rows}
    res["blocks"], res["per-hop"] = blocks_t, perhop_t

    # ---- end to end: seeds from pinned host memory, the step's result read back ----
    # The consumer of a batch (here the checksum; in training the GNN layers) runs on a HIGH-priority stream:
    # its kernels are then placed ahead of the thousands of queued CTAs of the sampling kernels, which run at
    # the default (lowest) priority.  Measured: four small dependent consumer kernels per step cost 0.146 ms
    # per step on a default-priority stream and 0.129 ms (nothing) on a high-priority one.
    chk_host = torch.zeros((64, 2), dtype=torch.float32).pin_memory()
    chk_dev = torch.zeros(2, dtype=torch.float32, device=dev)
    chk_state = {"i": 0}

    def checksum(fr, blocks, x):
        # 8 bytes leave the device every step, into a ring of pinned words: a checksum of the last 1 024
        # gathered rows and input nodes (what the gather kernel writes last; the copy is ordered behind the
        # whole batch on the stream either way).  The copies are asynchronous, the barrier that closes the
        # timed region waits for all of them.
        torch.sum(x[-1024:], dim=(0, 1), out=chk_dev[0])
        torch.sum(fr[-1024:], dim=(0,), dtype=torch.float32, out=chk_dev[1])
        chk_host[chk_state["i"] % 64].copy_(chk_dev, non_blocking=True)
        chk_state["i"] += 1
    with torch.cuda.stream(consumer_stream):
        timed_pipeline(host_batches, batch_ids(0, min(n_warm, 5)), checksum)
        e2e_ms, e2e_edges, _ = timed_pipeline(host_batches, ids, checksum)
    res["e2e"] = {"ms": e2e_ms, "edges": e2e_edges, "d2h_bytes_per_step": 8 + 8 * 2 * H}

    if full:
        # ---- end to end with the whole result copied out: input nodes, blocks, features -> pinned host buffers
        # (two sets, so that one step's copies overlap the next step's sampling) ----
        bounds, nb_ = [], args.batch
        for k in reversed(fanouts):
            bounds.append((nb_ * k, min(nb_ * (1 + k), nodes)))
            nb_ = bounds[-1][1]
        host_sets = []
        for _ in range(2):
            hs = {"fr": torch.empty(nb_, dtype=torch.int64).pin_memory(),
                  "x": torch.empty((nb_, dim), dtype=torch.float32).pin_memory(),
                  "rows": [torch.empty(e, dtype=torch.int64).pin_memory() for e, _ in bounds],
                  "cols": [torch.empty(e, dtype=torch.int64).pin_memory() for e, _ in bounds],
                  "event": torch.cuda.Event()}
            host_sets.append(hs)
        state = {"i": 0, "bytes": 0}

        def copy_out(fr, blocks, x):
            hs = host_sets[state["i"] % 2]
            hs["event"].synchronize()                          # this set's previous copies have landed
            n = fr.numel()
            hs["fr"][:n].copy_(fr, non_blocking=True)
            hs["x"][:n].copy_(x, non_blocking=True)
            nbytes = n * 8 + n * dim * 4
            for h, (r, c, _, _) in enumerate(reversed(blocks)):
                hs["rows"][h][:r.numel()].copy_(r, non_blocking=True)
                hs["cols"][h][:c.numel()].copy_(c, non_blocking=True)
                nbytes += 16 * r.numel()
            hs["event"].record()
            state["i"] += 1
            state["bytes"] += nbytes
        with torch.cuda.stream(consumer_stream):
            timed_pipeline(host_batches, batch_ids(0, min(n_warm, 5)), copy_out)
            state["bytes"] = 0
            full_ms, full_edges, _ = timed_pipeline(host_batches, ids, copy_out)
        res["e2e_full"] = {"ms": full_ms, "edges": full_edges, "d2h_bytes_per_step": state["bytes"] / steps + 8 * 2 * H}
        del host_sets

    # ---- the gather kernel on its own: back-to-back launches over the last frontiers, so that the events
    # bracket the kernel and not the host's launch gap; and the location classes of those frontiers ----
    env.barrier()
    n_k = max(16, min(steps, 64))
    kev = [torch.cuda.Event(enable_timing=True) for _ in range(n_k + 1)]
    for i in range(3):
        wl.c_feats._CAPI_index(kept[i % len(kept)])
    kev[0].record()
    k_rows = 0
    for i in range(n_k):
        wl.c_feats._CAPI_index(kept[i % len(kept)])
        kev[i + 1].record()
        k_rows += kept[i % len(kept)].numel()
    torch.cuda.synchronize()
    res["kernel"] = {"ms": sum(kev[i].elapsed_time(kev[i + 1]) for i in range(n_k)), "launches": n_k, "rows": k_rows}
    # the same launches in the form the pipeline queues per batch (row count on the device; bulk-copy kernel
    # where the rows qualify)
    counts = [torch.tensor([fr.numel()], dtype=torch.int64, device=dev) for fr in kept]
    for i in range(3):
        wl.c_feats._CAPI_index_counted(kept[i % len(kept)], counts[i % len(kept)])
    kev[0].record()
    for i in range(n_k):
        wl.c_feats._CAPI_index_counted(kept[i % len(kept)], counts[i % len(kept)])
        kev[i + 1].record()
    torch.cuda.synchronize()
    res["kernel_counted"] = {"ms": sum(kev[i].elapsed_time(kev[i + 1]) for i in range(n_k)), "launches": n_k,
                             "rows": k_rows}
    cls = [0, 0, 0]
    for fr in kept:
        for j, part in enumerate(wl.c_feats._CAPI_split_index(fr)):
            cls[j] += part.numel()
    tot = max(1, sum(cls))
    res["class_share"] = {"local": cls[0] / tot, "peer": cls[1] / tot, "host": cls[2] / tot}
    env.barrier()

    # ---- untimed verification of one batch through the headline path ----
    if full:
        try:
            b = my[(warmup + steps) % len(my)]
            torch.manual_seed(99 + rank)
            (fr, blocks, e, x), = list(sampler([dev_batches[b]]))
            res["verified"] = dict(verify_batch(env, pkg, wl, dev_batches[b], fr, blocks, x), ok=True)
        except AssertionError as err:
            res["verified"] = {"ok": False, "error": str(err)}
    del sampler, kept
    return res


def reduce_over_ranks(env, res):
    """max of the times, sum of the work, over ranks."""
    import torch
    import torch.distributed as dist
    keys = [("pipeline", "ms"), ("blocks", "ms"), ("blocks", "sample_ms"), ("blocks", "gather_ms"), ("per-hop", "ms"),
            ("e2e", "ms"), ("e2e_full", "ms")]
    works = [("pipeline", "edges"), ("pipeline", "rows"), ("blocks", "edges"), ("blocks", "rows"), ("per-hop", "edges"),
             ("e2e", "edges"), ("e2e_full", "edges")]
    get = lambda a, b: float(res[a][b]) if res.get(a) and b in res[a] else 0.0      # noqa: E731
    t = torch.tensor([get(a, b) for a, b in keys], dtype=torch.float64, device=env.dev)
    wk = torch.tensor([get(a, b) for a, b in works], dtype=torch.float64, device=env.dev)
    ok = torch.tensor([1.0 if res.get("verified", {"ok": True}).get("ok") else 0.0], dtype=torch.float64, device=env.dev)
    if env.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(wk, op=dist.ReduceOp.SUM)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    out = {}
    for (a, b), v in zip(keys, t.tolist()):
        out.setdefault(a, {})[b] = v
    for (a, b), v in zip(works, wk.tolist()):
        out.setdefault(a, {})[b + "_all"] = v
    out["verified_all"] = bool(ok.item() > 0.5)
    return out


def roofline_dict(res, w, peaks, hbm_peak, hbm_kind):
    """The gather kernel against the roofline of the class that binds it."""
    dim = w["dim"]
    k = res["kernel"]
    rows = k["rows"] / k["launches"]
    ms = k["ms"] / k["launches"]
    sh = res["class_share"]
    row_bytes = dim * 4
    n_loc, n_peer, n_host = rows * sh["local"], rows * sh["peer"], rows * sh["host"]
    # bytes per launch that each resource has to move
    b_hbm = n_loc * (8 + 2 * row_bytes) + (n_peer + n_host) * (8 + row_bytes)    # ids + local reads + all writes
    b_nvl = n_peer * row_bytes
    b_host = n_host * row_bytes
    nvl_peak = peaks.get("nvlink_gbs") or NVLINK_FALLBACK_GBS
    host_peak = peaks.get("host_gbs") or 50.0
    t = {"hbm": b_hbm / (hbm_peak * 1e9), "nvlink": b_nvl / (nvl_peak * 1e9), "host": b_host / (host_peak * 1e9)}
    bound = max(t, key=t.get)
    bytes_of = {"hbm": b_hbm, "nvlink": b_nvl, "host": b_host}[bound]
    peak = {"hbm": hbm_peak, "nvlink": nvl_peak, "host": host_peak}[bound]
    achieved = bytes_of / (ms * 1e-3) / 1e9
    per_row = NCU_TRAFFIC_BYTES_PER_ROW.get(dim)
    kc = res.get("kernel_counted")
    ms_counted = kc["ms"] / kc["launches"] if kc else None
    return {"kernel": "gather_rows_kernel (features._CAPI_index; the register form, used by the one-batch-at-a-time "
                      "APIs)", "bound": bound,
            "pipeline_form": None if ms_counted is None else {
                "kernel": "gather_rows_bulk_kernel where rows are 16-byte aligned multiples of 16 bytes between 256 "
                          "and 8192 bytes, else gather_rows_kernel (features._CAPI_index_counted = "
                          "dgs_gather_rows_counted, what BlockPipeline queues per batch)",
                "ms_per_launch": ms_counted, "achieved": bytes_of / (ms_counted * 1e-3) / 1e9,
                "frac": bytes_of / (ms_counted * 1e-3) / 1e9 / peak},
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_kind": {"hbm": hbm_kind + " (MEASURED_PEAKS.json hbm_gbs)", "nvlink": peaks.get("nvlink_kind"),
                          "host": "measured: pinned host->device copy of 256 MiB, best of 6"}[bound],
            "t_min_ms": t[bound] * 1e3, "ms_per_launch": ms, "t_min_over_t": t[bound] * 1e3 / ms,
            "rows_per_launch": rows, "launches_timed": k["launches"],
            "timing": "CUDA events around back-to-back launches on the frontiers of the last timed steps (rank 0)",
            "classes": {
                "local": {"rows": n_loc, "bytes": n_loc * (8 + 2 * row_bytes), "bytes_per_row": 8 + 2 * row_bytes,
                          "peak_gbs": hbm_peak, "t_ms": t["hbm"] * 1e3},
                "peer": {"rows": n_peer, "bytes": b_nvl, "bytes_per_row": row_bytes, "peak_gbs": nvl_peak,
                         "t_ms": t["nvlink"] * 1e3, "achieved_gbs_if_alone": b_nvl / (ms * 1e-3) / 1e9,
                         # a row that starts on a 16-byte boundary covers this many 128-byte lines, each one
                         # read request on the link; the link moves requests, not bytes, at a fixed rate
                         "line_requests_per_row": -(-(row_bytes + 112) // 128),
                         "line_requests_per_s": n_peer * (-(-(row_bytes + 112) // 128)) / (ms * 1e-3)},
                "host": {"rows": n_host, "bytes": b_host, "bytes_per_row": row_bytes, "peak_gbs": host_peak,
                         "t_ms": t["host"] * 1e3}},
            "traffic": per_row * rows if (per_row and bound == "hbm") else None}


def main_ours(args):
    import torch
    import torch.distributed as dist
    pkg = importlib.import_module("dist-gpu-sampling_b200")

    env = Env()
    env.world = world = int(os.environ.get("WORLD_SIZE", "1"))
    env.rank = rank = int(os.environ.get("RANK", "0"))
    env.local_rank = local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path")
    torch.cuda.set_device(local_rank)
    env.dev = dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    pkg.load_ops()
    if world > 1:
        pkg.create_dgs_communicator(world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    env.barrier = barrier
    env.clocks = None
    peaks = measure_link_peaks(env)
    torch.manual_seed(1234 + rank)

    w = workload(args.workload, args)
    want_cpu = rank == 0 and not args.no_cpu_baseline and world == 1 and args.workload in ("products", "small") \
        and not args.weighted
    wl = setup_workload(env, args, w, want_cpu)
    if rank == 0:
        env.clocks = ClockSampler(local_rank)
        env.clocks.start()
    res = measure_workload(env, args, pkg, wl, args.steps, args.warmup, full=True)
    clock_info = env.clocks.stop(*res["clock_window"]) if rank == 0 else None
    env.clocks = None
    red = reduce_over_ranks(env, res)
    host_graph, batches_np, n_edges_graph = wl.host_graph, wl.batches_np, wl.n_edges_graph
    teardown_workload(env, wl)
    del wl

    # ---- the Papers100M-shaped configuration, briefly, in the same run ----
    extra = None
    if args.workload == "products" and not args.no_extra_configs and not args.weighted and args.scale <= 0:
        w2 = workload("papers100m", args)
        wl2 = setup_workload(env, args, w2, False)
        res2 = measure_workload(env, args, pkg, wl2, args.extra_steps, 5, full=False)
        red2 = reduce_over_ranks(env, res2)
        extra = (w2, wl2.n_edges_graph, res2, red2)
        teardown_workload(env, wl2)
        del wl2

    if rank == 0:
        hbm_peak, hbm_kind = measured_peak_gbs()
        fanouts, dim = w["fanouts"], w["dim"]
        H = len(fanouts)

        def rate(r, name):
            return r[name]["edges_all"] / (r[name]["ms"] * 1e-3) if r.get(name) and r[name].get("ms") else None

        def entry(r, name, steps):
            if not r.get(name) or not r[name].get("ms"):
                return None
            label = API_NAMES[name] % args.depth if name == "pipeline" else API_NAMES[name]
            return {"api": label, "value": rate(r, name), "unit": "edges/s", "ms_per_step": r[name]["ms"] / steps}
        main = args.api
        others = [entry(red, n, args.steps) for n in ("pipeline", "blocks", "per-hop") if n != main]
        launches_step = {"pipeline": LAUNCHES_STEP_FUSED + H * LAUNCHES_HOP_FUSED + LAUNCHES_GATHER,
                         "blocks": LAUNCHES_STEP_FUSED + H * LAUNCHES_HOP_FUSED + LAUNCHES_GATHER,
                         "per-hop": H * (LAUNCHES_SAMPLE + LAUNCHES_RELABEL) + LAUNCHES_GATHER}[main]
        bl = red["blocks"]
        line = {
            "library": "dist-gpu-sampling_b200/lib/libdgs.so",
            "metric": "sampled_edges_per_s", "value": rate(red, main), "unit": "edges/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": red[main]["ms"] / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64",
            "data": "synthetic", "config": config_dict(args, w, n_edges_graph, world),
            "api": API_NAMES[main] % args.depth if main == "pipeline" else API_NAMES[main],
            "other_api": [o for o in others if o],
            "breakdown": {"of": "the one-batch-at-a-time `blocks` pass (in the pipeline the phases of different "
                                "batches overlap and cannot be told apart by stream events)",
                          "sample_relabel_ms_per_step": bl["sample_ms"] / args.steps,
                          "gather_ms_per_step": bl["gather_ms"] / args.steps,
                          "sampling_only_edges_per_s": bl["edges_all"] / (bl["sample_ms"] * 1e-3),
                          "edges_per_step_per_rank": res["pipeline"]["edges"] / args.steps,
                          "input_nodes_per_step_per_rank": res["pipeline"]["rows"] / args.steps,
                          "gather_payload_gbs_all_ranks": bl["rows_all"] * dim * 4 / (bl["gather_ms"] * 1e-3) / 1e9,
                          "gather_class_share": res["class_share"]},
            "e2e": {"value": red["e2e"]["edges_all"] / (red["e2e"]["ms"] * 1e-3), "unit": "edges/s",
                    "h2d_bytes_per_step": args.batch * 8, "d2h_bytes_per_step": res["e2e"]["d2h_bytes_per_step"],
                    "result_left_on_device": True,
                    "what": "pipeline; every batch's seeds copied from pinned host memory; a checksum of the last "
                            "1 024 gathered feature rows and input nodes plus the sizes read back every step; the "
                            "consumer (checksum kernels, copies) runs on a %s-priority stream"
                            % args.consumer_stream},
            "e2e_full_d2h": {"value": red["e2e_full"]["edges_all"] / (red["e2e_full"]["ms"] * 1e-3), "unit": "edges/s",
                             "ms_per_step": red["e2e_full"]["ms"] / args.steps,
                             "h2d_bytes_per_step": args.batch * 8,
                             "d2h_bytes_per_step": res["e2e_full"]["d2h_bytes_per_step"],
                             "d2h_gbs_per_rank": res["e2e_full"]["d2h_bytes_per_step"] * args.steps / (red["e2e_full"]["ms"] * 1e-3) / 1e9,
                             "host_link_peak_gbs": peaks.get("host_gbs"),
                             "what": "as e2e, but input nodes, every block's COO and the gathered features are copied "
                                     "to pinned host buffers every step (bound by the host link)"},
            "gpu_launches": args.steps * launches_step,
            "roofline": roofline_dict(res, w, peaks, hbm_peak, hbm_kind),
            "link_peaks": peaks,
            "verified": red["verified_all"] and res.get("verified", {}).get("ok", False),
            "verification": res.get("verified"),
            "clocks": clock_info,
        }
        if extra is not None:
            w2, ne2, res2, red2 = extra
            v2 = rate(red2, "pipeline")
            rf2 = roofline_dict(res2, w2, peaks, hbm_peak, hbm_kind)
            line["configs"] = {"papers100m": {
                "config": config_dict(args, w2, ne2, world), "api": API_NAMES["pipeline"] % args.depth,
                "value": v2, "unit": "edges/s", "steps": args.extra_steps, "ms_per_step": red2["pipeline"]["ms"] / args.extra_steps,
                "edges_per_s_per_gpu": v2 / world, "target_edges_per_s_per_gpu": 1e9,
                "meets_target": bool(v2 / world >= 1e9),
                "blocks_api": entry(red2, "blocks", args.extra_steps),
                "e2e": {"value": red2["e2e"]["edges_all"] / (red2["e2e"]["ms"] * 1e-3), "unit": "edges/s"},
                "edges_per_step_per_rank": res2["pipeline"]["edges"] / args.extra_steps,
                "input_nodes_per_step_per_rank": res2["pipeline"]["rows"] / args.extra_steps,
                "gather_roofline": {k: rf2[k] for k in ("bound", "achieved", "peak", "frac", "t_min_over_t",
                                                        "rows_per_launch", "ms_per_launch")}}}
        if host_graph is not None:
            v, ms, done, threads = run_cpu(fanouts, host_graph[0], host_graph[1], host_graph[2], batches_np,
                                           steps=10 ** 6, warmup=1, budget_s=args.cpu_seconds)
            line["cpu_baseline"] = {"value": v, "unit": "edges/s", "cores": threads, "kind": "port",
                                    "sample": "%d batches of %d seeds in %.1f s (same graph and step)"
                                              % (done, args.batch, done * ms / 1e3)}
        else:
            line["cpu_baseline"] = None
        del host_graph
        if world == 1 and not args.no_ref_gpu and not args.weighted and args.workload in ("products", "small"):
            torch.cuda.empty_cache()
            line["ref_gpu_baseline"] = run_ref_gpu(args, min(args.steps, 200))
        else:
            line["ref_gpu_baseline"] = {"unavailable": "measured at --gpus 1 on the products / small workloads only"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.ref_gpu_worker:
        main_ref_gpu_worker(a)
    elif a.impl == "reference":
        main_reference(a)
    else:
        main_ours(a)
