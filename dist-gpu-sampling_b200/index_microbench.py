"""ChunkTensor index micro-benchmark: GB/s per location class.

The tool the reference ships as python/compute_loading_factor.py (written
against a constructor that no longer exists there), rebuilt on the real
operator API: one [rows, dim] fp32 table split over the GPUs of the node plus
an optional pinned host tail; random row ids are split with _CAPI_split_index
and each class is gathered with _CAPI_local_index / _CAPI_remote_index /
_CAPI_host_index, plus the mixed _CAPI_index.  Instead of the reference's
assumed bandwidths (1300 / 260 / 31 GB/s, :110-122) every class is compared
with a bandwidth measured on the machine it runs on.

  python dist-gpu-sampling_b200/index_microbench.py --rows 4000000 --dim 128 --ids 1000000
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
      dist-gpu-sampling_b200/index_microbench.py --rows 8000000 --host-frac 0.2 \
      --ids 1000,16000,256000,1000000,4000000 --dist zipf

--ids takes a list (one query size after the other on the same table), --dist uniform|zipf|uniform,zipf picks
the id distribution (Zipf(1.1) ranks mapped to rows by a fixed permutation), --misalign B adds B bytes to the
capacity so that chunk boundaries fall inside rows (the straddle and off-grid paths of the gather).

The table is filled in place, chunk by chunk, with a hash of the flat element
index, so every gathered row can be verified without a second copy.
Prints one JSON object per measured case (rank 0).
"""
import argparse
import importlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4_000_000)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--ids", type=str, default="1000000",
                    help="row ids per query; a comma-separated list runs one query size after the other")
    ap.add_argument("--host-frac", type=float, default=0.0, help="fraction of rows kept in the host tail")
    ap.add_argument("--dist", default="uniform",
                    help="uniform | zipf | uniform,zipf (both, one after the other on the same table)")
    ap.add_argument("--id-window", type=int, default=0,
                    help="draw the ids from a window of this many rows at the start of the next rank's chunk "
                         "(all remote, one peer, limited address range); 0 = whole table")
    ap.add_argument("--misalign", type=int, default=0, help="extra bytes of capacity: rows straddle chunks")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--hbm-peak", type=float, default=0.0, help="GB/s; 0 = measure a device copy here")
    ap.add_argument("--nvlink-peak", type=float, default=770.0,
                    help="GB/s per direction the peer class is compared with (default: a measured peer copy on B200)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    pkg = importlib.import_module("dist-gpu-sampling_b200")
    synth = importlib.import_module("dist-gpu-sampling_b200.synth")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg.load_ops()
    if world > 1:
        pkg.create_dgs_communicator(world)

    D, rows = args.dim, args.rows
    gpu_rows = int(rows * (1.0 - args.host_frac))
    # whole rows per GPU, rounded DOWN: a capacity that covers the whole table makes the placement rule
    # (src/chunk_tensor.cc:57-68) recompute the chunk as ceil(elements / world), which cuts a row in two
    # whenever the row count does not divide evenly, and every later chunk then starts off the 16-byte grid
    cap = (gpu_rows // world) * D * 4 + args.misalign
    table = torch.classes.dgs_classes.ChunkTensor([rows, D], torch.float32, cap)
    sub = table._CAPI_get_sub_device_tensor()
    each = sub.numel()
    step = 1 << 26
    nofill = os.environ.get("DGS_MB_NOFILL") == "1"   # bandwidth-only runs on uninitialised data
    for lo in range(0, 0 if nofill else each, step):
        n = min(step, each - lo)
        sub[lo:lo + n] = synth.hashed_values(rank * each + lo, n, device=dev)
    host = table._CAPI_get_host_tensor()
    if rank == 0 and host.numel():
        thr = rows * D - host.numel()
        for lo in range(0, host.numel(), step):
            n = min(step, host.numel() - lo)
            host[lo:lo + n] = synth.hashed_values(thr + lo, n, device=dev).cpu()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()

    id_counts = [int(x) for x in str(args.ids).split(",")]
    dists = [d for d in str(args.dist).split(",") if d]
    for d in dists:
        if d not in ("uniform", "zipf"):
            raise SystemExit("--dist: uniform, zipf or uniform,zipf")
    hbm_cached = [args.hbm_peak]
    for d in dists:
        args.dist = d
        for n_ids in id_counts:
            run_query(args, n_ids, table, sub, host, each, world, rank, dev, synth, torch, hbm_cached)
    del table, sub, host
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_query(args, n_ids, table, sub, host, each, world, rank, dev, synth, torch, hbm_cached):
    D, rows = args.dim, args.rows
    g = torch.Generator(device=dev)
    g.manual_seed(100 + rank)
    if args.id_window > 0:
        per_gpu = each // D
        ids = torch.randint(0, min(args.id_window, per_gpu), (n_ids,), device=dev, generator=g) \
            + ((rank + 1) % world) * per_gpu
    elif args.dist == "uniform":
        ids = torch.randint(0, rows, (n_ids,), device=dev, generator=g)
    else:  # Zipf(1.1) ranks by inverse CDF, rank -> row through a fixed permutation
        u = torch.rand(n_ids, device=dev, generator=g, dtype=torch.float64)
        a = 1.1
        r = ((1.0 - u * (1.0 - float(rows) ** (1.0 - a))) ** (1.0 / (1.0 - a))).floor().clamp_(1, rows).long() - 1
        gp = torch.Generator(device=dev)
        gp.manual_seed(7)
        ids = torch.randperm(rows, device=dev, generator=gp)[r]

    def timed(fn, idx):
        for _ in range(args.warmup):
            out = fn(idx)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(args.iters + 1)]
        e[0].record()
        for i in range(args.iters):
            out = fn(idx)
            e[i + 1].record()
        torch.cuda.synchronize()
        ms = sorted(e[i].elapsed_time(e[i + 1]) for i in range(args.iters))
        return out, ms[len(ms) // 2]

    # measured denominators
    hbm = hbm_cached[0]
    if hbm <= 0:
        a_ = torch.empty(1 << 28, dtype=torch.float32, device=dev)
        b_ = torch.empty_like(a_)
        _, ms = timed(lambda _: b_.copy_(a_), None)
        hbm = 2 * a_.numel() * 4 / ms / 1e6
        hbm_cached[0] = hbm
        del a_, b_
    host_link = None
    if host.numel():
        src = torch.empty(1 << 26, dtype=torch.float32).pin_memory()
        dst = torch.empty(1 << 26, dtype=torch.float32, device=dev)
        _, ms = timed(lambda _: dst.copy_(src, non_blocking=True), None)
        host_link = src.numel() * 4 / ms / 1e6

    lo_ids, re_ids, ho_ids = table._CAPI_split_index(ids)
    _, split_ms = timed(table._CAPI_split_index, ids)

    def verify(out, idx):
        k = min(2048, idx.numel())
        if k == 0:
            return True
        for sel, got in ((idx[:k], out[:k]), (idx[-k:], out[-k:])):      # both ends of the result
            flat = (sel[:, None] * D + torch.arange(D, device=dev)[None, :]).reshape(-1)
            if not torch.equal(got, synth.hash_of_index(flat).reshape(k, D)):
                return False
        return True

    cases = [("index (mixed)", table._CAPI_index, ids, None),
             ("local_index", table._CAPI_local_index, lo_ids, hbm),
             ("remote_index", table._CAPI_remote_index, re_ids, args.nvlink_peak),
             ("host_index", table._CAPI_host_index, ho_ids, host_link)]
    solo = os.environ.get("DGS_MB_SOLO_RANK")       # only this rank issues requests, the others just serve
    for name, fn, idx, peak in cases:
        if idx.numel() == 0 or (solo is not None and int(solo) != rank):
            continue
        out, ms = timed(fn, idx)
        payload = idx.numel() * D * 4
        line = {"case": name, "rank": rank, "world": world, "ids": n_ids, "rows": idx.numel(), "dim": D, "dist": args.dist,
                "ms": ms, "payload_gbs": payload / ms / 1e6,
                "algorithmic_gbs": idx.numel() * (8 + 2 * D * 4) / ms / 1e6, "verified": verify(out, idx)}
        if name == "local_index":
            line.update(bound="hbm", peak_gbs=hbm, frac=line["algorithmic_gbs"] / hbm)
        elif peak:
            line.update(bound="nvlink" if name == "remote_index" else "host link", peak_gbs=peak,
                        frac=line["payload_gbs"] / peak)
        else:
            line.update(class_sizes={"local": lo_ids.numel(), "remote": re_ids.numel(), "host": ho_ids.numel()},
                        split_index_ms=split_ms)
        if rank == 0 or name != "index (mixed)":
            print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
