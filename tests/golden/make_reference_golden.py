"""Golden vectors from the reference's OWN kernels, run on a GPU.

The reference (gpzlx1/Dist-GPU-sampling) has no CPU implementation, so its
deterministic outputs can only be recorded on a GPU box.  This script loads the
library built by oracle/build_reference.sh (oracle/_ref/libdgs_reference.so --
the reference's unmodified kernels compiled for sm_100a), runs every operator on
small seeded inputs whose result does not depend on random numbers, and writes
the file given as its argument (default: reference_b200.json beside this script).

It must run in a process of its own: the reference and this repository register
the same torch class and operator names.

    python tests/golden/make_reference_golden.py [output.json]

What is recorded: placement views (the README demo and a 2-D table with a host
tail), _CAPI_index / split_index / local / host index, tensor_relabel (int64 and
int32), sampling outputs for graphs where every row has deg <= fan-out (fully
deterministic), per-seed grouping (coo_row) for mixed-degree graphs with and
without replacement, and the cache operators.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIB = os.path.join(ROOT, "oracle", "_ref", "libdgs_reference.so")


def main():
    torch.ops.load_library(LIB)
    torch.cuda.set_device(0)
    ops = torch.ops.dgs_ops
    ops._CAPI_set_nccl(1, ops._CAPI_get_unique_id(), 0)      # the constructor reads the communicator's size
    CT = torch.classes.dgs_classes.ChunkTensor
    rng = np.random.default_rng(20260101)
    out = {"source": "reference kernels (src/cuda/*.cu, src/chunk_tensor.cc) compiled for sm_100a, run on "
                     + torch.cuda.get_device_name(0)}

    def dev(a, dt=torch.int64):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dt).cuda()

    # ---- README demo (example/demo.py) ----
    c = CT([100], torch.int64, 200)
    c._CAPI_load_from_tensor(torch.arange(100))
    out["demo"] = {"host": c._CAPI_get_host_tensor().tolist(), "device": c._CAPI_get_sub_device_tensor().tolist(),
                   "allocated": int(ops._CAPI_get_current_allocated())}
    del c

    # ---- 2-D table, capacity not row aligned: one row straddles the device/host boundary ----
    rows, D = 60, 6
    table = rng.integers(-1000, 1000, size=(rows, D)).astype(np.int32)
    cap = 4 * (D * 37 + 2)
    c = CT([rows, D], torch.int32, cap)
    c._CAPI_load_from_tensor(torch.from_numpy(table))
    idx = rng.integers(0, rows, size=48).astype(np.int64)
    lo, re, ho = c._CAPI_split_index(dev(idx))
    out["table"] = {"table": table.tolist(), "capacity_per_gpu": cap, "idx": idx.tolist(),
                    "host_view": c._CAPI_get_host_tensor().tolist(),
                    "device_view": c._CAPI_get_sub_device_tensor().tolist(),
                    "index": c._CAPI_index(dev(idx)).tolist(),
                    "index_i32": c._CAPI_index(dev(idx, torch.int32)).tolist(),
                    "split": [lo.tolist(), re.tolist(), ho.tolist()],
                    # rows wholly inside their class (the unchecked accessors read past the chunk otherwise)
                    "local_ids": [int(x) for x in lo.tolist() if (x + 1) * D <= cap // 4],
                    "host_ids": [int(x) for x in ho.tolist() if x * D >= cap // 4]}
    t = out["table"]
    t["local_index"] = c._CAPI_local_index(dev(np.array(t["local_ids"], dtype=np.int64))).tolist()
    t["host_index"] = c._CAPI_host_index(dev(np.array(t["host_ids"], dtype=np.int64))).tolist()
    feats = rng.standard_normal((40, 5)).astype(np.float32)
    cf = CT([40, 5], torch.float32, 4 * 5 * 40)
    cf._CAPI_load_from_tensor(torch.from_numpy(feats))
    fidx = rng.integers(0, 40, size=30)
    out["float_table"] = {"table_bits": feats.view(np.int32).tolist(), "idx": fidx.tolist(),
                          "index_bits": cf._CAPI_index(dev(fidx)).cpu().numpy().view(np.int32).tolist()}
    del c, cf

    # ---- relabel ----
    seeds = rng.permutation(500)[:40]
    col = rng.integers(0, 500, size=400)
    row = np.repeat(seeds, 10)
    for name, dt in (("relabel_i64", torch.int64), ("relabel_i32", torch.int32)):
        f, (r, cc) = ops._CAPI_tensor_relabel([dev(seeds, dt), dev(col, dt)], [dev(row, dt), dev(col, dt)])
        out[name] = {"seeds": seeds.tolist(), "col": col.tolist(), "frontier": f.tolist(), "row_out": r.tolist(),
                     "col_out": cc.tolist()}
    q = rng.integers(0, 700, size=50)
    f, (qq,) = ops._CAPI_tensor_relabel([dev(seeds)], [dev(q)])
    out["relabel_absent"] = {"mapping": seeds.tolist(), "query": q.tolist(), "frontier": f.tolist(), "out": qq.tolist()}

    # ---- sampling: every row has deg <= k -> fully deterministic ----
    deg = rng.integers(0, 7, size=50)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, 50, size=int(indptr[-1])).astype(np.int64)
    probs = (rng.random(indices.size) + 0.1).astype(np.float32)
    sd = rng.permutation(50)[:30].astype(np.int64)
    g = {"indptr": indptr.tolist(), "indices": indices.tolist(), "probs_bits": probs.view(np.int32).tolist(),
         "seeds": sd.tolist(), "k": 6}
    ip, ix, pr, s_ = dev(indptr), dev(indices), torch.from_numpy(probs).cuda(), dev(sd)
    c_ip = CT([indptr.size], torch.int64, 8 * 20)
    c_ix = CT([indices.size], torch.int64, 8 * 50)
    c_pr = CT([indices.size], torch.float32, 4 * 64)
    c_ip._CAPI_load_from_tensor(torch.from_numpy(indptr))
    c_ix._CAPI_load_from_tensor(torch.from_numpy(indices))
    c_pr._CAPI_load_from_tensor(torch.from_numpy(probs))
    for name, fn in (("plain", lambda: ops._CAPI_sample_neighbors(s_, ip, ix, 6, False)),
                     ("chunk", lambda: ops._CAPI_sample_neighbors_with_chunk_tensor(s_, c_ip, c_ix, 6, False)),
                     ("probs", lambda: ops._CAPI_sample_neighbors_with_probs(s_, ip, ix, pr, 6, False)),
                     ("probs_chunk", lambda: ops._CAPI_sample_neighbors_with_probs_with_chunk_tensor(
                         s_, c_ip, c_ix, c_pr, 6, False))):
        r, cc = fn()
        g[name] = {"coo_row": r.tolist(), "coo_col": cc.tolist()}
    out["full_rows"] = g

    # ---- sampling: mixed degrees -> the grouping (coo_row) is deterministic, the picks are not ----
    deg = rng.integers(0, 40, size=60)
    indptr2 = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices2 = rng.integers(0, 60, size=int(indptr2[-1])).astype(np.int64)
    probs2 = (rng.random(indices2.size) + 0.1).astype(np.float32)
    sd2 = rng.integers(0, 60, size=80).astype(np.int64)
    m = {"indptr": indptr2.tolist(), "seeds": sd2.tolist(), "k": 8}
    ip2, ix2, pr2, s2 = dev(indptr2), dev(indices2), torch.from_numpy(probs2).cuda(), dev(sd2)
    for name, fn in (("uniform", lambda rep: ops._CAPI_sample_neighbors(s2, ip2, ix2, 8, rep)),
                     ("weighted", lambda rep: ops._CAPI_sample_neighbors_with_probs(s2, ip2, ix2, pr2, 8, rep))):
        for rep in (False, True):
            r, cc = fn(rep)
            m["%s_replace%d_coo_row" % (name, int(rep))] = r.tolist()
            # validity of the reference's own picks: every (seed, col) is an edge
            rr, c2 = r.cpu().numpy(), cc.cpu().numpy()
            ok = all(c2[i] in indices2[indptr2[rr[i]]:indptr2[rr[i] + 1]] for i in range(rr.size))
            m["%s_replace%d_valid" % (name, int(rep))] = bool(ok)
    out["mixed_rows"] = m

    # ---- cache operators ----
    n, Dc = 80, 4
    cpu = rng.standard_normal((n, Dc)).astype(np.float32)
    hot = rng.permutation(n)[:24]
    gpu = (cpu[hot] + 100.0).astype(np.float32)
    nid = rng.integers(0, n, size=60)
    hk, hv = ops._CAPI_create_hash_map(dev(hot), dev(np.arange(24)))
    cpu_t = torch.from_numpy(cpu).pin_memory()
    fetched = ops._CAPI_fetch_data(cpu_t, torch.from_numpy(gpu).cuda(), dev(nid), hk, hv)
    out["cache"] = {"cpu_bits": cpu.view(np.int32).tolist(), "hot": hot.tolist(), "gpu_bits": gpu.view(np.int32).tolist(),
                    "nid": nid.tolist(), "table_slots": int(hk.numel()),
                    "fetched_bits": fetched.cpu().numpy().view(np.int32).tolist()}
    torch.cuda.synchronize()
    del c_ip, c_ix, c_pr
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_b200.json")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump(out, f)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
