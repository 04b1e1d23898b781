"""The index micro-benchmark tool (dist-gpu-sampling_b200/index_microbench.py, the rebuilt
python/compute_loading_factor.py of the reference) on a tiny table: it must run, verify every gathered row
against the generator, and print one well-formed JSON object per case."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "dist-gpu-sampling_b200", "index_microbench.py")


@pytest.mark.parametrize("dist,misalign", [("uniform", 0), ("zipf", 4)])
def test_index_microbench_runs_and_verifies(dist, misalign):
    cmd = [sys.executable, TOOL, "--rows", "200000", "--dim", "100", "--ids", "1000,50000", "--host-frac", "0.2",
           "--dist", dist, "--misalign", str(misalign), "--iters", "3", "--warmup", "1", "--hbm-peak", "6544"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:]
    lines = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    cases = {(ln["case"], ln["ids"]) for ln in lines}
    for n in (1000, 50000):
        for case in ("index (mixed)", "local_index", "host_index"):       # one GPU: no remote class
            assert (case, n) in cases, (case, n, r.stdout[-2000:])
    for ln in lines:
        assert ln["verified"] is True, ln
        assert ln["dim"] == 100 and ln["dist"] == dist and ln["world"] == 1 and ln["ms"] > 0
        assert ln["payload_gbs"] > 0 and ln["algorithmic_gbs"] > ln["payload_gbs"]
        if ln["case"] == "index (mixed)":
            cs = ln["class_sizes"]
            assert cs["local"] + cs["remote"] + cs["host"] == ln["ids"] and cs["remote"] == 0 and cs["host"] > 0
            assert ln["split_index_ms"] > 0
        else:
            assert ln["bound"] in ("hbm", "host link") and ln["peak_gbs"] > 0 and 0 < ln["frac"] < 2
