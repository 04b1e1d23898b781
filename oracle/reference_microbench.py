"""Runs the index micro-benchmark against the reference's own kernels compiled for this GPU.

TEST INFRASTRUCTURE ONLY (like everything under oracle/): this process loads
oracle/_ref/libdgs_reference.so -- the reference's unmodified CUDA sources built by build_reference.sh --
instead of the product's operator library, and then drives the same tool
(dist-gpu-sampling_b200/index_microbench.py), which only speaks the operator API the two libraries share
(src/pybind.cc:11-38).  One GPU; same arguments as the tool:

    python oracle/reference_microbench.py --rows 4000000 --dim 128 --ids 1000000

The product package has no switch of this kind; the same-box comparison of the whole sampling step is
bench.py's `ref_gpu_baseline` leg.
"""
import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)


def main():
    import torch
    lib = os.path.join(HERE, "_ref", "libdgs_reference.so")
    if not os.path.exists(lib):
        raise SystemExit("no %s: build it with oracle/build_reference.sh <reference checkout>" % lib)
    torch.ops.load_library(lib)
    ops = torch.ops.dgs_ops
    ops._CAPI_set_nccl(1, ops._CAPI_get_unique_id(), 0)      # its ChunkTensor constructor reads the communicator
    pkg = importlib.import_module("dist-gpu-sampling_b200")
    pkg.load_ops = lambda: lib                               # the tool must not load the product's library on top
    tool = importlib.import_module("dist-gpu-sampling_b200.index_microbench")
    tool.main()


if __name__ == "__main__":
    main()
