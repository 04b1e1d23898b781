"""In-tree build of the two shared libraries.

  lib/libdgs_b200.so  C ABI (include/dgs_b200.h): sm_100a kernels + HMGStore + NCCL bootstrap
  lib/libdgs.so       PyTorch custom-class / operator layer on top of it

Plain nvcc / g++ command lines, no build system.  nvcc cross-compiles for
sm_100a without a GPU; the built files stay in the tree (git-ignored) so that
they travel with a snapshot of the repository.
"""
import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
OBJ = os.path.join(PKG, "build")

ABI_SOURCES = [
    "kernels/gather.cu",
    "kernels/split.cu",
    "kernels/sample.cu",
    "kernels/relabel.cu",
    "kernels/blocks.cu",
    "host/error.cc",
    "host/comm.cc",
    "host/store.cc",
]
HEADERS = [
    "kernels/common.cuh",
    "kernels/philox.cuh",
    "kernels/tile_scan.cuh",
    "kernels/launchers.h",
    "kernels/relabel_device.cuh",
    "host/comm.h",
    "../../include/dgs_b200.h",
]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0 or verbose:
        sys.stdout.write(r.stdout)
    if r.returncode != 0:
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return r.stdout


def abi_path():
    return os.path.join(LIB, "libdgs_b200.so")


def binding_path():
    return os.path.join(LIB, "libdgs.so")


def build_abi(force=False, verbose=False, ptxas_info=False):
    """nvcc -> lib/libdgs_b200.so (rebuilds only the objects whose inputs changed)."""
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    objs, relink, log = [], force or not os.path.exists(abi_path()), ""
    for rel in ABI_SOURCES:
        src = os.path.join(CSRC, rel)
        obj = os.path.join(OBJ, rel.replace("/", "_") + ".o")
        stamp = obj + ".sha"
        dig = _digest([src] + headers, " ".join(flags))
        old = open(stamp).read() if os.path.exists(stamp) else ""
        if force or ptxas_info or old != dig or not os.path.exists(obj):
            cmd = [_nvcc()] + flags + ["-x", "cu", "-c", src, "-o", obj]
            log += _run(cmd, verbose)
            with open(stamp, "w") as f:
                f.write(dig)
            relink = True
        objs.append(obj)
    if relink:
        cmd = [_nvcc(), "-shared", "-cudart", "shared", "-o", abi_path()] + objs + [
            "-ldl", "-Xlinker", "-rpath", "-Xlinker", "/usr/local/cuda/lib64"]
        log += _run(cmd, verbose)
    return log


def build_binding(force=False, verbose=False):
    """g++ -> lib/libdgs.so (the TORCH_LIBRARY layer); needs lib/libdgs_b200.so."""
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "binding", "ops.cc")
    hdrs = [os.path.join(ROOT, "include", "dgs_b200.h")] + \
        [os.path.join(CSRC, "binding", h) for h in ("chunk_tensor.h", "host_words.h", "pipeline.h")]
    out = binding_path()
    stamp = out + ".sha"
    dig = _digest([src] + hdrs, torch.__version__)
    if not force and os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == dig:
        return ""
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    incs = []
    for p in cpp_extension.include_paths(device_type="cuda") if "device_type" in \
            cpp_extension.include_paths.__code__.co_varnames else cpp_extension.include_paths(cuda=True):
        incs += ["-isystem", p]
    cuda_inc = "/usr/local/cuda/include"
    if os.path.isdir(cuda_inc):
        incs += ["-isystem", cuda_inc]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi,
           "-Wno-deprecated-declarations"] + incs + [src, "-o", out,
           "-L" + LIB, "-ldgs_b200", "-L" + tlib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
           "-lc10_cuda", "-L/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib, "-Wl,-rpath,/usr/local/cuda/lib64"]
    log = _run(cmd, verbose)
    with open(stamp, "w") as f:
        f.write(dig)
    return log


def build_all(force=False, verbose=False):
    log = build_abi(force=force, verbose=verbose)
    log += build_binding(force=force or bool(log), verbose=verbose)
    return log


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built", abi_path(), binding_path())
