"""Builds the reference's own CUDA kernels for sm_100a into oracle/_ref/ (build_reference.sh).

TEST INFRASTRUCTURE ONLY, like everything under oracle/: the resulting library produces the golden vectors
(tests/golden/make_reference_golden.py) and the same-box "reference kernels on this GPU" timing of bench.py's
baseline leg.  The product package never loads it.

The reference checkout is named by the caller or by DGS_REFERENCE_DIR; when neither is given, a directory
called `reference` next to this repository is used if it holds the sources.  Nothing is built when the
sources are absent or the library exists already.
"""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(_HERE, "_ref", "libdgs_reference.so")


def find_sources(ref_dir=None):
    root = os.path.dirname(_HERE)
    for cand in (ref_dir, os.environ.get("DGS_REFERENCE_DIR"), os.path.join(os.path.dirname(root), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src", "cuda")):
            return cand
    return None


def build_if_sources_present(ref_dir=None, quiet=True):
    """Returns the library path if it exists afterwards, else None.  About five minutes of nvcc, once."""
    if os.path.exists(LIBRARY):
        return LIBRARY
    if os.environ.get("DGS_SKIP_REFERENCE_BUILD") == "1":
        return None
    src = find_sources(ref_dir)
    if src is None:
        return None
    out = subprocess.DEVNULL if quiet else None
    subprocess.run(["bash", os.path.join(_HERE, "build_reference.sh"), src], check=False, stdout=out, stderr=out)
    return LIBRARY if os.path.exists(LIBRARY) else None
