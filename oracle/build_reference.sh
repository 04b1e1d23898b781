#!/bin/bash
# Builds the reference's own CUDA library for sm_100a into oracle/_ref/libdgs_reference.so
# (test infrastructure: used only to generate golden vectors and same-box comparison timings).
#
# The reference sources are compiled from a scratch copy under /tmp -- nothing from them is
# written into this repository -- with the three build-only fixes its 2022-era sources need
# with CUDA 12.9 / torch 2.11:
#   1. -std=c++17 and `-include thrust/execution_policy.h` (the sampling files use thrust::device
#      without including it);
#   2. const_cast in _getTensorVoidDataPtr (storage().data() is const void* now);
#   3. `&cuda::X` -> `&dgs::cuda::X` in pybind.cc (ambiguous with libcu++'s ::cuda).
# Its own build system (cmake) is not used.  Needs libtorch and NCCL headers; ~2 min per file.
# Usage: build_reference.sh <checkout of gpzlx1/Dist-GPU-sampling>   (or DGS_REFERENCE_DIR in the environment)
set -e
REF=${1:-$DGS_REFERENCE_DIR}
if [ -z "$REF" ] || [ ! -d "$REF/src/cuda" ]; then
  echo "usage: $0 <reference checkout> (no src/cuda under '$REF')" >&2
  exit 2
fi
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
WORK=$(mktemp -d /tmp/dgs_ref_build.XXXXXX)
T=$(python -c 'import torch,os;print(os.path.dirname(torch.__file__))')
PYINC=$(python -c 'import sysconfig;print(sysconfig.get_paths()["include"])')
ABI=$(python -c 'import torch;print(int(torch._C._GLIBCXX_USE_CXX11_ABI))')
mkdir -p "$OUT"
cp -r "$REF/src" "$WORK/src"
sed -i 's/return data.storage().data();/return const_cast<void*>(data.storage().data());/' "$WORK/src/chunk_tensor.cc"
sed -i 's/&cuda::/\&dgs::cuda::/g' "$WORK/src/pybind.cc"
INC="-I$T/include -I$T/include/torch/csrc/api/include -I$PYINC -I/usr/local/cuda/include"
DEF="-D_GLIBCXX_USE_CXX11_ABI=$ABI"
OBJS=""
build_one() {
  f=$1; o=$WORK/$(echo "$f" | tr '/' '_').o
  case "$f" in
    *.cu) nvcc -std=c++17 -O2 --expt-extended-lambda --expt-relaxed-constexpr -gencode arch=compute_100a,code=sm_100a \
            -Xcompiler -fPIC $DEF $INC -include thrust/execution_policy.h -w -c "$WORK/$f" -o "$o" ;;
    *.cc) nvcc -std=c++17 -O2 -x cu --expt-extended-lambda --expt-relaxed-constexpr -gencode arch=compute_100a,code=sm_100a \
            -Xcompiler -fPIC $DEF $INC -include thrust/execution_policy.h -w -c "$WORK/$f" -o "$o" ;;
  esac
}
FILES=$(cd "$WORK" && ls src/*.cc src/cuda/*.cu)
JOBS=${JOBS:-4}
for f in $FILES; do
  build_one "$f" &
  while [ "$(jobs -r | wc -l)" -ge "$JOBS" ]; do sleep 1; done
done
wait
for f in $FILES; do OBJS="$OBJS $WORK/$(echo "$f" | tr '/' '_').o"; done
nvcc -shared -o "$OUT/libdgs_reference.so" $OBJS -L"$T/lib" -ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -lnccl \
     -Xlinker -rpath -Xlinker "$T/lib"
rm -rf "$WORK"
echo "built $OUT/libdgs_reference.so"
