#!/bin/sh
# Builds liblpp_b200.so (sm_100a only) next to the Python package.  nvcc cross-compiles without a GPU.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/../liblpp_b200.so"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 \
    -ccbin "${HOSTCXX:-g++}" --shared -Xcompiler -fPIC -Xptxas -v \
    -o "$OUT" "$HERE/engine.cu" "$HERE/ops_api.cu" -ldl "$@"
echo "built $OUT"
