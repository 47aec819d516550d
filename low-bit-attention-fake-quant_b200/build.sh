#!/usr/bin/env bash
# Builds liblbfq.so (sm_100a) next to this script. nvcc cross-compiles without a GPU.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
FLAGS=(-gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 --expt-relaxed-constexpr
       -Xcompiler -fPIC -I"$here/../include" ${LBFQ_NVCC_EXTRA:-})
mkdir -p "$here/build"
objs=()
for f in api quant preprocess prep_fused qm_corr_tc kmeans kmeans_tc attention attention_fast; do
  src="$here/csrc/$f.cu"; obj="$here/build/$f.o"
  if [[ ! -f "$obj" || "$src" -nt "$obj" || "$here/csrc/common.cuh" -nt "$obj" || "$here/csrc/attn_prims.cuh" -nt "$obj" || "$here/csrc/tile_ops.cuh" -nt "$obj" || "$here/csrc/kmeans_tc.h" -nt "$obj" || "$here/csrc/qm_corr_tc.h" -nt "$obj" || "$here/../include/lbfq.h" -nt "$obj" ]]; then
    "$NVCC" "${FLAGS[@]}" -c "$src" -o "$obj" &
  fi
  objs+=("$obj")
done
wait
"$NVCC" -shared -o "$here/liblbfq.so" "${objs[@]}" -lcudart
echo "built $here/liblbfq.so"
