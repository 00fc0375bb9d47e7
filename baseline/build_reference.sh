#!/bin/bash
# Builds the reference's own Op benchmarks, UNMODIFIED, for the B200 (plain sm_100) into baseline/_ref/bin.
#
#   baseline/build_reference.sh [REFERENCE_TREE] [BUILD_DIR]
#
# The reference is a CMake C++/CUDA project.  Its top-level CMakeLists.txt requires FFmpeg development packages
# through pkg-config even when only the Op library and the benches are built (those do not use FFmpeg), so the
# configure step is given placeholder .pc files for the four FFmpeg modules; nothing that is built links them.
# An `a`-suffixed architecture would need CUDA >= 13.1 (its own gate); plain `100` needs CUDA >= 12.0.
# Every source file comes from the reference tree as it is; only the build directory and baseline/_ref are written.
set -euo pipefail
REF=${1:-/root/reference}
BUILD=${2:-/tmp/ninfer_ref_build}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT="$HERE/_ref"
PC="$BUILD/placeholder_pc"
mkdir -p "$PC" "$OUT/bin"
for mod in libavformat:61.1.100 libavcodec:61.3.100 libavutil:59.8.100 libswscale:8.1.100; do
  name=${mod%%:*}; ver=${mod##*:}
  printf 'Name: %s\nDescription: placeholder so that configure passes; nothing that is built uses it\nVersion: %s\nLibs:\nCflags:\n' \
    "$name" "$ver" > "$PC/$name.pc"
done
PKG_CONFIG_PATH="$PC" cmake -S "$REF" -B "$BUILD" -G Ninja -DCMAKE_BUILD_TYPE=Release -DNINFER_BUILD_APPS=OFF \
  -DNINFER_BUILD_BENCHMARKS=ON -DBUILD_TESTING=OFF -DCMAKE_CUDA_ARCHITECTURES=100 \
  -DCMAKE_CUDA_COMPILER="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
TARGETS="ninfer_linear_bench ninfer_bf16_linear_add_bench ninfer_fp8_linear_add_bench ninfer_fp8_linear_swiglu_bench \
ninfer_attn_input_proj_bench ninfer_gdn_input_proj_bench ninfer_gated_delta_net_bench ninfer_causal_conv1d_silu_bench \
ninfer_causal_softmax_attention_bench ninfer_rmsnorm_bench ninfer_argmax_bench ninfer_sparse_moe_bench"
ninja -C "$BUILD" -k 0 ${JOBS:+-j$JOBS} $TARGETS || true
for t in $TARGETS; do
  if [ -x "$BUILD/bench/$t" ]; then cp "$BUILD/bench/$t" "$OUT/bin/"; else echo "not built: $t" >&2; fi
done
ls -la "$OUT/bin"
