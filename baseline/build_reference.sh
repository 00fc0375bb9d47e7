#!/bin/bash
# Builds the reference's own Op benchmarks, from its UNMODIFIED sources, for the B200 (plain sm_100) into
# baseline/_ref/bin/ninfer_ref_benches (one executable, see ref_bench_mux.cpp).
#
#   baseline/build_reference.sh [REFERENCE_TREE] [BUILD_DIR]
#
# What this has to work around, none of it by touching a reference source file:
#  * The top-level CMakeLists.txt requires FFmpeg development packages through pkg-config even when only the Op
#    library and the benches are built (those do not use FFmpeg): configure gets placeholder .pc files.
#  * An `a`-suffixed architecture needs CUDA >= 13.1 there; plain `100` needs CUDA >= 12.0, which this image has.
#  * Two translation units (ops/launcher/gqa_attention_decode_i8.cu and ..._e8.cu: 1.7 GB of PTX for the first) keep
#    ptxas busy for hours; the object build is cut off after REF_BUILD_SECONDS and whatever compiled is used.
#  * The library's own device link fails for sm_100: "Entry function ... w8_rowsplit_medium_t_splitk_kernel ... uses
#    too much shared data (0xe800 bytes, 0xc000 max)" (same for w8_small_t_mma_kernel and nvfp4_w4a4_mma_kernel): those
#    kernels are sized for the reference's own GPU.  The W8 and NVFP4-W4A4 objects are therefore left out of the
#    device link, together with the attention variants the benches below do not call; symbols of left-out objects
#    stay unresolved (-Wl,--unresolved-symbols=ignore-all) and are only reachable through routes that are not run.
#  * Each bench has its own main() and would link the whole Op library (~740 MB each): the `main` symbol of every
#    compiled bench OBJECT is renamed (objcopy) and all of them are linked once behind ref_bench_mux.cpp.
set -euo pipefail
REF=${1:-${NINFER_REFERENCE_TREE:?give the reference source tree as the first argument or in NINFER_REFERENCE_TREE}}
BUILD=${2:-/tmp/ninfer_ref_build}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT="$HERE/_ref"
PC="$BUILD/placeholder_pc"
CUDA=${CUDA_HOME:-/usr/local/cuda}
mkdir -p "$PC" "$OUT/bin"
for mod in libavformat:61.1.100 libavcodec:61.3.100 libavutil:59.8.100 libswscale:8.1.100; do
  name=${mod%%:*}; ver=${mod##*:}
  printf 'Name: %s\nDescription: placeholder so that configure passes; nothing that is built uses it\nVersion: %s\nLibs:\nCflags:\n' \
    "$name" "$ver" > "$PC/$name.pc"
done
PKG_CONFIG_PATH="$PC" cmake -S "$REF" -B "$BUILD" -G Ninja -DCMAKE_BUILD_TYPE=Release -DNINFER_BUILD_APPS=OFF \
  -DNINFER_BUILD_BENCHMARKS=ON -DBUILD_TESTING=OFF -DCMAKE_CUDA_ARCHITECTURES=100 \
  -DCMAKE_CUDA_COMPILER="$CUDA/bin/nvcc"
BENCHES="bf16_linear_add fp8_linear_add fp8_linear_swiglu attn_input_proj gdn_input_proj gated_delta_net \
causal_conv1d_silu causal_softmax_attention rmsnorm argmax sparse_moe linear"
TARGETS=""
for b in $BENCHES; do TARGETS="$TARGETS ninfer_${b}_bench"; done
# objects only matter; the library / executable link steps of these targets are expected to fail (see above)
timeout "${REF_BUILD_SECONDS:-7200}" ninja -C "$BUILD" -k 0 ${JOBS:+-j$JOBS} $TARGETS || true

cd "$BUILD"
MUX="$BUILD/mux"
mkdir -p "$MUX"
EXCL='/w8/.*\.cu\.o|w4a4|gqa_attention_decode_e8|gqa_attention_decode_i8|gqa_attention_prefill|gqa_attention_decode_nvfp4|gqa_attention_decode_iso3|softmax_attention/dense'
OBJS=$(find src/CMakeFiles/ninfer_ops.dir -name "*.o" | grep -Ev "$EXCL" | sort | tr '\n' ' ')
BOBJS=""
for b in $BENCHES; do
  o=$(find "bench/CMakeFiles/ninfer_${b}_bench.dir" -name "*.o" | head -1)
  if [ -z "$o" ]; then echo "bench object missing: $b" >&2; exit 1; fi
  objcopy --redefine-sym main=ref_main_$b "$o" "$MUX/$b.o"
  BOBJS="$BOBJS $MUX/$b.o"
done
"$CUDA/bin/nvcc" -O3 -DNDEBUG "--generate-code=arch=compute_100,code=[compute_100,sm_100]" -Xcompiler=-fPIC \
  -Wno-deprecated-gpu-targets -shared -dlink $OBJS $BOBJS -o "$MUX/dlink.o" -L"$CUDA/targets/x86_64-linux/lib" \
  -lcudadevrt -lcudart_static
g++ -O2 -c "$HERE/ref_bench_mux.cpp" -o "$MUX/mux_main.o"
g++ -O3 "$MUX/mux_main.o" $BOBJS $OBJS "$MUX/dlink.o" -o "$OUT/bin/ninfer_ref_benches" \
  -Wl,--unresolved-symbols=ignore-all -L"$CUDA/targets/x86_64-linux/lib" \
  src/libninfer_artifact.a src/libninfer_nvfp4_tma.a src/libninfer_core.a "$CUDA/targets/x86_64-linux/lib/libcudart.so" \
  "$CUDA/targets/x86_64-linux/lib/stubs/libcuda.so" -ldl -lcudadevrt -lcudart_static -lrt -lpthread
strip "$OUT/bin/ninfer_ref_benches"
ls -la "$OUT/bin"
