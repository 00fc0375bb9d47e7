// One executable for the reference's Op benchmarks.
//
// Each of the reference's bench/ops/*_bench.cu files has its own main() and links the whole Op library (several
// hundred MB of device code).  Twelve such executables do not fit a snapshot that travels to the GPU box, so the
// build script renames the `main` symbol of every compiled bench OBJECT (objcopy --redefine-sym, the sources stay
// untouched) and links them all, once, behind this dispatcher:
//
//     ninfer_ref_benches <bench name> [that bench's own arguments...]
//
// Nothing here measures anything: the timing loops, the L2 flush and the printed rows are the reference's.
#include <cstdio>
#include <cstring>

#define REF_BENCHES(X)                                                                                              \
  X(bf16_linear_add) X(fp8_linear_add) X(fp8_linear_swiglu) X(attn_input_proj) X(gdn_input_proj) X(gated_delta_net) \
  X(causal_conv1d_silu) X(causal_softmax_attention) X(rmsnorm) X(argmax) X(sparse_moe) X(linear)

#define DECLARE(name) extern "C" int ref_main_##name(int, char**);
REF_BENCHES(DECLARE)
#undef DECLARE

int main(int argc, char** argv) {
  if (argc >= 2) {
#define TRY(name) \
  if (std::strcmp(argv[1], #name) == 0) return ref_main_##name(argc - 1, argv + 1);
    REF_BENCHES(TRY)
#undef TRY
  }
  std::fprintf(stderr, "usage: %s <bench> [args...]\nbenches:", argv[0]);
#define LIST(name) std::fprintf(stderr, " " #name);
  REF_BENCHES(LIST)
#undef LIST
  std::fprintf(stderr, "\n");
  return 2;
}
