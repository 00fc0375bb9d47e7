// Weight-streaming linear layers over groupwise-integer weights, read straight from the artifact's row-split planes
// (no decode to bf16 first): Q4 / Q5 / Q6 with 64-value groups and W8 with 32-value groups, fp16 group scales.
//
// Same operator family as the reference's groupwise-int row-split kernels (src/ops/linear/{q4,q5,q6,w8}_*: gemv,
// small_t_mma, rowsplit_gemm_mma), its linear_add over those formats and its linear_pair
// (src/ops/linear_pair/w8/*: two projections of one input in one launch).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace nfb {

enum GroupIntFormat : int { kQ4G64 = 0, kQ5G64 = 1, kQ6G64 = 2, kW8G32 = 3 };

struct GroupIntWeight {
  const uint8_t* base = nullptr;   // Q4/5/6: [N, Kp / 2] low nibbles, k even in bits 0-3; W8: [N, Kp] int8
  const uint8_t* high = nullptr;   // Q5: [N, Kp / 8], Q6: [N, Kp / 4]; bit (k * hb + j) of a row is bit 4 + j of code k
  const __half* scale = nullptr;   // [N, Kp / group]
  int N = 0;                       // rows (a multiple of 16)
  __nv_bfloat16* out = nullptr;    // [T, N] with leading dimension ldo
  int64_t ldo = 0;
};

struct GroupIntLinearParams {
  int T = 0;                       // tokens, 1 .. 32 per launch
  int K = 0;                       // logical reduction length (a multiple of 64)
  int Kp = 0;                      // K rounded up to 128 (row pitch of the planes, in codes)
  int fmt = 0;                     // GroupIntFormat
  int n_weights = 1;               // 1, or 2 for a pair (both read the same x)
  GroupIntWeight w[2];
  const __nv_bfloat16* x = nullptr;      // [T, K] with leading dimension ldx (multiple of 8 elements, 16-byte aligned)
  int64_t ldx = 0;
  const __nv_bfloat16* resid = nullptr;  // optional [T, N] added to out of weight 0 (may alias out)
  int64_t ldr = 0;
  int* status = nullptr;                 // optional device status word: a bounded wait that ran out is recorded here
};

// out[t, n] = sum_k x[t, k] * code[n, k] * scale[n, k / group] (+ resid[t, n]); fp32 accumulation, group sums of the
// exact integer codes scaled in fp32.  Returns nullptr or a static error string.
const char* groupint_linear(const GroupIntLinearParams& p, cudaStream_t stream);

}  // namespace nfb
