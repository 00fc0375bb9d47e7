// Block Hadamard rotation of activation rows: every run of `block` consecutive values of a row is multiplied by the
// normalised Hadamard matrix of that size (fast Walsh-Hadamard transform inside a warp).  With weights whose input
// dimension was rotated the same way when they were quantised, x W^T = (x H)(W H)^T: the rotation spreads outlier input
// channels over the block, so group scales stop being set by one loud column.
// Reference: the activation-side 64-point Hadamard and the fold of the rotation into the weights
// (src/ops/linear e8act / prism_fold).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace nfb {

// x, out: [T, K] bf16 with leading dimensions ldx / ldo (may alias); K a multiple of block; block in {64, 128, 256}.
const char* hadamard_blocks(const __nv_bfloat16* x, int64_t ldx, __nv_bfloat16* out, int64_t ldo, int T, int K, int block,
                            cudaStream_t stream);

}  // namespace nfb
