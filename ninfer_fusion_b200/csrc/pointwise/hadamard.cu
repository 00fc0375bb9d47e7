// One warp per (row, block): VPL = block / 32 values per lane, log2(VPL) butterflies in registers, five across lanes.
#include "hadamard.h"

namespace nfb {
namespace {

template <int VPL>
__global__ void __launch_bounds__(128) hadamard_blocks_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                                              __nv_bfloat16* __restrict__ out, int64_t ldo, int T,
                                                              int blocks_per_row) {
  const int lane = threadIdx.x & 31;
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (unit >= static_cast<int64_t>(T) * blocks_per_row) return;
  const int row = static_cast<int>(unit / blocks_per_row), blk = static_cast<int>(unit % blocks_per_row);
  const int col = blk * (VPL * 32) + lane * VPL;
  float v[VPL];
  const __nv_bfloat16* src = x + row * ldx + col;
#pragma unroll
  for (int j = 0; j < VPL; j += 2) {
    const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(src + j);
    v[j] = __bfloat162float(p.x); v[j + 1] = __bfloat162float(p.y);
  }
  // index inside the block = lane * VPL + j: the low log2(VPL) bits live in j, the upper five in the lane id
#pragma unroll
  for (int s = 1; s < VPL; s <<= 1) {
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      if ((j & s) == 0) {
        const float a = v[j], b = v[j | s];
        v[j] = a + b;
        v[j | s] = a - b;
      }
    }
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = (lane & m) ? o - v[j] : v[j] + o;
    }
  }
  const float norm = rsqrtf(static_cast<float>(VPL * 32));
  __nv_bfloat16* dst = out + row * ldo + col;
#pragma unroll
  for (int j = 0; j < VPL; j += 2)
    *reinterpret_cast<__nv_bfloat162*>(dst + j) = __floats2bfloat162_rn(v[j] * norm, v[j + 1] * norm);
}

}  // namespace

const char* hadamard_blocks(const __nv_bfloat16* x, int64_t ldx, __nv_bfloat16* out, int64_t ldo, int T, int K, int block,
                            cudaStream_t stream) {
  if (T <= 0 || K <= 0) return nullptr;
  if (block != 64 && block != 128 && block != 256) return "hadamard_blocks: block must be 64, 128 or 256";
  if (K % block) return "hadamard_blocks: K must be a multiple of the block";
  if (ldx % 2 || ldo % 2 || (reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(out) & 3))
    return "hadamard_blocks: rows must be 4-byte aligned";
  const int bpr = K / block;
  const int64_t units = static_cast<int64_t>(T) * bpr;
  const unsigned grid = static_cast<unsigned>((units + 3) / 4);
  if (block == 64) hadamard_blocks_kernel<2><<<grid, 128, 0, stream>>>(x, ldx, out, ldo, T, bpr);
  else if (block == 128) hadamard_blocks_kernel<4><<<grid, 128, 0, stream>>>(x, ldx, out, ldo, T, bpr);
  else hadamard_blocks_kernel<8><<<grid, 128, 0, stream>>>(x, ldx, out, ldo, T, bpr);
  return cudaGetLastError() == cudaSuccess ? nullptr : "hadamard_blocks: launch failed";
}

}  // namespace nfb
