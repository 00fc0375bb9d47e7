// One 16-value block of an nvfp4 (W4A4) activation row: e4m3 block scale = amax / 6, e2m1 codes, and the place of both
// in the operand the block-scaled GEMM reads -- codes row-major [T][K / 2], scales in the 512-byte tiles of the
// scale plane (128 rows x 4 scales, the layout tcgen05.cp expects).  Shared by the stand-alone quantiser and by the
// producers that quantise their own output (SwiGLU epilogue, GDN step, attention merge), so that all of them write the
// same bits.
#pragma once
#include <stdint.h>

#include "../kv/codec.cuh"

namespace nfb {

constexpr int kNvfp4SfTileBytes = 512;   // 128 rows x 4 scales

// `v`: the block's sixteen values as the consumer would read them from a bf16 tensor (already rounded to bf16);
// token row t, block g of the row (K / 16 blocks per row).
__device__ __forceinline__ void nvfp4_store_block(const float* v, int t, int g, int K, uint8_t* codes, uint8_t* sf_plane) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const uint8_t sc = float_to_e4m3(amax / 6.f);
  const float sf = e4m3_to_float(sc);
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    lo |= float_to_e2m1(sf > 0.f ? __fdiv_rn(v[i], sf) : 0.f) << (4 * i);
    hi |= float_to_e2m1(sf > 0.f ? __fdiv_rn(v[8 + i], sf) : 0.f) << (4 * i);
  }
  *reinterpret_cast<uint2*>(codes + static_cast<long long>(t) * (K / 2) + g * 8) = make_uint2(lo, hi);
  const int k_tiles = K / 64;
  const long long off = (static_cast<long long>(t / 128) * k_tiles + g / 4) * kNvfp4SfTileBytes + (t % 32) * 16 +
                        ((t % 128) / 32) * 4 + (g % 4);
  sf_plane[off] = sc;
}

}  // namespace nfb
