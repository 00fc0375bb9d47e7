// KV-cache row codecs shared by the quantize-append kernels and by the
// attention kernels' in-register dequantisation.
//
// A "row" is one (token, kv-head) vector of D values.  Storage per row:
//   BF16        : 2*D bytes of codes, no scales
//   FP8_ROW     : D bytes e4m3 codes + 1 fp16 scale        (scale = fp16(clamp(amax/448, 2^-24, 65504)))
//   INT8_GROUP  : D bytes int8 codes + D/G fp16 scales     (scale = fp16(amax_g/127), codes clamp +-127)
//   NVFP4       : D/2 bytes e2m1 codes + D/16 e4m3 scales  (scale = e4m3(amax_16/6))
// These follow the reference's codec contracts (include/ninfer/ops/kv_cache_append.h:54-83,
// src/ops/kv_cache/int8_g64_codec.cuh, fp8_e4m3_row_codec.cuh, nvfp4_group16_codec.cuh) with the
// int8 group size and the page size as parameters instead of constants.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "kv_layout.h"

namespace nfb {

// ---- scalar converters ----
__device__ __forceinline__ float e4m3_to_float(uint8_t c) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(c, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&hr));
}
__device__ __forceinline__ uint8_t float_to_e4m3(float f) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3));
}
// four packed e4m3 -> four floats
__device__ __forceinline__ void e4m3x4_to_float(uint32_t c, float* o) {
  const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(c & 0xffff), __NV_E4M3);
  const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(c >> 16), __NV_E4M3);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
// e2m1 magnitude table: 0, .5, 1, 1.5, 2, 3, 4, 6 ; bit 3 = sign
__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
  const uint32_t m = nib & 7;
  const float mag = m < 4 ? 0.5f * m : (m == 4 ? 2.f : (m == 5 ? 3.f : (m == 6 ? 4.f : 6.f)));
  return (nib & 8) ? -mag : mag;
}
// round-to-nearest-even onto the e2m1 grid
__device__ __forceinline__ uint32_t float_to_e2m1(float f) {
  const uint32_t sign = f < 0.f ? 8u : 0u;
  const float a = fabsf(f);
  uint32_t m;
  if (a <= 0.25f) m = 0;          // tie at .25 -> 0 (even)
  else if (a < 0.75f) m = 1;
  else if (a <= 1.25f) m = 2;     // ties .75 -> 1.0, 1.25 -> 1.0
  else if (a < 1.75f) m = 3;
  else if (a <= 2.5f) m = 4;      // ties 1.75 -> 2, 2.5 -> 2
  else if (a < 3.5f) m = 5;
  else if (a <= 5.f) m = 6;       // ties 3.5 -> 4, 5 -> 4
  else m = 7;
  return sign | m;
}

// ---- where the row of (logical page, kv head, token in page) lives ----
// Uniform layers: the row index inside the layer's planes.  Mixed layers: the row index inside the cell's tier,
// with the tier in bits 56.. (kv_row_tier / kv_row_index take it apart).  -1: no page / no cell.
constexpr long long kRowIndexMask = (1LL << 56) - 1;
__device__ __forceinline__ long long kv_row_of(const KvLayer& kv, int page, int kvh, int in_page) {
  if (page < 0) return -1;
  if (kv.format != kKvMixed)
    return (static_cast<long long>(page) * kv.n_kv_heads + kvh) * kv.page_size + in_page;
  const int cell = kv.cell_map[page];
  if (cell < 0) return -1;
  const long long slot = cell & ((1 << kCellTierShift) - 1);
  return ((slot * kv.n_kv_heads + kvh) * kv.page_size + in_page) |
         (static_cast<long long>(cell >> kCellTierShift) << 56);
}
__device__ __forceinline__ int kv_row_tier(long long r) { return static_cast<int>(r >> 56); }
__device__ __forceinline__ long long kv_row_index(long long r) { return r & kRowIndexMask; }

// ---- dequantise 8 consecutive values [d0, d0+8) of a row into floats ----
template <int FORMAT>
__device__ __forceinline__ void kv_load8(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                         int d0, int group, float* out) {
  if constexpr (FORMAT == kKvBf16) {
    const uint4 r = *reinterpret_cast<const uint4*>(codes + 2 * d0);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) { out[2 * j] = __bfloat162float(p[j].x); out[2 * j + 1] = __bfloat162float(p[j].y); }
  } else if constexpr (FORMAT == kKvFp8Row) {
    const uint2 r = *reinterpret_cast<const uint2*>(codes + d0);
    const float s = __half2float(*reinterpret_cast<const __half*>(scales));
    e4m3x4_to_float(r.x, out);
    e4m3x4_to_float(r.y, out + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] *= s;
  } else if constexpr (FORMAT == kKvInt8Group) {
    const uint2 r = *reinterpret_cast<const uint2*>(codes + d0);
    const float s = __half2float(reinterpret_cast<const __half*>(scales)[d0 / group]);
    const int8_t* c = reinterpret_cast<const int8_t*>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = static_cast<float>(c[j]) * s;
  } else {
    const uint32_t r = *reinterpret_cast<const uint32_t*>(codes + d0 / 2);
    const float s = e4m3_to_float(scales[d0 / 16]);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = e2m1_to_float((r >> (4 * j)) & 0xf) * s;
  }
}

// ---- quantise one row held by a full warp: lane owns D/32 consecutive values ----
// D must be 128 or 256 (4 or 8 values per lane).  `vals` are the lane's values
// [lane*VPL, lane*VPL+VPL).  Writes codes and scales for the whole row.
template <int VPL>
__device__ __forceinline__ void kv_store_row_warp(int format, int group, const float* vals,
                                                  uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                                  int lane) {
  const int d0 = lane * VPL;
  if (format == kKvBf16) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(codes) + d0;
#pragma unroll
    for (int j = 0; j < VPL; ++j) o[j] = __float2bfloat16(vals[j]);
    return;
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) amax = fmaxf(amax, fabsf(vals[j]));
  if (format == kKvFp8Row) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sf = fminf(fmaxf(amax / 448.f, 5.9604644775390625e-8f), 65504.f);
    const __half sh = __float2half_rn(sf);
    sf = __half2float(sh);
    if (lane == 0) *reinterpret_cast<__half*>(scales) = sh;
    // true division (not a reciprocal multiply): the codec contract is code = e4m3(x / scale)
#pragma unroll
    for (int j = 0; j < VPL; ++j) codes[d0 + j] = float_to_e4m3(__fdiv_rn(vals[j], sf));
  } else if (format == kKvInt8Group) {
    const int lanes_per_group = group / VPL;  // 32/8=4, 64/8=8, 32/4=8, 64/4=16
    for (int o = lanes_per_group / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const __half sh = __float2half_rn(amax / 127.f);
    const float sf = __half2float(sh);
    if ((lane % lanes_per_group) == 0) reinterpret_cast<__half*>(scales)[d0 / group] = sh;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      float q = sf > 0.f ? rintf(__fdiv_rn(vals[j], sf)) : 0.f;
      q = fminf(fmaxf(q, -127.f), 127.f);
      reinterpret_cast<int8_t*>(codes)[d0 + j] = static_cast<int8_t>(q);
    }
  } else {  // nvfp4, blocks of 16
    const int lanes_per_group = 16 / VPL;  // 2 or 4
    for (int o = lanes_per_group / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint8_t sc = float_to_e4m3(amax / 6.f);
    const float sf = e4m3_to_float(sc);
    if ((lane % lanes_per_group) == 0) scales[d0 / 16] = sc;
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < VPL; ++j) packed |= float_to_e2m1(sf > 0.f ? __fdiv_rn(vals[j], sf) : 0.f) << (4 * j);
    if (VPL == 8) *reinterpret_cast<uint32_t*>(codes + d0 / 2) = packed;
    else *reinterpret_cast<uint16_t*>(codes + d0 / 2) = static_cast<uint16_t>(packed);
  }
}

}  // namespace nfb
