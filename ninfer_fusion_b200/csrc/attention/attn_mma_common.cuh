// Shared pieces of the mma.sync attention kernels (decode split-KV and prefill): tile geometry,
// ldmatrix / mma wrappers and the raw-unit loader that dequantises 16 cache values to fp16 pairs.
#pragma once
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "../kv/codec.cuh"

namespace nfb {
namespace attn_mma {

constexpr int D = 256;
constexpr int kTileKeys = 64;
constexpr int kLdK = D + 8;          // halves per K-tile row
constexpr int kLdV = kTileKeys + 8;  // halves per V^T-tile row
constexpr int kLdP = kTileKeys + 8;
constexpr int kLdQ = D + 8;


__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// One "unit" = 16 consecutive values [16*part, 16*part+16) of a cache row.  Loading (raw bytes into
// registers) and converting (to 8 packed fp16 pairs) are separate so that a thread can put all of a
// tile's loads in flight before it converts the first one.  The fp8-row scale is NOT applied here (it
// multiplies scores / probabilities instead).
template <int FORMAT>
struct RawUnit {
  uint4 a;
  uint4 b;      // second half of a bf16 unit only
  float scale;  // int8-group / nvfp4 block scale
  int tier;     // mixed layers: the tier this unit was read from (decides how it is converted)

  __device__ __forceinline__ void clear() {
    a = make_uint4(0, 0, 0, 0);
    b = make_uint4(0, 0, 0, 0);
    scale = 0.f;
    tier = 0;
  }
  // `which` 0 = K, 1 = V; `r` as returned by kv_row_of (mixed layers: tier in the top bits)
  __device__ __forceinline__ void load_row(const KvLayer& kv, int which, long long r, int part) {
    if constexpr (FORMAT == kKvMixed) {
      tier = kv_row_tier(r);
      const long long rr = kv_row_index(r);
      const uint8_t* codes = which ? kv.tier_v_codes[tier] : kv.tier_k_codes[tier];
      if (tier == 0) {
        const uint4* src = reinterpret_cast<const uint4*>(codes + rr * (2 * D) + part * 32);
        a = src[0];
        b = src[1];
      } else if (tier == 1) {
        a = *reinterpret_cast<const uint4*>(codes + rr * D + part * 16);
      } else {
        const uint2 c = *reinterpret_cast<const uint2*>(codes + rr * (D / 2) + part * 8);
        a = make_uint4(c.x, c.y, 0, 0);
        const uint8_t* scales = which ? kv.tier_v_scales[2] : kv.tier_k_scales[2];
        scale = e4m3_to_float(scales[rr * (D / 16) + part]);
      }
    } else {
      load(kv, which ? kv.v_codes : kv.k_codes, which ? kv.v_scales : kv.k_scales, r, part);
    }
  }
  __device__ __forceinline__ void load(const KvLayer& kv, const uint8_t* codes, const uint8_t* scales, long long r,
                                       int part) {
    if constexpr (FORMAT == kKvFp8Row) {
      a = *reinterpret_cast<const uint4*>(codes + r * D + part * 16);
    } else if constexpr (FORMAT == kKvBf16) {
      const uint4* src = reinterpret_cast<const uint4*>(codes + r * (2 * D) + part * 32);
      a = src[0];
      b = src[1];
    } else if constexpr (FORMAT == kKvInt8Group) {
      a = *reinterpret_cast<const uint4*>(codes + r * D + part * 16);
      scale = __half2float(reinterpret_cast<const __half*>(scales + r * (2 * (D / kv.group)))[part * 16 / kv.group]);
    } else {
      const uint2 c = *reinterpret_cast<const uint2*>(codes + r * (D / 2) + part * 8);
      a = make_uint4(c.x, c.y, 0, 0);
      scale = e4m3_to_float(scales[r * (D / 16) + part]);
    }
  }
  __device__ __forceinline__ void convert(uint32_t* out) const {
    if constexpr (FORMAT == kKvMixed) {
      // one of the three tier codecs, chosen per unit
      if (tier == 0) {
        RawUnit<kKvBf16> u;
        u.a = a; u.b = b; u.scale = 0.f; u.tier = 0;
        u.convert(out);
      } else if (tier == 1) {
        RawUnit<kKvFp8Row> u;
        u.a = a; u.b = b; u.scale = 0.f; u.tier = 0;
        u.convert(out);
      } else {
        RawUnit<kKvNvfp4> u;
        u.a = a; u.b = b; u.scale = scale; u.tier = 0;
        u.convert(out);
      }
    } else if constexpr (FORMAT == kKvFp8Row) {
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffff), __NV_E4M3);
        const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
        out[2 * i] = *reinterpret_cast<const uint32_t*>(&lo);
        out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
    } else if constexpr (FORMAT == kKvBf16) {
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
        out[i] = pack_half2(__bfloat162float(v.x), __bfloat162float(v.y));
      }
    } else if constexpr (FORMAT == kKvInt8Group) {
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c0 = static_cast<int8_t>((w[i / 2] >> (16 * (i % 2))) & 0xff);
        const int c1 = static_cast<int8_t>((w[i / 2] >> (16 * (i % 2) + 8)) & 0xff);
        out[i] = pack_half2(static_cast<float>(c0) * scale, static_cast<float>(c1) * scale);
      }
    } else {
      // two e2m1 codes per byte -> fp16 pair in one conversion instruction, then the block scale (the product of an
      // e2m1 value and an e4m3 scale is exact in fp16, so this equals the fp32 route bit for bit)
      const uint32_t w[2] = {a.x, a.y};
      const __half2 s2 = __float2half2_rn(scale);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const __nv_fp4x2_storage_t pair = static_cast<__nv_fp4x2_storage_t>((w[i / 4] >> (8 * (i % 4))) & 0xff);
        const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(pair, __NV_E2M1);
        const __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&hr), s2);
        out[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
  }
};

}  // namespace attn_mma
}  // namespace nfb
