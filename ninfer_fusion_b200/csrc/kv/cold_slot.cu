// Cold-slot pack / restore kernels: element-wise, one thread per group (16 values when packing or restoring to bf16,
// 64 when restoring the int8 tier's planes).  They run on the copy path of a retiring page, never on the decode path.
#include "cold_slot.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "codec.cuh"

namespace nfb {
namespace {

__device__ __forceinline__ void write_header(uint8_t* slot, int rows, int dim) {
  uint32_t* h = reinterpret_cast<uint32_t*>(slot);
  h[0] = kColdSlotMagic;
  h[1] = static_cast<uint32_t>(rows) | (static_cast<uint32_t>(dim) << 16);
  h[2] = 0; h[3] = 0;
}

__global__ void __launch_bounds__(256) pack_int8_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales,
                                                        int n_slots, int rows, int dim, uint8_t* __restrict__ slots,
                                                        long long slot_bytes) {
  const long long g16 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;    // group of 16 values
  const int per_row = dim / 16;
  const long long per_slot = static_cast<long long>(rows) * per_row;
  if (g16 >= per_slot * n_slots) return;
  const int slot = static_cast<int>(g16 / per_slot);
  const long long in_slot = g16 % per_slot;
  const long long row = static_cast<long long>(slot) * rows + in_slot / per_row;
  const int c0 = static_cast<int>(in_slot % per_row) * 16;
  uint8_t* dst = slots + slot * slot_bytes;
  if (in_slot == 0) write_header(dst, rows, dim);
  const float s64 = __half2float(scales[row * (dim / 64) + c0 / 64]);
  const int4 raw = *reinterpret_cast<const int4*>(codes + row * dim + c0);
  const int8_t* c = reinterpret_cast<const int8_t*>(&raw);
  float v[16];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) { v[i] = static_cast<float>(c[i]) * s64; amax = fmaxf(amax, fabsf(v[i])); }
  const uint8_t sc = float_to_e4m3(amax / 6.0f);
  const float s = e4m3_to_float(sc);
  const float inv = s > 0.f ? 1.0f / s : 0.f;
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i >> 3] |= float_to_e2m1(v[i] * inv) << (4 * (i & 7));
  *reinterpret_cast<uint2*>(dst + kColdSlotHeader + in_slot * 8) = make_uint2(w[0], w[1]);
  dst[kColdSlotHeader + per_slot * 8 + in_slot] = sc;
}

__device__ __forceinline__ void decode16(const uint8_t* slot, long long per_slot, long long in_slot, float* v) {
  const uint2 w = *reinterpret_cast<const uint2*>(slot + kColdSlotHeader + in_slot * 8);
  const float s = e4m3_to_float(slot[kColdSlotHeader + per_slot * 8 + in_slot]);
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = e2m1_to_float(((i < 8 ? w.x : w.y) >> (4 * (i & 7))) & 0xF) * s;
}

__global__ void __launch_bounds__(256) restore_bf16_kernel(const uint8_t* __restrict__ slots, int n_slots, int rows, int dim,
                                                           __nv_bfloat16* __restrict__ out, long long slot_bytes) {
  const long long g16 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = dim / 16;
  const long long per_slot = static_cast<long long>(rows) * per_row;
  if (g16 >= per_slot * n_slots) return;
  const int slot = static_cast<int>(g16 / per_slot);
  const long long in_slot = g16 % per_slot;
  float v[16];
  decode16(slots + slot * slot_bytes, per_slot, in_slot, v);
  __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + (static_cast<long long>(slot) * rows + in_slot / per_row) * dim +
                                                          (in_slot % per_row) * 16);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
}

__global__ void __launch_bounds__(256) restore_int8_kernel(const uint8_t* __restrict__ slots, int n_slots, int rows, int dim,
                                                           int8_t* __restrict__ codes, __half* __restrict__ scales,
                                                           long long slot_bytes) {
  const long long g64 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;    // group of 64 values
  const int per_row64 = dim / 64;
  const long long per_slot64 = static_cast<long long>(rows) * per_row64;
  if (g64 >= per_slot64 * n_slots) return;
  const int slot = static_cast<int>(g64 / per_slot64);
  const long long in64 = g64 % per_slot64;
  const long long per_slot16 = per_slot64 * 4;
  float v[64];
  float amax = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) decode16(slots + slot * slot_bytes, per_slot16, in64 * 4 + q, v + 16 * q);
#pragma unroll
  for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const __half sh = __float2half_rn(amax / 127.0f);
  const float s = __half2float(sh);
  const float inv = s > 0.f ? 1.0f / s : 0.f;
  const long long row = static_cast<long long>(slot) * rows + in64 / per_row64;
  const int c0 = static_cast<int>(in64 % per_row64) * 64;
  scales[row * per_row64 + c0 / 64] = sh;
  int8_t* dst = codes + row * dim + c0;
#pragma unroll
  for (int i = 0; i < 64; i += 4) {
    char4 o;
    o.x = static_cast<signed char>(fminf(127.f, fmaxf(-127.f, rintf(v[i] * inv))));
    o.y = static_cast<signed char>(fminf(127.f, fmaxf(-127.f, rintf(v[i + 1] * inv))));
    o.z = static_cast<signed char>(fminf(127.f, fmaxf(-127.f, rintf(v[i + 2] * inv))));
    o.w = static_cast<signed char>(fminf(127.f, fmaxf(-127.f, rintf(v[i + 3] * inv))));
    *reinterpret_cast<char4*>(dst + i) = o;
  }
}

const char* check(int n_slots, int rows, int dim) {
  if (n_slots <= 0 || rows <= 0 || rows > 65535 || dim <= 0 || dim > 65535) return "cold slot: bad geometry";
  if (dim % 64) return "cold slot: dim must be a multiple of 64";
  if (cold_slot_bytes(rows, dim) % 16) return "cold slot: slot size must be a multiple of 16 bytes";
  return nullptr;
}

}  // namespace

const char* cold_slot_pack_int8(const int8_t* codes, const void* scales_fp16, int n_slots, int rows, int dim, uint8_t* slots,
                                cudaStream_t stream) {
  if (const char* e = check(n_slots, rows, dim)) return e;
  const long long groups = static_cast<long long>(n_slots) * rows * (dim / 16);
  pack_int8_kernel<<<static_cast<unsigned>((groups + 255) / 256), 256, 0, stream>>>(
      codes, static_cast<const __half*>(scales_fp16), n_slots, rows, dim, slots, cold_slot_bytes(rows, dim));
  return cudaGetLastError() == cudaSuccess ? nullptr : "cold_slot_pack_int8: launch failed";
}

const char* cold_slot_restore_int8(const uint8_t* slots, int n_slots, int rows, int dim, int8_t* codes, void* scales_fp16,
                                   cudaStream_t stream) {
  if (const char* e = check(n_slots, rows, dim)) return e;
  const long long groups = static_cast<long long>(n_slots) * rows * (dim / 64);
  restore_int8_kernel<<<static_cast<unsigned>((groups + 255) / 256), 256, 0, stream>>>(
      slots, n_slots, rows, dim, codes, static_cast<__half*>(scales_fp16), cold_slot_bytes(rows, dim));
  return cudaGetLastError() == cudaSuccess ? nullptr : "cold_slot_restore_int8: launch failed";
}

const char* cold_slot_restore_bf16(const uint8_t* slots, int n_slots, int rows, int dim, void* out_bf16, cudaStream_t stream) {
  if (const char* e = check(n_slots, rows, dim)) return e;
  const long long groups = static_cast<long long>(n_slots) * rows * (dim / 16);
  restore_bf16_kernel<<<static_cast<unsigned>((groups + 255) / 256), 256, 0, stream>>>(
      slots, n_slots, rows, dim, static_cast<__nv_bfloat16*>(out_bf16), cold_slot_bytes(rows, dim));
  return cudaGetLastError() == cudaSuccess ? nullptr : "cold_slot_restore_bf16: launch failed";
}

}  // namespace nfb
