// Device side of the cold slot (the requantised form a retired KV page plane takes before it leaves the device):
// 16-byte header | packed E2M1 nibbles | E4M3 scale per 16 values.  Same bytes as kv/cold_codec.py writes on the host.
// Reference: include/ninfer/ops/cold_i8.h (cold_i8_slot_pack_raw / _restore_raw / _restore_bf16_raw).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace nfb {

constexpr uint32_t kColdSlotMagic = 0x31534C43u;   // "CLS1"
constexpr int kColdSlotHeader = 16;

inline int64_t cold_slot_bytes(int rows, int dim) { return kColdSlotHeader + int64_t(rows) * dim / 2 + int64_t(rows) * dim / 16; }

// int8 group-64 planes (codes [n_slots * rows, dim], fp16 scales [n_slots * rows, dim / 64]) -> n_slots slots
const char* cold_slot_pack_int8(const int8_t* codes, const void* scales_fp16, int n_slots, int rows, int dim, uint8_t* slots,
                                cudaStream_t stream);
// slots -> int8 group-64 planes (scale = fp16(amax / 127), codes clamped to +-127)
const char* cold_slot_restore_int8(const uint8_t* slots, int n_slots, int rows, int dim, int8_t* codes, void* scales_fp16,
                                   cudaStream_t stream);
// slots -> bf16 plane [n_slots * rows, dim]
const char* cold_slot_restore_bf16(const uint8_t* slots, int n_slots, int rows, int dim, void* out_bf16, cudaStream_t stream);

}  // namespace nfb
