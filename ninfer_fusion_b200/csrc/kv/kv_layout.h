// KV-cache page layout descriptors shared by host and device code.
//
// A "row" is one (token, kv-head) vector of D values.  Storage per row:
//   BF16        : 2*D bytes of codes, no scales
//   FP8_ROW     : D bytes e4m3 codes + 1 fp16 scale
//   INT8_GROUP  : D bytes int8 codes + D/G fp16 scales
//   NVFP4       : D/2 bytes e2m1 codes + D/16 e4m3 scales
// Pages are [page, kv_head, token_in_page, row_bytes] for codes and
// [page, kv_head, token_in_page, scale_bytes] for scales.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define NFB_HD __host__ __device__
#else
#define NFB_HD
#endif

namespace nfb {

// kKvMixed: the layer's (64-token block x layer) cells live in one of three tiers, each with its own planes and
// codec (tier 0 bf16, tier 1 fp8-row, tier 2 nvfp4); `cell_map[page]` says where a logical page's cell is:
// tier << 28 | slot inside that tier's planes, or -1.  This is the storage side of per-cell precision descent
// (the reference's contract: src/product/kv_block_descent.h:1-58, narrow sentinels in its block-table entries,
// src/core/paged_kv_cache.h).
enum KvFormat : int { kKvBf16 = 0, kKvFp8Row = 1, kKvInt8Group = 2, kKvNvfp4 = 3, kKvMixed = 4 };
constexpr int kKvTiers = 3;
constexpr int kCellTierShift = 28;

struct KvLayer {
  uint8_t* k_codes;   // [pages, Hkv, P, row_bytes]
  uint8_t* v_codes;
  uint8_t* k_scales;  // [pages, Hkv, P, scale_bytes]  (nullptr for bf16)
  uint8_t* v_scales;
  int page_size;      // tokens per page
  int n_kv_heads;
  int head_dim;
  int format;         // KvFormat
  int group;          // int8 group size (32 or 64); 16 for nvfp4; head_dim for fp8 row
  // kKvMixed only
  const int* cell_map = nullptr;             // [logical pages]
  uint8_t* tier_k_codes[kKvTiers] = {};      // per tier: [slots, Hkv, P, row_bytes(tier format)]
  uint8_t* tier_v_codes[kKvTiers] = {};
  uint8_t* tier_k_scales[kKvTiers] = {};
  uint8_t* tier_v_scales[kKvTiers] = {};
};

NFB_HD inline int kv_tier_format(int tier) { return tier == 0 ? kKvBf16 : (tier == 1 ? kKvFp8Row : kKvNvfp4); }
NFB_HD inline int kv_tier_group(int tier, int D) { return tier == 2 ? 16 : D; }

NFB_HD inline int kv_row_bytes(int format, int D) {
  return format == kKvBf16 ? 2 * D : (format == kKvNvfp4 ? D / 2 : D);
}
NFB_HD inline int kv_scale_bytes(int format, int D, int group) {
  switch (format) {
    case kKvFp8Row: return 2;
    case kKvInt8Group: return 2 * (D / group);
    case kKvNvfp4: return D / 16;
    default: return 0;
  }
}

}  // namespace nfb
