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

enum KvFormat : int { kKvBf16 = 0, kKvFp8Row = 1, kKvInt8Group = 2, kKvNvfp4 = 3 };

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
};

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
