// Moves KV cells of a mixed-precision layer from one tier to another, re-encoding every row with the target
// tier's codec (tier 0 bf16 -> tier 1 fp8-row -> tier 2 nvfp4; any pair works, also upwards).  One warp per
// (cell, kv head, token, K or V) row: the lane's eight values are decoded with the source codec and stored with the
// same row quantiser the append path uses, so a cell that descends holds exactly what an append of the represented
// values in the target format would have written.
//
// This is the device half of per-cell precision descent (the reference's contract for it:
// src/product/kv_block_descent.h:1-58; its device side re-encodes blocks inside the attention launchers).  The host
// half (which cells, under which budgets) is kv/descent.py, driven by the engine between rounds.
#include "../attention/attention.h"
#include "../common/ptx.cuh"
#include "codec.cuh"

namespace nfb {

namespace {

__device__ __forceinline__ void load_row8(int tier, const uint8_t* codes, const uint8_t* scales, long long r, int D,
                                          int d0, float* v) {
  if (tier == 0) {
    kv_load8<kKvBf16>(codes + r * (2 * D), nullptr, d0, D, v);
  } else if (tier == 1) {
    kv_load8<kKvFp8Row>(codes + r * D, scales + r * 2, d0, D, v);
  } else {
    kv_load8<kKvNvfp4>(codes + r * (D / 2), scales + r * (D / 16), d0, 16, v);
  }
}

__global__ void __launch_bounds__(128) kv_requant_kernel(const KvRequantParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long id = static_cast<long long>(blockIdx.x) * 4 + warp;
  const int P = p.kv.page_size, H = p.kv.n_kv_heads, D = p.kv.head_dim;
  const long long rows = static_cast<long long>(p.n_cells) * H * P * 2;
  if (id >= rows) return;
  const int which = static_cast<int>(id & 1);
  const int tok = static_cast<int>((id >> 1) % P);
  const int h = static_cast<int>(((id >> 1) / P) % H);
  const int c = static_cast<int>((id >> 1) / P / H);
  const int src = p.src_cell[c], dst = p.dst_cell[c];
  if (src < 0 || dst < 0) return;
  const int st = src >> kCellTierShift, dt = dst >> kCellTierShift;
  const long long rs = (static_cast<long long>(src & ((1 << kCellTierShift) - 1)) * H + h) * P + tok;
  const long long rd = (static_cast<long long>(dst & ((1 << kCellTierShift) - 1)) * H + h) * P + tok;
  float v[8];
  load_row8(st, which ? p.kv.tier_v_codes[st] : p.kv.tier_k_codes[st],
            which ? p.kv.tier_v_scales[st] : p.kv.tier_k_scales[st], rs, D, lane * 8, v);
  const int fmt = kv_tier_format(dt), group = kv_tier_group(dt, D);
  const int rb = kv_row_bytes(fmt, D), sb = kv_scale_bytes(fmt, D, group);
  uint8_t* codes = (which ? p.kv.tier_v_codes[dt] : p.kv.tier_k_codes[dt]) + rd * rb;
  uint8_t* scales = sb ? (which ? p.kv.tier_v_scales[dt] : p.kv.tier_k_scales[dt]) + rd * sb : nullptr;
  kv_store_row_warp<8>(fmt, group, v, codes, scales, lane);
}

}  // namespace

const char* kv_requant(const KvRequantParams& p, cudaStream_t stream) {
  if (p.n_cells <= 0) return nullptr;
  if (p.kv.head_dim != 256) return "kv_requant: head_dim must be 256";
  if (p.src_cell == nullptr || p.dst_cell == nullptr) return "kv_requant: missing cell lists";
  for (int t = 0; t < kKvTiers; ++t)
    if (p.kv.tier_k_codes[t] == nullptr || p.kv.tier_v_codes[t] == nullptr) return "kv_requant: a tier has no planes";
  const long long rows = static_cast<long long>(p.n_cells) * p.kv.n_kv_heads * p.kv.page_size * 2;
  kv_requant_kernel<<<static_cast<unsigned int>((rows + 3) / 4), 128, 0, stream>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
