// Split-KV paged GQA attention for decode and small-T verify, reading
// bf16 / fp8-row / int8-group / nvfp4 pages with in-register dequantisation.
//
// Work item = (query token, kv head, key split).  A split covers an ABSOLUTE
// key range [s*split_keys, (s+1)*split_keys), and inside a split warp w owns
// the 32-key blocks w, w+4, ...; both are functions of key position only, so
// the decode of a token and a later verify pass over the same token reduce the
// same keys in the same order (the determinism the reference pins with its
// split_reference_keys envelope, include/ninfer/ops/gqa_attention.h:22-48).
// Partials are the (m, l, o) monoid with un-normalised o (base-2 exponent
// domain); the merge kernel applies the layer's sigmoid output gate.
//
// Reference kernels covered: kernel/gqa_attention_decode{,_bf16,_i8,_fp8,_nvfp4}.cuh,
// launcher/gqa_attention_decode*.cu (mma.sync / FFMA routes for sm_120a).
#include "attention.h"

#include <cstdlib>

#include <math_constants.h>

#include "../common/ptx.cuh"
#include "../kv/codec.cuh"
#include "../gemm/nvfp4_act.cuh"

namespace nfb {

namespace {

constexpr int kWarps = 4;

template <int FORMAT>
__device__ __forceinline__ float row_scale(const uint8_t* scales, long long r) {
  if constexpr (FORMAT == kKvFp8Row) return __half2float(reinterpret_cast<const __half*>(scales)[r]);
  return 1.f;
}

// 8 values [d0, d0+8) of row r, WITHOUT the per-row scale for fp8-row (applied by the caller).
template <int FORMAT, int D>
__device__ __forceinline__ void load8(const KvLayer& kv, const uint8_t* codes, const uint8_t* scales,
                                      long long r, int d0, float* out) {
  if constexpr (FORMAT == kKvBf16) {
    kv_load8<kKvBf16>(codes + r * (2 * D), nullptr, d0, 0, out);
  } else if constexpr (FORMAT == kKvFp8Row) {
    const uint2 c = *reinterpret_cast<const uint2*>(codes + r * D + d0);
    e4m3x4_to_float(c.x, out);
    e4m3x4_to_float(c.y, out + 4);
  } else if constexpr (FORMAT == kKvInt8Group) {
    kv_load8<kKvInt8Group>(codes + r * D, scales + r * (2 * (D / kv.group)), d0, kv.group, out);
  } else {
    kv_load8<kKvNvfp4>(codes + r * (D / 2), scales + r * (D / 16), d0, 16, out);
  }
}

template <int FORMAT, int G, int D>
__global__ void __launch_bounds__(kWarps * 32) paged_attn_split_kernel(const PagedAttnParams p) {
  constexpr int VPL = D / 32;  // output dims per lane
  __shared__ __align__(16) float q_s[G][D];
  __shared__ float p_s[kWarps][G][32];
  __shared__ long long row_s[kWarps][32];
  __shared__ __align__(16) float mrg_o[kWarps][G][D];
  __shared__ float mrg_m[kWarps][G], mrg_l[kWarps][G];

  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.q_seq[t];
  // selected-block mode: the key list is sel_count blocks of four tokens + the incomplete last block, addressed by ordinal
  const bool selected = p.sel_blocks != nullptr;
  const int real_len = p.q_kv_len[t];
  const int sel_keys = selected ? 4 * p.sel_count[t] : 0;
  const int sel_tail0 = (real_len / 4) * 4;                       // first token of the incomplete block
  const int kv_len = selected ? sel_keys + (real_len - sel_tail0) : real_len;
  const int* sel = selected ? p.sel_blocks + static_cast<long long>(t) * p.sel_stride : nullptr;
  // a sliding window drops the keys before kv_len - window; the split then starts at the window's edge
  const int k_begin = max(split * p.split_keys, p.window > 0 ? kv_len - p.window : 0);
  const int k_end = min(kv_len, (split + 1) * p.split_keys);
  const long long part_base = (static_cast<long long>(t) * p.n_q_heads + kvh * G) * p.n_splits + split;

  if (seq < 0 || k_begin >= k_end) {
    for (int g = threadIdx.x; g < G; g += blockDim.x) {
      float* ml = p.part_ml + (part_base + static_cast<long long>(g) * p.n_splits) * 2;
      ml[0] = -CUDART_INF_F;
      ml[1] = 0.f;
    }
    return;
  }

  // q, pre-scaled by sm_scale * log2(e) so that softmax runs on exp2.
  const float qscale = p.sm_scale * 1.4426950408889634f;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    q_s[g][d] = __bfloat162float(p.q[(static_cast<long long>(t) * p.n_q_heads + kvh * G + g) * D + d]) * qscale;
  }
  __syncthreads();

  const unsigned long long tmask = p.tree_mask ? p.tree_mask[t] : ~0ull;
  const int tbase = p.tree_mask ? p.tree_base[t] : 0x7fffffff;

  float m[G], l[G], o[G][VPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -CUDART_INF_F;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) o[g][j] = 0.f;
  }

  const int* table = p.block_table + static_cast<long long>(seq) * p.table_stride;
  const int P = p.kv.page_size;

  for (int kb = k_begin + warp * 32; kb < k_end; kb += kWarps * 32) {
    const int key = kb + lane;
    bool valid = key < k_end;
    if (valid && key >= tbase) valid = (tmask >> (key - tbase)) & 1ull;
    long long r = 0;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    if (valid) {
      const int pos = !selected ? key : key < sel_keys ? sel[key >> 2] * 4 + (key & 3) : sel_tail0 + key - sel_keys;
      const int page = table[pos / P];
      r = (static_cast<long long>(page) * p.kv.n_kv_heads + kvh) * P + pos % P;
#pragma unroll 4
      for (int c = 0; c < D / 8; ++c) {
        float kf[8];
        load8<FORMAT, D>(p.kv, p.kv.k_codes, p.kv.k_scales, r, c * 8, kf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
          s[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y +
                  kf[6] * qb.z + kf[7] * qb.w;
        }
      }
      const float ks = row_scale<FORMAT>(p.kv.k_scales, r);
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] *= ks;
    }
    const float vs = valid ? row_scale<FORMAT>(p.kv.v_scales, r) : 0.f;
    bool any = false;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float mb = warp_max(valid ? s[g] : -CUDART_INF_F);
      const float mn = fmaxf(m[g], mb);
      float pj = 0.f, corr = 1.f;
      if (mn > -CUDART_INF_F) {
        any = true;
        corr = exp2f(m[g] - mn);  // m[g] = -inf -> 0
        pj = valid ? exp2f(s[g] - mn) : 0.f;
        m[g] = mn;
      }
      l[g] = l[g] * corr + warp_sum(pj);
#pragma unroll
      for (int j = 0; j < VPL; ++j) o[g][j] *= corr;
      p_s[warp][g][lane] = pj * vs;
    }
    row_s[warp][lane] = valid ? r : -1;
    __syncwarp();
    if (any) {
      const int nblk = min(32, k_end - kb);
      for (int j = 0; j < nblk; ++j) {
        const long long rv = row_s[warp][j];
        if (rv < 0) continue;
        float vf[8];
        if constexpr (VPL == 8) {
          load8<FORMAT, D>(p.kv, p.kv.v_codes, p.kv.v_scales, rv, lane * 8, vf);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pj = p_s[warp][g][j];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[g][i] += pj * vf[i];
          }
        } else {
          // D = 128: lane pairs share one 8-wide load, each keeps its 4 dims
          load8<FORMAT, D>(p.kv, p.kv.v_codes, p.kv.v_scales, rv, (lane >> 1) * 8, vf);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pj = p_s[warp][g][j];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[g][i] += pj * vf[(lane & 1) * 4 + i];
          }
        }
      }
    }
    __syncwarp();
  }

  // ---- merge the four warps ----
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { mrg_m[warp][g] = m[g]; mrg_l[warp][g] = l[g]; }
#pragma unroll
    for (int j = 0; j < VPL; ++j) mrg_o[warp][g][lane * VPL + j] = o[g][j];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float mt = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, mrg_m[w][g]);
    float acc = 0.f, lt = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = mrg_m[w][g];
      if (mw > -CUDART_INF_F) {
        const float f = exp2f(mw - mt);
        acc += mrg_o[w][g][d] * f;
        lt += mrg_l[w][g] * f;
      }
    }
    const long long pb = part_base + static_cast<long long>(g) * p.n_splits;
    p.part_o[pb * D + d] = acc;
    if (d == 0) { p.part_ml[pb * 2] = mt; p.part_ml[pb * 2 + 1] = lt; }
  }
}

template <int D>
__global__ void __launch_bounds__(D / 4) paged_attn_merge_kernel(const PagedAttnParams p) {
  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x, h = blockIdx.y;
  const int d0 = threadIdx.x * 4;
  const long long pb = (static_cast<long long>(t) * p.n_q_heads + h) * p.n_splits;
  float mt = -CUDART_INF_F;
  for (int s = 0; s < p.n_splits; ++s) mt = fmaxf(mt, p.part_ml[(pb + s) * 2]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, lt = 0.f;
  for (int s = 0; s < p.n_splits; ++s) {
    const float ms = p.part_ml[(pb + s) * 2];
    if (ms > -CUDART_INF_F) {
      const float f = exp2f(ms - mt);
      const float4 o = *reinterpret_cast<const float4*>(p.part_o + (pb + s) * D + d0);
      acc[0] += o.x * f; acc[1] += o.y * f; acc[2] += o.z * f; acc[3] += o.w * f;
      lt += p.part_ml[(pb + s) * 2 + 1] * f;
    }
  }
  const float inv = lt > 0.f ? 1.f / lt : 0.f;
  float r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) r[i] = acc[i] * inv;
  if (p.gate != nullptr) {
    const uint2 gv = *reinterpret_cast<const uint2*>(p.gate + static_cast<long long>(t) * p.ld_gate + h * D + d0);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
    // attention output crosses a bf16 boundary before the gate in the reference schedule
    const float g0 = __bfloat162float(gp[0].x), g1 = __bfloat162float(gp[0].y);
    const float g2 = __bfloat162float(gp[1].x), g3 = __bfloat162float(gp[1].y);
    r[0] = __bfloat162float(__float2bfloat16(r[0])) / (1.f + __expf(-g0));
    r[1] = __bfloat162float(__float2bfloat16(r[1])) / (1.f + __expf(-g1));
    r[2] = __bfloat162float(__float2bfloat16(r[2])) / (1.f + __expf(-g2));
    r[3] = __bfloat162float(__float2bfloat16(r[3])) / (1.f + __expf(-g3));
  }
  uint2 ov;
  ov.x = pack_bf16x2(r[0], r[1]);
  ov.y = pack_bf16x2(r[2], r[3]);
  *reinterpret_cast<uint2*>(p.out + (static_cast<long long>(t) * p.n_q_heads + h) * D + d0) = ov;
  if (p.q_codes != nullptr) {
    // the output row also as the next GEMM's nvfp4 operand: four threads hold one 16-value block
    const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&ov);
    const float mine[4] = {__bfloat162float(ob[0].x), __bfloat162float(ob[0].y), __bfloat162float(ob[1].x),
                           __bfloat162float(ob[1].y)};
    float v[16];
    const int base = threadIdx.x & ~3;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * j + i] = __shfl_sync(0xffffffffu, mine[i], (base + j) & 31);
    if ((threadIdx.x & 3) == 0)
      nvfp4_store_block(v, t, (h * D + d0) / 16, p.n_q_heads * D, p.q_codes, p.q_sf);
  }
}

template <typename K>
cudaError_t launch(K kern, dim3 grid, dim3 block, const PagedAttnParams& p, cudaStream_t stream, bool pdl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int FORMAT, int D>
cudaError_t launch_g(int G, dim3 grid, const PagedAttnParams& p, cudaStream_t stream, bool pdl) {
  const dim3 block(kWarps * 32);
  switch (G) {
    case 1: return launch(paged_attn_split_kernel<FORMAT, 1, D>, grid, block, p, stream, pdl);
    case 2: return launch(paged_attn_split_kernel<FORMAT, 2, D>, grid, block, p, stream, pdl);
    case 3: return launch(paged_attn_split_kernel<FORMAT, 3, D>, grid, block, p, stream, pdl);
    case 4: return launch(paged_attn_split_kernel<FORMAT, 4, D>, grid, block, p, stream, pdl);
    case 6: return launch(paged_attn_split_kernel<FORMAT, 6, D>, grid, block, p, stream, pdl);
    case 8: return launch(paged_attn_split_kernel<FORMAT, 8, D>, grid, block, p, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

template <int D>
cudaError_t launch_f(int G, dim3 grid, const PagedAttnParams& p, cudaStream_t stream, bool pdl) {
  switch (p.kv.format) {
    case kKvBf16: return launch_g<kKvBf16, D>(G, grid, p, stream, pdl);
    case kKvFp8Row: return launch_g<kKvFp8Row, D>(G, grid, p, stream, pdl);
    case kKvInt8Group: return launch_g<kKvInt8Group, D>(G, grid, p, stream, pdl);
    case kKvNvfp4: return launch_g<kKvNvfp4, D>(G, grid, p, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// NFB_ATTN_TC=0 keeps the mma.sync kernel for fp8-row pages (comparison runs).
static bool tc_attention_enabled() {
  static const bool on = [] {
    const char* e = getenv("NFB_ATTN_TC");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

const char* paged_attention(const PagedAttnParams& p, cudaStream_t stream, bool pdl) {
  if (p.Tq <= 0) return nullptr;
  if (p.head_dim != 256 && p.head_dim != 128) return "paged_attention: head_dim must be 128 or 256";
  if (p.n_q_heads % p.n_kv_heads) return "paged_attention: q heads must be a multiple of kv heads";
  if (p.split_keys <= 0 || p.split_keys % 128) return "paged_attention: split_keys must be a positive multiple of 128";
  if (p.n_splits < 1) return "paged_attention: need at least one split";
  if (p.sel_blocks != nullptr) {
    if (p.sel_count == nullptr || p.sel_stride <= 0) return "paged_attention: selection needs counts and a row stride";
    if (p.window > 0 || p.tree_mask != nullptr) return "paged_attention: selection excludes a window or a tree mask";
  }
  if (p.gate != nullptr && (p.ld_gate % 4 || reinterpret_cast<uintptr_t>(p.gate) % 8))
    return "paged_attention: gate rows must be 8-byte aligned";
  const int G = p.n_q_heads / p.n_kv_heads;
  const dim3 grid(p.Tq, p.n_kv_heads, p.n_splits);
  cudaError_t e = cudaErrorNotSupported;
  if ((p.impl == 3 || (p.impl == 0 && tc_attention_enabled())) && p.sel_blocks == nullptr) {
    e = paged_attention_tc_split(p, stream, pdl);   // fp8-row pages straight into tcgen05.mma
    if (e == cudaErrorNotSupported && p.impl == 3) return "paged_attention: problem not supported by the tcgen05 kernel";
  }
  if (e == cudaErrorNotSupported && p.impl != 1 && p.sel_blocks == nullptr) {   // the gathered key list runs on the SIMT kernel
    e = paged_attention_mma_split(p, stream, pdl);
    if (e == cudaErrorNotSupported && p.impl == 2) return "paged_attention: geometry not supported by the tensor-core kernel";
  }
  if (e == cudaErrorNotSupported)
    e = p.head_dim == 256 ? launch_f<256>(G, grid, p, stream, pdl) : launch_f<128>(G, grid, p, stream, pdl);
  if (e == cudaErrorInvalidValue) return "paged_attention: unsupported GQA group size or KV format";
  if (e != cudaSuccess) return cudaGetErrorString(e);
  const dim3 mgrid(p.Tq, p.n_q_heads);
  e = p.head_dim == 256 ? launch(paged_attn_merge_kernel<256>, mgrid, dim3(64), p, stream, pdl)
                        : launch(paged_attn_merge_kernel<128>, mgrid, dim3(32), p, stream, pdl);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
