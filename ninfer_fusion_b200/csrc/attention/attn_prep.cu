// Attention-layer prologue, one launch for all heads of all tokens:
//   q: per-head RMSNorm(+1) -> partial NeoX RoPE (first rot_dim dims) -> bf16 [T, Hq, D]
//   k: per-head RMSNorm(+1) -> RoPE -> quantise -> paged KV cache row
//   v: quantise -> paged KV cache row
// One warp per (token, head) row; D = 256 (8 values per lane) or 128 (4 per lane).
// Reference ops this replaces: rmsnorm on q/k, ops::rope, gqa_kv_append /
// kv_cache_append (include/ninfer/ops/rope.h:76-104, kv_cache_append.h:54-83).
#include "attention.h"

#include "../common/ptx.cuh"
#include "../kv/codec.cuh"

namespace nfb {

namespace {

template <int VPL>
__global__ void __launch_bounds__(128) attn_prep_kernel(const AttnPrepParams p) {
  pdl_launch_next();
  pdl_wait_prior();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int heads_per_tok = p.n_q_heads + 2 * p.n_kv_heads;
  if (row >= p.T * heads_per_tok) return;
  const int t = row / heads_per_tok;
  const int hh = row % heads_per_tok;
  const int D = VPL * 32;
  const int d0 = lane * VPL;

  int kind, h;  // 0 = q, 1 = k, 2 = v
  const __nv_bfloat16* src;
  if (hh < p.n_q_heads) { kind = 0; h = hh; src = p.proj + static_cast<long long>(t) * p.ld_proj + p.q_off + h * D; }
  else if (hh < p.n_q_heads + p.n_kv_heads) { kind = 1; h = hh - p.n_q_heads; src = p.proj + static_cast<long long>(t) * p.ld_proj + p.k_off + h * D; }
  else { kind = 2; h = hh - p.n_q_heads - p.n_kv_heads; src = p.proj + static_cast<long long>(t) * p.ld_proj + p.v_off + h * D; }

  float v[VPL];
  if (VPL == 8) {
    const uint4 r = *reinterpret_cast<const uint4*>(src + d0);
    const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[2 * j] = __bfloat162float(rp[j].x); v[2 * j + 1] = __bfloat162float(rp[j].y); }
  } else {
    const uint2 r = *reinterpret_cast<const uint2*>(src + d0);
    const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < VPL / 2; ++j) { v[2 * j] = __bfloat162float(rp[j].x); v[2 * j + 1] = __bfloat162float(rp[j].y); }
  }

  if (kind != 2) {
    // ---- RMSNorm over the head ----
    const __nv_bfloat16* w = kind == 0 ? p.q_norm_w : p.k_norm_w;
    if (w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VPL; ++j) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / D + p.eps);
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        float wd = __bfloat162float(w[d0 + j]);
        if (p.unit_offset) wd += 1.f;
        // bf16 rounding point of the reference's stand-alone norm op
        v[j] = __bfloat162float(__float2bfloat16(v[j] * inv * wd));
      }
    }
    // ---- partial NeoX RoPE: pairs (i, i + rot/2), i < rot/2 ----
    const int half = p.rot_dim / 2;
    if (half > 0) {
      const int lanes_half = half / VPL;  // lanes covering the first half
      float other[VPL];
#pragma unroll
      for (int j = 0; j < VPL; ++j) other[j] = __shfl_xor_sync(0xffffffffu, v[j], lanes_half);
      if (lane < 2 * lanes_half) {
        const bool first = lane < lanes_half;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          const int i = (d0 + j) % half;  // pair index
          const int axis = p.pos_axes == 3 ? (i % 3) : 0;
          const float pos = static_cast<float>(p.rope_pos[static_cast<long long>(t) * p.pos_axes + axis]);
          float sn, cs;
          sincosf(pos * p.inv_freq[i], &sn, &cs);
          sn *= p.rope_attn_factor; cs *= p.rope_attn_factor;
          v[j] = first ? (v[j] * cs - other[j] * sn) : (v[j] * cs + other[j] * sn);
        }
      }
    }
  }

  if (kind != 2 && p.k_hadamard) {
    // fast Walsh-Hadamard transform over the head: index = lane * VPL + j, one butterfly per index bit
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
    const float norm = rsqrtf(static_cast<float>(D));
#pragma unroll
    for (int j = 0; j < VPL; ++j) v[j] *= norm;
  }

  if (kind != 2 && p.k_row_scale != nullptr) {
    // balance the channels of the stored K frame; q takes the inverse so that q . k does not change
    const int kvh = kind == 1 ? h : h / (p.n_q_heads / p.n_kv_heads);
    const __nv_bfloat16* s = p.k_row_scale + static_cast<long long>(kvh) * D + d0;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const float sd = __bfloat162float(s[j]);
      v[j] = kind == 1 ? v[j] * sd : v[j] / sd;
    }
  }

  if (kind == 0) {
    __nv_bfloat16* dst = p.q_out + (static_cast<long long>(t) * p.n_q_heads + h) * D + d0;
    uint32_t packed[VPL / 2];
#pragma unroll
    for (int j = 0; j < VPL / 2; ++j) packed[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    if (VPL == 8) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(packed);
    else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(packed);
    return;
  }

  // ---- K / V: quantise-append into the page that owns this token ----
  const int seq = p.token_seq[t];
  const int pos = p.cache_pos[t];
  if (seq < 0 || pos < 0) return;  // padded token
  const int page = p.block_table[static_cast<long long>(seq) * p.table_stride + pos / p.kv.page_size];
  if (page < 0) return;
  const long long rt = kv_row_of(p.kv, page, h, pos % p.kv.page_size);
  if (rt < 0) return;
  // a mixed layer appends into whatever tier the page's cell is in (new pages start in the hot tier)
  const int tier = p.kv.format == kKvMixed ? kv_row_tier(rt) : 0;
  const long long r = p.kv.format == kKvMixed ? kv_row_index(rt) : rt;
  const int fmt = p.kv.format == kKvMixed ? kv_tier_format(tier) : p.kv.format;
  const int group = p.kv.format == kKvMixed ? kv_tier_group(tier, D) : p.kv.group;
  const int rb = kv_row_bytes(fmt, D), sb = kv_scale_bytes(fmt, D, group);
  uint8_t* cbase = p.kv.format == kKvMixed ? (kind == 1 ? p.kv.tier_k_codes[tier] : p.kv.tier_v_codes[tier])
                                           : (kind == 1 ? p.kv.k_codes : p.kv.v_codes);
  uint8_t* sbase = p.kv.format == kKvMixed ? (kind == 1 ? p.kv.tier_k_scales[tier] : p.kv.tier_v_scales[tier])
                                           : (kind == 1 ? p.kv.k_scales : p.kv.v_scales);
  uint8_t* codes = cbase + r * rb;
  uint8_t* scales = sb ? sbase + r * sb : nullptr;
  // K is stored from its bf16-rounded value so that bf16 KV is a bit copy of what attention would see.
#pragma unroll
  for (int j = 0; j < VPL; ++j) v[j] = __bfloat162float(__float2bfloat16(v[j]));
  kv_store_row_warp<VPL>(fmt, group, v, codes, scales, lane);
}

}  // namespace

const char* attn_prep(const AttnPrepParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0) return nullptr;
  if (p.head_dim != 256 && p.head_dim != 128) return "attn_prep: head_dim must be 128 or 256";
  const int vpl = p.head_dim / 32;
  // each lane loads its vpl values with one vector load: rows and column offsets must keep that alignment
  if (p.ld_proj % vpl || p.q_off % vpl || p.k_off % vpl || p.v_off % vpl ||
      (reinterpret_cast<uintptr_t>(p.proj) % (2 * vpl)))
    return "attn_prep: projection rows must be aligned to head_dim/32 elements";
  if (p.rot_dim % (2 * vpl)) return "attn_prep: rot_dim/2 must be a multiple of head_dim/32";
  if (p.kv.format == kKvInt8Group && (p.kv.group % vpl || p.head_dim % p.kv.group)) return "attn_prep: bad int8 group";
  const int rows = p.T * (p.n_q_heads + 2 * p.n_kv_heads);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((rows + 3) / 4); cfg.blockDim = dim3(128); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = p.head_dim == 256 ? cudaLaunchKernelEx(&cfg, attn_prep_kernel<8>, p)
                                    : cudaLaunchKernelEx(&cfg, attn_prep_kernel<4>, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
