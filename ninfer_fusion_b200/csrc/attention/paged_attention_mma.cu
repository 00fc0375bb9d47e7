// Tensor-core split-KV paged attention for decode / small-T verify, head_dim 256.
//
// Work item = (query token, kv head, key split), 8 warps.  The GQA group's query
// heads are the M rows of a 16-row MMA tile.  Per 64-key tile:
//   1. all threads gather the tile's raw K / V rows from their pages (16-byte
//      coalesced loads), dequantise (bf16 / fp8-row / int8-group / nvfp4) and
//      store fp16 into shared memory, K and V both as [key][d] rows (16-byte
//      stores): K is a plain ldmatrix B operand, V goes through ldmatrix.trans;
//   2. warp w computes S = Q K^T for keys 8w..8w+7 (mma.sync m16n8k16 f16),
//      applies the per-row K scale, masks, and publishes its row maxima;
//   3. a tile-wide running max gives P = exp2(S - m); P (times the per-row V
//      scale) goes to shared memory as fp16;
//   4. warp w accumulates O[:, 32w..32w+31] += P V over the tile's 64 keys.
// Eight warps on a 64-key tile (rather than four) halve each thread's serial dequantisation work and double the
// warps per SM that cover shared-memory latency: the kernel is bound by that latency, not by bandwidth.
// Splits cover absolute key ranges and tiles start at split boundaries, so the
// reduction order for a query depends only on key positions.  Output partials
// (m, l, un-normalised O) use the same layout as the SIMT kernel and are
// finished by the same merge kernel.
//
// mma.sync is the right tensor path here: the M dimension is the 3..8 query heads
// of one GQA group, far below the 64/128 rows a tcgen05 tile needs.
#include "attention.h"

#include <math_constants.h>

#include "../common/ptx.cuh"
#include "../kv/codec.cuh"
#include "attn_mma_common.cuh"

namespace nfb {

namespace {

using namespace attn_mma;

// Page-table look-ups and row-scale loads are a chain of dependent global loads; doing them for 512 keys at once
// (four keys per thread, all in flight together) takes that chain out of the per-tile critical path.
constexpr int kSuperKeys = 512;
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kUnits = kTileKeys * 16 / kThreads;   // 16-value units of a K (or V) tile per thread

struct Smem {
  __half k[kTileKeys][kLdK];   // 33,792 B
  __half v[kTileKeys][kLdK];   // 33,792 B, row-major like K: the PV product reads it through ldmatrix.trans
  __half q[16][kLdQ];          //  8,448 B
  __half p[16][kLdP];          //  2,304 B
  float kscale[kSuperKeys];    // row scales and row indices of one super-tile of keys, looked up in one go
  float vscale[kSuperKeys];
  float rowmax[kWarps][16];
  float rowsum[kWarps][16];
  long long rowidx[kSuperKeys];
};

template <int FORMAT>
__global__ void __launch_bounds__(kThreads, 2) paged_attn_mma_kernel(const PagedAttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int kv_len = p.q_kv_len[t];
  const int seq = p.q_seq[t];
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

  // Q rows (g < G valid, rest zero), pre-scaled so that softmax runs on exp2
  const float qscale = p.sm_scale * 1.4426950408889634f;
  for (int i = threadIdx.x; i < 16 * (D / 2); i += blockDim.x) {
    const int g = i / (D / 2), d2 = i % (D / 2);
    float2 f = make_float2(0.f, 0.f);
    if (g < G) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(
          p.q + (static_cast<long long>(t) * p.n_q_heads + kvh * G + g) * D + 2 * d2);
      f = make_float2(__bfloat162float(v.x) * qscale, __bfloat162float(v.y) * qscale);
    }
    *reinterpret_cast<uint32_t*>(&sm.q[g][2 * d2]) = pack_half2(f.x, f.y);
  }

  const unsigned long long tmask = p.tree_mask ? p.tree_mask[t] : ~0ull;
  const int tbase = p.tree_mask ? p.tree_base[t] : 0x7fffffff;
  const int* table = p.block_table + static_cast<long long>(seq) * p.table_stride;
  const int P = p.kv.page_size;
  const int row0 = lane >> 2, cq = lane & 3;  // accumulator rows row0 / row0+8, column pair 2*cq

  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l_run[2] = {0.f, 0.f};
  float o[4][4];
#pragma unroll
  for (int n = 0; n < 4; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.f;

  // Raw (still quantised) K / V units of one tile, held in registers between their global loads and
  // their conversion into shared memory.  With a narrow KV format the next tile's loads are issued
  // before the current tile's math, so that their latency hides behind the MMAs; bf16 rows would
  // need twice the registers and keep the load-then-convert order.
  constexpr bool kPrefetch = FORMAT != kKvBf16 && FORMAT != kKvMixed;   // (a mixed unit may be a 32-byte bf16 one)
  RawUnit<FORMAT> rawk[kUnits], rawv[kUnits];

  auto gather_super = [&](int sb) {
    for (int i = threadIdx.x; i < kSuperKeys; i += blockDim.x) {
      const int key = sb + i;
      long long r = -1;
      float ks = 0.f, vs = 0.f;
      if (key < k_end) {
        const int page = table[key / P];
        // a released or unpublished page (-1) contributes nothing: no row, no scale read
        r = kv_row_of(p.kv, page, kvh, key % P);   // (mixed layers: the cell's tier rides in the top bits)
        if (FORMAT == kKvFp8Row && r >= 0) {
          ks = __half2float(reinterpret_cast<const __half*>(p.kv.k_scales)[r]);
          vs = __half2float(reinterpret_cast<const __half*>(p.kv.v_scales)[r]);
        } else if (FORMAT == kKvMixed && r >= 0 && kv_row_tier(r) == 1) {
          ks = __half2float(reinterpret_cast<const __half*>(p.kv.tier_k_scales[1])[kv_row_index(r)]);
          vs = __half2float(reinterpret_cast<const __half*>(p.kv.tier_v_scales[1])[kv_row_index(r)]);
        } else if (r >= 0) {
          ks = 1.f;
          vs = 1.f;
        }
      }
      sm.rowidx[i] = r;
      sm.kscale[i] = ks;
      sm.vscale[i] = vs;
    }
  };
  // K and V: unit = (key, part), 1024 units each, kUnits per thread; consecutive lanes read consecutive 16 values of a
  // row.  All of a thread's loads are in flight together.
  auto load_raw = [&](int off) {
#pragma unroll
    for (int it = 0; it < kUnits; ++it) {
      const int u = it * kThreads + threadIdx.x;
      const long long r = sm.rowidx[off + (u >> 4)];
      rawk[it].clear();
      if (r >= 0) rawk[it].load_row(p.kv, 0, r, u & 15);
    }
#pragma unroll
    for (int it = 0; it < kUnits; ++it) {
      const int u = it * kThreads + threadIdx.x;
      const long long r = sm.rowidx[off + (u >> 4)];
      rawv[it].clear();
      if (r >= 0) rawv[it].load_row(p.kv, 1, r, u & 15);
    }
  };
  // Dequantise to fp16, K and V both as [key][d] rows (16-byte stores, conflict-free with the 8-half row padding).
  auto store_tile = [&]() {
#pragma unroll
    for (int it = 0; it < kUnits; ++it) {
      const int u = it * kThreads + threadIdx.x;
      uint32_t h[8];
      rawk[it].convert(h);
      uint4* dst = reinterpret_cast<uint4*>(&sm.k[u >> 4][(u & 15) * 16]);
      dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
      dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
#pragma unroll
    for (int it = 0; it < kUnits; ++it) {
      const int u = it * kThreads + threadIdx.x;
      uint32_t h[8];
      rawv[it].convert(h);
      uint4* dst = reinterpret_cast<uint4*>(&sm.v[u >> 4][(u & 15) * 16]);
      dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
      dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
  };

  for (int sb = k_begin; sb < k_end; sb += kSuperKeys) {
  __syncthreads();  // the previous super-tile's index readers are done (also orders the Q stores on the first pass)
  gather_super(sb);
  __syncthreads();
  const int s_end = min(k_end, sb + kSuperKeys);
  if constexpr (kPrefetch) load_raw(0);
  for (int kb = sb; kb < s_end; kb += kTileKeys) {
    // ---- 1. dequantise the tile ----
    const int off = kb - sb;
    const bool has_next = kb + kTileKeys < s_end;
    __syncthreads();  // previous tile fully consumed
    if constexpr (kPrefetch) {
      store_tile();
      __syncthreads();
      if (has_next) load_raw(off + kTileKeys);  // in flight during this tile's math
    } else {
      load_raw(off);
      store_tile();
      __syncthreads();
    }
    const float* kscale = sm.kscale + off;
    const float* vscale = sm.vscale + off;

    // ---- 2. S = Q K^T for this warp's 16 keys ----
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const uint32_t q_addr = smem_u32(&sm.q[(lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
      // one ldmatrix.x4 brings this warp's 8 keys for two k-steps: d columns 0-7, 8-15, 16-23, 24-31 of the pair
      const uint32_t k_addr = smem_u32(&sm.k[warp * 8 + (lane & 7)][8 * (lane >> 3)]);
#pragma unroll 4
      for (int ks2 = 0; ks2 < D / 32; ++ks2) {
        uint32_t a0, a1, a2, a3, c0, c1, c2, c3, b0, b1, b2, b3;
        ldmatrix_x4(k_addr + ks2 * 64, b0, b1, b2, b3);
        ldmatrix_x4(q_addr + ks2 * 64, a0, a1, a2, a3);
        ldmatrix_x4(q_addr + ks2 * 64 + 32, c0, c1, c2, c3);
        mma_f16(s, a0, a1, a2, a3, b0, b1);
        mma_f16(s, c0, c1, c2, c3, b2, b3);
      }
    }
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kl = warp * 8 + 2 * cq + (j & 1);  // key inside the tile
      const int key = kb + kl;
      bool valid = key < k_end;
      if (valid && key >= tbase) valid = (tmask >> (key - tbase)) & 1ull;
      const float v = valid ? s[j] * kscale[kl] : -CUDART_INF_F;
      s[j] = v;
      mx[j >> 1] = fmaxf(mx[j >> 1], v);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    if (cq == 0) {
      sm.rowmax[warp][row0] = mx[0];
      sm.rowmax[warp][row0 + 8] = mx[1];
    }
    __syncthreads();

    // ---- 3. tile-wide running max, P to shared memory ----
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = row0 + 8 * h;
      float mt = sm.rowmax[0][r];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) mt = fmaxf(mt, sm.rowmax[w][r]);
      const float mn = fmaxf(m_run[h], mt);
      corr[h] = (mn == -CUDART_INF_F) ? 1.f : exp2f(m_run[h] - mn);
      m_run[h] = mn;
      l_run[h] *= corr[h];
    }
    {
      const int kl = warp * 8 + 2 * cq;
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float mn = m_run[j >> 1];
        pv[j] = (s[j] == -CUDART_INF_F) ? 0.f : exp2f(s[j] - mn);
        l_run[j >> 1] += pv[j];
        pv[j] *= vscale[kl + (j & 1)];
      }
      *reinterpret_cast<uint32_t*>(&sm.p[row0][kl]) = pack_half2(pv[0], pv[1]);
      *reinterpret_cast<uint32_t*>(&sm.p[row0 + 8][kl]) = pack_half2(pv[2], pv[3]);
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    __syncthreads();

    // ---- 4. O[:, 32*warp .. +31] += P V ----
    {
      const uint32_t p_addr = smem_u32(&sm.p[(lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
#pragma unroll
      for (int kk = 0; kk < kTileKeys / 16; ++kk) {
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4(p_addr + kk * 32, a0, a1, a2, a3);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          // V[key][d] is k x n row-major: the transposing ldmatrix yields the col-major B fragments
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(smem_u32(&sm.v[kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][warp * 32 + np * 16 + 8 * (lane >> 4)]),
                            b0, b1, b2, b3);
          mma_f16(o[2 * np], a0, a1, a2, a3, b0, b1);
          mma_f16(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
  }
  }

  // ---- row sums: quad reduce, then across warps ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  __syncthreads();
  if (cq == 0) {
    sm.rowsum[warp][row0] = l_run[0];
    sm.rowsum[warp][row0 + 8] = l_run[1];
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int g = row0 + 8 * h;
    if (g < G) {
      const long long pb = part_base + static_cast<long long>(g) * p.n_splits;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int d = warp * 32 + n * 8 + 2 * cq;
        *reinterpret_cast<float2*>(p.part_o + pb * D + d) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
      }
      if (warp == 0 && cq == 0) {
        p.part_ml[pb * 2] = m_run[h];
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tot += sm.rowsum[w][g];
        p.part_ml[pb * 2 + 1] = tot;
      }
    }
  }
}

template <int FORMAT>
cudaError_t launch_fmt(const PagedAttnParams& p, cudaStream_t stream, bool pdl) {
  auto kern = paged_attn_mma_kernel<FORMAT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(Smem));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.Tq, p.n_kv_heads, p.n_splits);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = sizeof(Smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

// Returns cudaErrorNotSupported when the geometry is outside this kernel (caller falls back to SIMT).
cudaError_t paged_attention_mma_split(const PagedAttnParams& p, cudaStream_t stream, bool pdl) {
  const int G = p.n_q_heads / p.n_kv_heads;
  if (p.head_dim != D || G > 16 || p.split_keys % kTileKeys) return cudaErrorNotSupported;
  if (p.kv.format == kKvInt8Group && (p.kv.group % 16)) return cudaErrorNotSupported;
  switch (p.kv.format) {
    case kKvBf16: return launch_fmt<kKvBf16>(p, stream, pdl);
    case kKvFp8Row: return launch_fmt<kKvFp8Row>(p, stream, pdl);
    case kKvInt8Group: return launch_fmt<kKvInt8Group>(p, stream, pdl);
    case kKvNvfp4: return launch_fmt<kKvNvfp4>(p, stream, pdl);
    case kKvMixed: return launch_fmt<kKvMixed>(p, stream, pdl);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace nfb
