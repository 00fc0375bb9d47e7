// Causal paged attention for prefill chunks and wide verify passes (head_dim 256), tensor cores.
//
// One CTA = one block of consecutive query tokens of one sequence x one KV head, 8 warps.  The M rows
// of the MMA tiles are (query token, query head of the GQA group) pairs: warp w owns rows 16w..16w+15
// for the whole key loop (flash-attention-2 layout: running max / sum / O stay in that warp's registers,
// P never leaves registers).  Per 64-key tile all threads gather the raw K / V rows from their pages,
// dequantise them ONCE for the whole query block (bf16 / fp8-row / int8-group / nvfp4 -> fp16) into
// shared memory (K as [key][d], V transposed and XOR-swizzled) and every warp runs
// S = Q K^T (128 mma), online softmax, O += P V (128 mma).  The epilogue normalises, applies the layer's
// sigmoid output gate and stores bf16.  K/V of the chunk itself were appended by attn_prep before this
// kernel runs, so the key loop simply covers [0, last visible key] with a per-row causal limit.
//
// Reference kernels covered: kernel/gqa_attention_prefill_{bf16,i8,nvfp4}.cuh (Br = 64 x Bc = 64
// mma.sync kernels that also quantise-append in-kernel).
#include "attention.h"

#include <math_constants.h>

#include "attn_mma_common.cuh"

namespace nfb {

namespace {

using namespace attn_mma;

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = kWarps * 16;  // query rows per CTA

struct PrefillSmem {
  __half k[kTileKeys][kLdK];
  __half vt[D][kLdV];
  __half q[kRows][kLdQ];
  // double buffered: while a tile is gathered and multiplied, the page rows and scales of the next one are looked up
  float kscale[2][kTileKeys];
  float vscale[2][kTileKeys];
  long long rowidx[2][kTileKeys];
};

template <int FORMAT>
__global__ void __launch_bounds__(kThreads, 1) paged_attn_prefill_kernel(const PrefillAttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(smem_raw);

  pdl_launch_next();
  pdl_wait_prior();
  // Longest first: a later query block of a causal prompt sees more keys, and CTAs are handed out in grid order, so
  // the grid runs the blocks from the last to the first (all KV heads of a block side by side); the short blocks
  // then fill the tail of the last wave instead of one long block running alone.
  const int kvh = blockIdx.x, blk = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int t0 = p.blk_start[blk];
  const int n_tok = p.blk_count[blk];
  if (n_tok <= 0) return;
  const int seq = p.q_seq[t0];
  if (seq < 0) return;
  const int k_end = p.q_kv_len[t0 + n_tok - 1];  // the last token of the block sees the most keys
  const int n_rows = n_tok * G;

  // ---- Q tile: row r = (token r / G, head r % G), pre-scaled for exp2 softmax ----
  const float qscale = p.sm_scale * 1.4426950408889634f;
  for (int i = threadIdx.x; i < kRows * (D / 2); i += kThreads) {
    const int r = i / (D / 2), d2 = i % (D / 2);
    float2 f = make_float2(0.f, 0.f);
    if (r < n_rows) {
      const int j = r / G, g = r % G;
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(
          p.q + (static_cast<long long>(t0 + j) * p.n_q_heads + kvh * G + g) * D + 2 * d2);
      f = make_float2(__bfloat162float(v.x) * qscale, __bfloat162float(v.y) * qscale);
    }
    *reinterpret_cast<uint32_t*>(&sm.q[r][2 * d2]) = pack_half2(f.x, f.y);
  }

  const int* table = p.block_table + static_cast<long long>(seq) * p.table_stride;
  const int P = p.kv.page_size;
  const int row0 = lane >> 2, cq = lane & 3;
  // causal limit of this thread's two rows (row0 and row0 + 8 of the warp's m-tile)
  int lim[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + row0 + 8 * h;
    lim[h] = r < n_rows ? p.q_kv_len[t0 + r / G] : 0;
  }
  // sliding window: row r sees keys [lim - window, lim); tiles entirely before the first token's window are skipped
  int lo[2] = {0, 0};
  int k_first = 0;
  if (p.window > 0) {
    lo[0] = max(0, lim[0] - p.window);
    lo[1] = max(0, lim[1] - p.window);
    k_first = max(0, p.q_kv_len[t0] - p.window) / kTileKeys * kTileKeys;
  }
  // keys this warp needs at all (rows of a warp are consecutive tokens): skip tiles beyond it
  const int warp_last_row = min(n_rows - 1, warp * 16 + 15);
  const int warp_k_end = warp * 16 < n_rows ? p.q_kv_len[t0 + warp_last_row / G] : 0;

  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l_run[2] = {0.f, 0.f};
  float o[32][4];
#pragma unroll
  for (int n = 0; n < 32; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.f;

  // page row and scales of one key of the tile starting at `kb`, written to buffer `b` (threads 0..63)
  auto lookup = [&](int kb, int b) {
    const int key = kb + threadIdx.x;
    long long r = -1;
    float ks = 0.f, vs = 0.f;
    if (key < k_end) {
      const int page = table[key / P];
      // a released or unpublished page (-1) contributes nothing: no row, no scale read
      r = kv_row_of(p.kv, page, kvh, key % P);   // (mixed layers: the cell's tier rides in the top bits)
      ks = r >= 0 ? 1.f : 0.f;
      vs = ks;
      if (FORMAT == kKvFp8Row && r >= 0) {
        ks = __half2float(reinterpret_cast<const __half*>(p.kv.k_scales)[r]);
        vs = __half2float(reinterpret_cast<const __half*>(p.kv.v_scales)[r]);
      } else if (FORMAT == kKvMixed && r >= 0 && kv_row_tier(r) == 1) {
        ks = __half2float(reinterpret_cast<const __half*>(p.kv.tier_k_scales[1])[kv_row_index(r)]);
        vs = __half2float(reinterpret_cast<const __half*>(p.kv.tier_v_scales[1])[kv_row_index(r)]);
      }
    }
    sm.rowidx[b][threadIdx.x] = r;
    sm.kscale[b][threadIdx.x] = ks;
    sm.vscale[b][threadIdx.x] = vs;
  };
  if (threadIdx.x < kTileKeys && k_first < k_end) lookup(k_first, 0);
  int buf = 0;
  for (int kb = k_first; kb < k_end; kb += kTileKeys, buf ^= 1) {
    __syncthreads();  // previous tile consumed; Q stores and this tile's look-up ordered
    {
      // K: 1024 units of 16 values, 4 per thread; V: 512 (key pair, part) units, 2 per thread.  All eight gathers
      // of a thread are issued before the first conversion, so a tile pays one L2 round trip instead of two (the
      // kernel is latency bound: 8 warps per SM, long scoreboard the top stall).  bf16 units are 32 bytes each, too
      // many registers to hold eight at once beside the 128 accumulator registers: that format loads K, then V.
      constexpr bool kTogether = FORMAT != kKvBf16 && FORMAT != kKvMixed;
      RawUnit<FORMAT> rk[4], rv[4];
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int u = it * kThreads + threadIdx.x;
        const long long r = sm.rowidx[buf][u >> 4];
        rk[it].clear();
        if (r >= 0) rk[it].load_row(p.kv, 0, r, u & 15);
      }
      auto load_v = [&]() {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int u = it * kThreads + threadIdx.x;
          const int jp = u >> 4, part = u & 15;
          const long long r0 = sm.rowidx[buf][2 * jp], r1 = sm.rowidx[buf][2 * jp + 1];
          rv[2 * it].clear();
          rv[2 * it + 1].clear();
          if (r0 >= 0) rv[2 * it].load_row(p.kv, 1, r0, part);
          if (r1 >= 0) rv[2 * it + 1].load_row(p.kv, 1, r1, part);
        }
      };
      if constexpr (kTogether) load_v();
      // the next tile's look-up (two dependent global reads) is issued behind this tile's gathers, so that it runs
      // beside them instead of in front of them
      if (threadIdx.x < kTileKeys && kb + kTileKeys < k_end) lookup(kb + kTileKeys, buf ^ 1);
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int u = it * kThreads + threadIdx.x;
        uint32_t h[8];
        rk[it].convert(h);
        uint4* dst = reinterpret_cast<uint4*>(&sm.k[u >> 4][(u & 15) * 16]);
        dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
        dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
      }
      if constexpr (!kTogether) load_v();
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int u = it * kThreads + threadIdx.x;
        const int jp = u >> 4, part = u & 15;
        uint32_t h0[8], h1[8];
        rv[2 * it].convert(h0);
        rv[2 * it + 1].convert(h1);
        const int col = (2 * jp) ^ ((part & 7) * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          *reinterpret_cast<uint32_t*>(&sm.vt[part * 16 + 2 * i][col]) = __byte_perm(h0[i], h1[i], 0x5410);
          *reinterpret_cast<uint32_t*>(&sm.vt[part * 16 + 2 * i + 1][col]) = __byte_perm(h0[i], h1[i], 0x7632);
        }
      }
    }
    __syncthreads();
    if (kb >= warp_k_end) continue;  // every key of this tile is in this warp's future (warp-uniform)

    // ---- S = Q K^T : 16 rows x 64 keys ----
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[n][j] = 0.f;
    {
      const uint32_t q_addr = smem_u32(&sm.q[warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
      const uint32_t k_addr = smem_u32(&sm.k[(lane & 7) + 8 * (lane >> 4)][8 * ((lane >> 3) & 1)]);
#pragma unroll 2
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4(q_addr + ks * 32, a0, a1, a2, a3);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(k_addr + np * 16 * kLdK * 2 + ks * 32, b0, b1, b2, b3);
          mma_f16(s[2 * np], a0, a1, a2, a3, b0, b1);
          mma_f16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    // ---- scale, causal mask, online softmax (rows live in one quad) ----
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kl = n * 8 + 2 * cq + (j & 1);
        const bool valid = kb + kl < lim[j >> 1] && kb + kl >= lo[j >> 1];
        const float v = valid ? s[n][j] * sm.kscale[buf][kl] : -CUDART_INF_F;
        s[n][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float mn = fmaxf(m_run[h], mx[h]);
      corr[h] = (mn == -CUDART_INF_F) ? 1.f : exp2f(m_run[h] - mn);
      m_run[h] = mn;
      l_run[h] *= corr[h];
    }
    uint32_t pa[8][2];  // P as fp16 pairs: pa[n][0] = row0 cols (2cq, 2cq+1), pa[n][1] = row0+8
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pv[j] = (s[n][j] == -CUDART_INF_F) ? 0.f : exp2f(s[n][j] - m_run[j >> 1]);
        l_run[j >> 1] += pv[j];
        pv[j] *= sm.vscale[buf][n * 8 + 2 * cq + (j & 1)];
      }
      pa[n][0] = pack_half2(pv[0], pv[1]);
      pa[n][1] = pack_half2(pv[2], pv[3]);
    }
#pragma unroll
    for (int n = 0; n < 32; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    // ---- O += P V : A fragments come straight from the S accumulators ----
#pragma unroll
    for (int kk = 0; kk < kTileKeys / 16; ++kk) {
      const uint32_t a0 = pa[2 * kk][0], a1 = pa[2 * kk][1], a2 = pa[2 * kk + 1][0], a3 = pa[2 * kk + 1][1];
#pragma unroll
      for (int np = 0; np < 16; ++np) {
        const int d = np * 16 + (lane & 7) + 8 * (lane >> 4);
        const int col = (kk * 16 + 8 * ((lane >> 3) & 1)) ^ (((d >> 4) & 7) * 8);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(smem_u32(&sm.vt[d][col]), b0, b1, b2, b3);
        mma_f16(o[2 * np], a0, a1, a2, a3, b0, b1);
        mma_f16(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }

  // ---- epilogue: normalise, gate, store ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    const int r = warp * 16 + row0 + 8 * h;
    if (r >= n_rows) continue;
    const int t = t0 + r / G, head = kvh * G + r % G;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    __nv_bfloat16* dst = p.out + (static_cast<long long>(t) * p.n_q_heads + head) * D;
    const __nv_bfloat16* gate = p.gate ? p.gate + static_cast<long long>(t) * p.ld_gate + head * D : nullptr;
#pragma unroll
    for (int n = 0; n < 32; ++n) {
      const int d = n * 8 + 2 * cq;
      float a = __bfloat162float(__float2bfloat16(o[n][2 * h] * inv));
      float b = __bfloat162float(__float2bfloat16(o[n][2 * h + 1] * inv));
      if (gate != nullptr) {
        const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(gate + d);
        a /= 1.f + __expf(-__bfloat162float(g2.x));
        b /= 1.f + __expf(-__bfloat162float(g2.y));
      }
      *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16x2(a, b);
    }
  }
}

template <int FORMAT>
cudaError_t launch_fmt(const PrefillAttnParams& p, cudaStream_t stream, bool pdl) {
  auto kern = paged_attn_prefill_kernel<FORMAT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(PrefillSmem));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_kv_heads, p.n_blocks);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = sizeof(PrefillSmem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

int prefill_attn_block_tokens(int n_q_heads, int n_kv_heads) {
  const int G = n_q_heads / n_kv_heads;
  return G > 0 && G <= kRows ? kRows / G : 0;
}

const char* paged_attention_prefill(const PrefillAttnParams& p, cudaStream_t stream, bool pdl) {
  if (p.n_blocks <= 0) return nullptr;
  if (p.head_dim != D) return "paged_attention_prefill: head_dim must be 256";
  if (p.n_q_heads % p.n_kv_heads) return "paged_attention_prefill: q heads must be a multiple of kv heads";
  if (p.kv.format == kKvInt8Group && (p.kv.group % 16)) return "paged_attention_prefill: int8 group must be a multiple of 16";
  cudaError_t e;
  switch (p.kv.format) {
    case kKvBf16: e = launch_fmt<kKvBf16>(p, stream, pdl); break;
    case kKvFp8Row: e = launch_fmt<kKvFp8Row>(p, stream, pdl); break;
    case kKvInt8Group: e = launch_fmt<kKvInt8Group>(p, stream, pdl); break;
    case kKvNvfp4: e = launch_fmt<kKvNvfp4>(p, stream, pdl); break;
    case kKvMixed: e = launch_fmt<kKvMixed>(p, stream, pdl); break;
    default: return "paged_attention_prefill: unknown KV format";
  }
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
