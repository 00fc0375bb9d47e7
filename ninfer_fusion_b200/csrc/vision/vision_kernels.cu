// Vision-tower row kernels and packed bidirectional attention (see vision.h).
#include "vision.h"

#include <math_constants.h>

#include "../common/ptx.cuh"

namespace nfb {

namespace {

// ------------------------------------------------------------------ layer norm
// One warp per row; the row lives in registers between the two statistics passes.
constexpr int kLnMaxPairs = 32;  // bf16 pairs per lane: rows of up to 2048 values

__global__ void __launch_bounds__(128) layer_norm_kernel(const LayerNormParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= p.T) return;
  const int pairs = p.D >> 1;
  const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(p.x + static_cast<long long>(row) * p.ldx);
  float2 v[kLnMaxPairs];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kLnMaxPairs; ++i) {
    const int c = i * 32 + lane;
    v[i] = make_float2(0.f, 0.f);
    if (c < pairs) {
      v[i] = __bfloat1622float2(x[c]);
      sum += v[i].x + v[i].y;
    }
  }
  const float mean = warp_sum(sum) / static_cast<float>(p.D);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < kLnMaxPairs; ++i) {
    const int c = i * 32 + lane;
    if (c < pairs) {
      const float a = v[i].x - mean, b = v[i].y - mean;
      sq += a * a + b * b;
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / static_cast<float>(p.D) + p.eps);
  const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(p.w);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(p.b);
  uint32_t* out = reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(row) * p.ldo);
#pragma unroll
  for (int i = 0; i < kLnMaxPairs; ++i) {
    const int c = i * 32 + lane;
    if (c < pairs) {
      const float2 wf = __bfloat1622float2(w[c]);
      const float2 bf = b ? __bfloat1622float2(b[c]) : make_float2(0.f, 0.f);
      out[c] = pack_bf16x2((v[i].x - mean) * rstd * wf.x + bf.x, (v[i].y - mean) * rstd * wf.y + bf.y);
    }
  }
}

// ------------------------------------------------------------------ position table
// Grid coordinate of patch index i in a grid of n positions, mapped onto the table's side.
__device__ __forceinline__ float table_coord(int i, int n, int side) {
  return n <= 1 ? 0.f : static_cast<float>(i) * static_cast<float>(side - 1) / static_cast<float>(n - 1);
}

__global__ void __launch_bounds__(192) vision_pos_embed_kernel(const VisionPosEmbedParams p) {
  const int patch = blockIdx.x;
  const int y = p.pos_yx[2 * patch], x = p.pos_yx[2 * patch + 1];
  const int h = p.grid_hw[2 * patch], w = p.grid_hw[2 * patch + 1];
  const float yf = table_coord(y, h, p.side), xf = table_coord(x, w, p.side);
  const int y0 = static_cast<int>(yf), x0 = static_cast<int>(xf);
  const int y1 = min(y0 + 1, p.side - 1), x1 = min(x0 + 1, p.side - 1);
  const float wy = yf - static_cast<float>(y0), wx = xf - static_cast<float>(x0);
  const float c00 = (1.f - wy) * (1.f - wx), c01 = (1.f - wy) * wx, c10 = wy * (1.f - wx), c11 = wy * wx;
  const int pairs = p.D >> 1;
  const __nv_bfloat162* t00 = reinterpret_cast<const __nv_bfloat162*>(p.table + static_cast<long long>(y0 * p.side + x0) * p.D);
  const __nv_bfloat162* t01 = reinterpret_cast<const __nv_bfloat162*>(p.table + static_cast<long long>(y0 * p.side + x1) * p.D);
  const __nv_bfloat162* t10 = reinterpret_cast<const __nv_bfloat162*>(p.table + static_cast<long long>(y1 * p.side + x0) * p.D);
  const __nv_bfloat162* t11 = reinterpret_cast<const __nv_bfloat162*>(p.table + static_cast<long long>(y1 * p.side + x1) * p.D);
  __nv_bfloat162* xr = reinterpret_cast<__nv_bfloat162*>(p.x + static_cast<long long>(patch) * p.D);
  for (int c = threadIdx.x; c < pairs; c += blockDim.x) {
    const float2 a = __bfloat1622float2(t00[c]), b = __bfloat1622float2(t01[c]);
    const float2 d = __bfloat1622float2(t10[c]), e = __bfloat1622float2(t11[c]);
    const float2 v = __bfloat1622float2(xr[c]);
    const float ox = v.x + (a.x * c00 + b.x * c01 + d.x * c10 + e.x * c11);
    const float oy = v.y + (a.y * c00 + b.y * c01 + d.y * c10 + e.y * c11);
    *reinterpret_cast<uint32_t*>(&xr[c]) = pack_bf16x2(ox, oy);
  }
}

// ------------------------------------------------------------------ 2-D rope
// Pair i of a head is (d = i, d = i + D/2); pairs [0, D/4) turn with the patch row, pairs [D/4, D/2) with the
// patch column, both over the ladder theta^(-2 j / (D/2)), j = i mod D/4.
__global__ void __launch_bounds__(192) vision_rope_kernel(const VisionRopeParams p) {
  const int patch = blockIdx.x;
  const int half = p.D >> 1, quarter = p.D >> 2;
  const float fy = static_cast<float>(p.pos_yx[2 * patch]), fx = static_cast<float>(p.pos_yx[2 * patch + 1]);
  __nv_bfloat16* row = p.qkv + static_cast<long long>(patch) * p.ld;
  const int items = 2 * p.H * half;  // q plane then k plane
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int plane = it / (p.H * half);
    const int r = it % (p.H * half);
    const int head = r / half, i = r % half;
    const int j = i % quarter;
    const float inv = exp2f(-2.f * static_cast<float>(j) / static_cast<float>(half) * log2f(p.theta));
    const float ang = (i < quarter ? fy : fx) * inv;
    float sn, cs;
    sincosf(ang, &sn, &cs);
    __nv_bfloat16* hp = row + (static_cast<long long>(plane) * p.H + head) * p.D;
    const float a = __bfloat162float(hp[i]), b = __bfloat162float(hp[i + half]);
    hp[i] = __float2bfloat16(a * cs - b * sn);
    hp[i + half] = __float2bfloat16(b * cs + a * sn);
  }
}

// ------------------------------------------------------------------ packed attention
constexpr int VD = kPackedAttnHeadDim;   // 72
constexpr int kKSteps = 5;               // k dimension padded to 80 for Q K^T
constexpr int kLd = 88;                  // row pitch in bf16: 176 B, so eight rows of an ldmatrix hit distinct banks
constexpr int kTile = kPackedAttnTile;   // 64
constexpr int kChunks = VD / 8;          // 16-byte chunks per row
constexpr int kNTilesO = VD / 8;         // 9 output n-tiles

struct PackedSmem {
  __nv_bfloat16 q[kTile][kLd];
  __nv_bfloat16 k[2][kTile][kLd];
  __nv_bfloat16 v[2][kTile][kLd];
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// CTA = 64 consecutive queries of one segment x one head, 4 warps of 16 query rows.  The segment's keys
// stream through a two-deep cp.async ring of 64-key tiles; S, P and O never leave the warp's registers.
__global__ void __launch_bounds__(128) packed_attention_kernel(const PackedAttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  PackedSmem& sm = *reinterpret_cast<PackedSmem*>(smem_raw);
  const int tile = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = p.tiles[3 * tile], seg_begin = p.tiles[3 * tile + 1], seg_end = p.tiles[3 * tile + 2];
  const int HD = p.H * VD;

  // columns 72..87 of every row are never written by the copies: clear them once, the Q K^T k loop reads up to 79
  {
    __nv_bfloat16(*rows)[kLd] = reinterpret_cast<__nv_bfloat16(*)[kLd]>(smem_raw);  // q, k[2], v[2]: 5 x 64 rows
    for (int i = threadIdx.x; i < 5 * kTile; i += blockDim.x) {
      *reinterpret_cast<uint4*>(rows[i] + VD) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(rows[i] + VD + 8) = make_uint4(0, 0, 0, 0);
    }
  }

  // rows past the segment are zero-filled (cp.async with zero source bytes from a clamped address)
  auto load_rows = [&](__nv_bfloat16(*dst)[kLd], int row0, int plane) {
    for (int i = threadIdx.x; i < kTile * kChunks; i += blockDim.x) {
      const int r = i / kChunks, c = i % kChunks;
      const int g = row0 + r;
      const bool ok = g < seg_end;
      const __nv_bfloat16* src = p.qkv + static_cast<long long>(ok ? g : seg_end - 1) * p.ld + plane * HD + head * VD + c * 8;
      cp_async_16(smem_u32(&dst[r][c * 8]), src, ok ? 16 : 0);
    }
  };
  load_rows(sm.q, q0, 0);
  load_rows(sm.k[0], seg_begin, 1);
  load_rows(sm.v[0], seg_begin, 2);
  cp_async_commit();

  const float sl2 = p.scale * 1.4426950408889634f;
  const int row0 = lane >> 2, cq = lane & 3;
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l_run[2] = {0.f, 0.f};
  float o[kNTilesO][4];
#pragma unroll
  for (int n = 0; n < kNTilesO; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.f;
  uint32_t qf[kKSteps][4];

  const int n_key_tiles = (seg_end - seg_begin + kTile - 1) / kTile;
  for (int kt = 0; kt < n_key_tiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < n_key_tiles) {
      load_rows(sm.k[buf ^ 1], seg_begin + (kt + 1) * kTile, 1);
      load_rows(sm.v[buf ^ 1], seg_begin + (kt + 1) * kTile, 2);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (kt == 0) {
      const uint32_t q_addr = smem_u32(&sm.q[warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) ldsm_x4(q_addr + ks * 32, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    // ---- S = Q K^T: 16 rows x 64 keys ----
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[n][j] = 0.f;
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      const uint32_t k_addr = smem_u32(&sm.k[buf][np * 16 + (lane & 7) + 8 * (lane >> 4)][8 * ((lane >> 3) & 1)]);
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(k_addr + ks * 32, b0, b1, b2, b3);
        mma_bf16(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
        mma_bf16(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
      }
    }

    // ---- online softmax (base 2) ----
    const int key0 = seg_begin + kt * kTile;
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = key0 + n * 8 + 2 * cq + (j & 1);
        const float v = key < seg_end ? s[n][j] * sl2 : -CUDART_INF_F;
        s[n][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float mn = fmaxf(m_run[h], mx[h]);   // finite: every tile holds at least one key of the segment
      corr[h] = exp2f(m_run[h] - mn);
      m_run[h] = mn;
      l_run[h] *= corr[h];
    }
    uint32_t pa[4][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      float e[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        e[j] = exp2f(s[n][j] - m_run[j >> 1]);
        l_run[j >> 1] += e[j];
      }
      pa[n >> 1][(n & 1) * 2] = pack_bf16x2(e[0], e[1]);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(e[2], e[3]);
    }
#pragma unroll
    for (int n = 0; n < kNTilesO; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int krow = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(smem_u32(&sm.v[buf][krow][np * 16 + 8 * (lane >> 4)]), b0, b1, b2, b3);
        mma_bf16(o[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
        mma_bf16(o[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
      }
      uint32_t b0, b1;
      ldsm_x2_trans(smem_u32(&sm.v[buf][krow][64]), b0, b1);
      mma_bf16(o[8], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
    }
    __syncthreads();  // this buffer is refilled two tiles from now
  }

  // ---- normalise and store ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    const int g = q0 + warp * 16 + row0 + 8 * h;
    if (g < seg_end) {
      const float inv = 1.f / l_run[h];
      __nv_bfloat16* dst = p.out + static_cast<long long>(g) * p.ldo + head * VD;
#pragma unroll
      for (int n = 0; n < kNTilesO; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * cq) = pack_bf16x2(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    }
  }
}

}  // namespace

const char* layer_norm(const LayerNormParams& p, cudaStream_t stream) {
  if (p.T <= 0) return nullptr;
  if (p.D % 2 || p.D > 64 * kLnMaxPairs) return "layer_norm: row width must be even and at most 2048";
  if ((p.ldx % 2) || (p.ldo % 2)) return "layer_norm: row pitches must be even";
  layer_norm_kernel<<<(p.T + 3) / 4, 128, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "layer_norm: launch failed";
}

const char* vision_pos_embed_add(const VisionPosEmbedParams& p, cudaStream_t stream) {
  if (p.P <= 0) return nullptr;
  if (p.D % 2 || p.side < 1) return "vision_pos_embed_add: bad shape";
  vision_pos_embed_kernel<<<p.P, 192, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "vision_pos_embed_add: launch failed";
}

const char* vision_rope(const VisionRopeParams& p, cudaStream_t stream) {
  if (p.P <= 0) return nullptr;
  if (p.D % 4) return "vision_rope: head_dim must be a multiple of 4";
  vision_rope_kernel<<<p.P, 192, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "vision_rope: launch failed";
}

const char* packed_attention(const PackedAttnParams& p, cudaStream_t stream) {
  if (p.n_tiles <= 0) return nullptr;
  if ((p.ld % 8) || (p.ldo % 2)) return "packed_attention: qkv rows must start on 16-byte boundaries";
  if ((reinterpret_cast<uintptr_t>(p.qkv) & 15) != 0) return "packed_attention: qkv must be 16-byte aligned";
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(packed_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(PackedSmem))) != cudaSuccess)
      return "packed_attention: cannot raise the shared-memory limit";
    attr_set = true;
  }
  packed_attention_kernel<<<dim3(p.n_tiles, p.H), 128, sizeof(PackedSmem), stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "packed_attention: launch failed";
}

}  // namespace nfb
