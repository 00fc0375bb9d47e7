// Groupwise-integer weight-streaming linear (Q4/Q5/Q6 g64, W8 g32) for 1..32 tokens: in-register dequant from the
// artifact's row-split planes into bf16 A fragments of mma.sync m16n8k16 (weights are the M side, tokens the N side).
//
// Why mma.sync and not tcgen05 here: the operand must be built in registers from packed codes (nibble plane + high-bit
// plane), and an UMMA A operand lives in shared memory or TMEM; at <= 32 tokens the kernel is bound by the weight
// stream (0.53-1.06 bytes per weight), not by tensor throughput.  Larger token counts take the tcgen05 GEMMs on
// re-encoded weights.
//
// Work split: a CTA of 8 warps owns ROWS = 16 * MT weight rows; warp w walks the 64-wide k blocks w, w + 8, ... and the
// eight partial tiles meet in shared memory.  Inside a k block, lane (g, t) of a warp holds rows g and g + 8 of each
// m16 tile and the 16 consecutive codes k = 16 t .. 16 t + 15 of the block (one 8-byte load per row).  A dot product
// does not care in which order k is visited, so the codes are fed to the MMA in the order the bit tricks produce them
// (code i and code i + 4 of a 32-bit word form one bf16 pair) and the activations are permuted to match.
#include "gemm_groupint.h"

#include <cstdint>
#include <cstdlib>

#include "../common/ptx.cuh"
#include "../common/tensor_map.h"

namespace nfb {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// (x & m) ^ c and a ^ (b & m) in one LOP3 each
__device__ __forceinline__ uint32_t and_xor(uint32_t x, uint32_t m, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(x), "r"(m), "r"(c));   // (a & b) ^ c
  return d;
}
__device__ __forceinline__ uint32_t xor_and(uint32_t a, uint32_t b, uint32_t m) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x78;" : "=r"(d) : "r"(a), "r"(b), "r"(m));   // a ^ (b & c)
  return d;
}

// Four bf16 pairs {code j, code j + 4}, j = 0..3, of the eight 4/5/6-bit two's-complement codes whose low nibbles are
// `w` and whose high bits are spread in `hs` (code i's extra bits at bit hb * i for i < 4, at 16 + hb * (i - 4) above).
// 0x4300 | v is the bf16 number 128 + v for v < 128; v = code ^ half is the code in offset binary.
template <int BITS>
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t hs, uint32_t (&p)[4]) {
  constexpr uint32_t half = 1u << (BITS - 1);
  constexpr uint32_t magic = 0x43004300u | half | (half << 16);
  constexpr uint32_t bias = magic;   // 128 + half as bf16 pair: (128 + (code ^ half)) - (128 + half) = code
  constexpr int hb = BITS - 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v = and_xor(w >> (4 * j), 0x000F000Fu, magic);
    if (hb > 0) {
      constexpr uint32_t hmask = ((1u << hb) - 1u) << 4;
      const int sh = 4 - hb * j;
      const uint32_t t = sh >= 0 ? (hs << sh) : (hs >> (-sh));
      v = xor_and(v, t, hmask | (hmask << 16));
    }
    p[j] = sub_bf16x2(v, bias);
  }
}

// two int8 codes (bytes sel0, sel1 of w ^ 0x80808080) -> bf16 pair, through the fp32 form 2^23 + v
__device__ __forceinline__ uint32_t int8_pair(uint32_t wx, uint32_t sel0, uint32_t sel1) {
  const float f0 = __uint_as_float(__byte_perm(wx, 0x4B000000u, sel0)) - 8388736.f;   // 2^23 + 128
  const float f1 = __uint_as_float(__byte_perm(wx, 0x4B000000u, sel1)) - 8388736.f;
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(f1), "f"(f0));
  return d;
}

template <int FMT, int MT>
struct Frag {
  static constexpr int H = FMT == kW8G32 ? 2 : 1;
  uint2 a[MT][2][H];
  uint32_t hi[MT][2];
  float s[MT][2][H];
};

constexpr int kStages = 4;        // TMA ring depth per warp
constexpr int kBoxBytes = 32;     // bytes of one weight row in a TMA box: 64 four-bit codes or 32 eight-bit codes

// dynamic shared memory of the TMA variant: per-warp rings (the cross-warp reduction reuses them), the CTA's scale
// rows, the ring barriers
__host__ __device__ constexpr int ring_bytes(int rows, int boxes) { return kWarps * kStages * boxes * rows * kBoxBytes; }
__host__ __device__ constexpr int red_bytes(int rows, int cols) { return kWarps * rows * (cols + 1) * 4; }
__host__ __device__ constexpr int max_i(int a, int b) { return a > b ? a : b; }

// TMA = true (Q4 and W8): every warp keeps its own ring of kStages k blocks in shared memory, filled by 2-D bulk
// tensor copies of [ROWS x 32 bytes] boxes that one lane issues and an mbarrier per slot completes; the fragments are
// then read from shared memory without bank conflicts (a box is 32 bytes wide, so the eight rows of a fragment load
// are 256 consecutive bytes).  This takes the weight stream off the load/store unit, which the register variant
// saturates with one 128-byte line per row and load.  No cluster multicast: every CTA loads its own rows.
template <int FMT, int MT, int NT, bool TMA>
__global__ void __launch_bounds__(kThreads) groupint_linear_kernel(const GroupIntLinearParams p,
                                                                   const __grid_constant__ CUtensorMap tm0,
                                                                   const __grid_constant__ CUtensorMap tm1) {
  constexpr int ROWS = 16 * MT;
  constexpr int COLS = 8 * NT;
  constexpr int BITS = FMT == kQ4G64 ? 4 : FMT == kQ5G64 ? 5 : FMT == kQ6G64 ? 6 : 8;
  constexpr int hb = BITS == 8 ? 0 : BITS - 4;
  static_assert(!TMA || hb == 0, "the TMA variant covers the formats without a high-bit plane");
  __shared__ float red_static[TMA ? 1 : kWarps * ROWS * (COLS + 1)];
  extern __shared__ __align__(128) uint8_t dyn[];
  float (*red)[ROWS][COLS + 1] = reinterpret_cast<float (*)[ROWS][COLS + 1]>(TMA ? reinterpret_cast<float*>(dyn) : red_static);

  const GroupIntWeight& W = p.w[blockIdx.y];
  const int r0 = blockIdx.x * ROWS;
  if (r0 >= W.N) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nblk = p.K >> 6;
  const int64_t base_pitch = BITS == 8 ? p.Kp : p.Kp / 2;
  const int64_t high_pitch = static_cast<int64_t>(p.Kp) * hb / 8;
  const int scale_pitch = BITS == 8 ? p.Kp / 32 : p.Kp / 64;

  auto load = [&](Frag<FMT, MT>& f, int blk) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int64_t row = r0 + mt * 16 + g + 8 * r;
        if constexpr (BITS == 8) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            f.a[mt][r][h] = __ldg(reinterpret_cast<const uint2*>(W.base + row * base_pitch + 64 * blk + 32 * h + 8 * t));
            f.s[mt][r][h] = __half2float(__ldg(W.scale + row * scale_pitch + 2 * blk + h));
          }
        } else {
          f.a[mt][r][0] = __ldg(reinterpret_cast<const uint2*>(W.base + row * base_pitch + 32 * blk + 8 * t));
          f.s[mt][r][0] = __half2float(__ldg(W.scale + row * scale_pitch + blk));
          if constexpr (hb == 1)
            f.hi[mt][r] = __ldg(reinterpret_cast<const uint16_t*>(W.high + row * high_pitch + 8 * blk + 2 * t));
          if constexpr (hb == 2)
            f.hi[mt][r] = __ldg(reinterpret_cast<const uint32_t*>(W.high + row * high_pitch + 16 * blk + 4 * t));
        }
      }
  };

  // activation rows of this lane's token column (column g of each n8 tile); tokens past T repeat the last one
  const __nv_bfloat16* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = min(nt * 8 + g, p.T - 1);
    xrow[nt] = p.x + static_cast<int64_t>(tok) * p.ldx;
  }

  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[mt][nt][c] = 0.f;

  // the lane's activations of one k block: [half][token tile] x 8 consecutive k (see the fragment order above)
  auto load_x = [&](int blk, uint4 (&xq)[2][NT]) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int k0 = BITS == 8 ? 64 * blk + 32 * h + 8 * t : 64 * blk + 16 * t + 8 * h;
        xq[h][nt] = __ldg(reinterpret_cast<const uint4*>(xrow[nt] + k0));
      }
  };

  auto compute = [&](const Frag<FMT, MT>& f, const uint4 (&xq)[2][NT]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {       // Q formats: h = 32-bit word of the lane's 16 codes; W8: h = group of 32
      // B fragments of both MMA steps of this half, per token tile
      uint32_t b[NT][2][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 xv = xq[h][nt];
        if constexpr (BITS == 8) {
          b[nt][0][0] = xv.x; b[nt][0][1] = xv.y; b[nt][1][0] = xv.z; b[nt][1][1] = xv.w;
        } else {
          b[nt][0][0] = __byte_perm(xv.x, xv.z, 0x5410); b[nt][0][1] = __byte_perm(xv.x, xv.z, 0x7632);
          b[nt][1][0] = __byte_perm(xv.y, xv.w, 0x5410); b[nt][1][1] = __byte_perm(xv.y, xv.w, 0x7632);
        }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t pa[2][4];   // [row half][pair]
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          if constexpr (BITS == 8) {
            const uint2 c = f.a[mt][r][h];
            const uint32_t w0 = c.x ^ 0x80808080u, w1 = c.y ^ 0x80808080u;
            pa[r][0] = int8_pair(w0, 0x7650, 0x7651); pa[r][1] = int8_pair(w0, 0x7652, 0x7653);
            pa[r][2] = int8_pair(w1, 0x7650, 0x7651); pa[r][3] = int8_pair(w1, 0x7652, 0x7653);
          } else {
            const uint32_t w = h == 0 ? f.a[mt][r][0].x : f.a[mt][r][0].y;
            uint32_t hs = 0;
            if constexpr (hb == 1) {
              const uint32_t hbits = (f.hi[mt][r] >> (8 * h)) & 0xFFu;
              hs = (hbits | (hbits << 12)) & 0x000F000Fu;
            }
            if constexpr (hb == 2) {
              const uint32_t hbits = (f.hi[mt][r] >> (16 * h)) & 0xFFFFu;
              hs = __byte_perm(hbits, 0u, 0x4140);
            }
            dequant_word<BITS == 8 ? 4 : BITS>(w, hs, pa[r]);
          }
        }
        if constexpr (BITS == 8) {
          // one scale group per h: accumulate its two steps apart, then scale rows g and g + 8
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            float tmp[4] = {0.f, 0.f, 0.f, 0.f};
            mma_bf16(tmp, pa[0][0], pa[1][0], pa[0][1], pa[1][1], b[nt][0][0], b[nt][0][1]);
            mma_bf16(tmp, pa[0][2], pa[1][2], pa[0][3], pa[1][3], b[nt][1][0], b[nt][1][1]);
            acc[mt][nt][0] += f.s[mt][0][h] * tmp[0]; acc[mt][nt][1] += f.s[mt][0][h] * tmp[1];
            acc[mt][nt][2] += f.s[mt][1][h] * tmp[2]; acc[mt][nt][3] += f.s[mt][1][h] * tmp[3];
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            float tmp[4] = {0.f, 0.f, 0.f, 0.f};
            mma_bf16(tmp, pa[0][0], pa[1][0], pa[0][1], pa[1][1], b[nt][0][0], b[nt][0][1]);
            mma_bf16(tmp, pa[0][2], pa[1][2], pa[0][3], pa[1][3], b[nt][1][0], b[nt][1][1]);
            acc[mt][nt][0] += f.s[mt][0][0] * tmp[0]; acc[mt][nt][1] += f.s[mt][0][0] * tmp[1];
            acc[mt][nt][2] += f.s[mt][1][0] * tmp[2]; acc[mt][nt][3] += f.s[mt][1][0] * tmp[3];
          }
        }
      }
    }
  };

  // One k block requested ahead of the one being multiplied.  Requesting four ahead did not help (measured): the
  // kernel is held by the load/store unit (8 distinct 128-byte lines per warp-wide load: one per weight row) and by
  // the 1.5-2 integer operations per dequantised weight, not by the depth of its DRAM queue.
  if constexpr (!TMA) {
    Frag<FMT, MT> cur, nxt;
    int blk = warp;
    if (blk < nblk) load(cur, blk);
    for (; blk < nblk; blk += kWarps) {
      const int nb = blk + kWarps;
      if (nb < nblk) load(nxt, nb);
      uint4 xq[2][NT];
      load_x(blk, xq);
      compute(cur, xq);
      cur = nxt;
    }
  } else {
    constexpr int NB = Frag<FMT, MT>::H;                 // boxes per k block: W8 has two groups of 32 codes
    constexpr int BOX = ROWS * kBoxBytes;
    constexpr int RING = ring_bytes(ROWS, NB);
    constexpr int FRONT = max_i(RING, red_bytes(ROWS, COLS));
    __shared__ int abort_flag;
    const int spitch = scale_pitch + 2;                  // halves; two spare so that rows start in different banks
    __half* sc = reinterpret_cast<__half*>(dyn + FRONT);
    uint64_t* bars = reinterpret_cast<uint64_t*>(dyn + FRONT + ((ROWS * spitch * 2 + 15) / 16) * 16);
    uint8_t* my_ring = dyn + warp * (kStages * NB * BOX);
    for (int i = threadIdx.x; i < ROWS * scale_pitch; i += kThreads) {
      const int r = i / scale_pitch, c = i - r * scale_pitch;
      sc[r * spitch + c] = r0 + r < W.N ? __ldg(W.scale + static_cast<int64_t>(r0 + r) * scale_pitch + c) : __float2half(0.f);
    }
    if (threadIdx.x == 0) abort_flag = 0;
    if (lane == 0) {
#pragma unroll
      for (int st = 0; st < kStages; ++st) mbar_init(smem_u32(&bars[warp * kStages + st]), 1);
      mbar_fence_init();
    }
    __syncthreads();
    const CUtensorMap* tm = blockIdx.y == 0 ? &tm0 : &tm1;
    const uint64_t policy = l2_policy_evict_first();     // weights are read once per launch
    auto issue = [&](int slot, int blk) {                // one lane
      const uint32_t bar = smem_u32(&bars[warp * kStages + slot]);
      mbar_expect_tx(bar, NB * BOX);
#pragma unroll
      for (int b = 0; b < NB; ++b)
        tma_load_2d(smem_u32(my_ring + (slot * NB + b) * BOX), tm, bar, BITS == 8 ? 64 * blk + 32 * b : 32 * blk, r0, policy);
    };
    const int n_my = warp < nblk ? (nblk - warp + kWarps - 1) / kWarps : 0;
    if (lane == 0)
      for (int st = 0; st < kStages && st < n_my; ++st) issue(st, warp + st * kWarps);
    __syncwarp();
    for (int i = 0; i < n_my; ++i) {
      const int slot = i % kStages, blk = warp + i * kWarps;
      // bounded: a copy that never lands sets the status word and the CTA unwinds instead of spinning
      if (!mbar_wait(smem_u32(&bars[warp * kStages + slot]), (i / kStages) & 1, &abort_flag, p.status, kStatusTmaWaitTimeout)) break;
      Frag<FMT, MT> f;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int row = mt * 16 + g + 8 * r;
#pragma unroll
          for (int h = 0; h < NB; ++h) {
            f.a[mt][r][h] = *reinterpret_cast<const uint2*>(my_ring + (slot * NB + h) * BOX + row * kBoxBytes + 8 * t);
            f.s[mt][r][h] = __half2float(sc[row * spitch + (BITS == 8 ? 2 * blk + h : blk)]);
          }
        }
      __syncwarp();
      if (lane == 0 && i + kStages < n_my) {
        fence_proxy_async_smem();                        // the slot's reads above are ordered before the refill
        issue(slot, warp + (i + kStages) * kWarps);
      }
      // (fetching the next block's activations a block ahead was tried: no gain up to 16 tokens, a loss at 32 from
      // the 32 extra registers)
      uint4 xq[2][NT];
      load_x(blk, xq);
      compute(f, xq);
    }
    __syncthreads();                                     // every ring is drained before the reduction reuses the space
  }

#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) red[warp][mt * 16 + g + (c >= 2 ? 8 : 0)][nt * 8 + 2 * t + (c & 1)] = acc[mt][nt][c];
  __syncthreads();
  const bool add = p.resid != nullptr && blockIdx.y == 0;
  for (int idx = threadIdx.x; idx < ROWS * p.T; idx += kThreads) {
    const int row = idx % ROWS, tok = idx / ROWS;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += red[w][row][tok];
    if (add) v += __bfloat162float(p.resid[static_cast<int64_t>(tok) * p.ldr + r0 + row]);
    W.out[static_cast<int64_t>(tok) * W.ldo + r0 + row] = __float2bfloat16(v);
  }
}

bool tma_enabled() {
  static const bool on = [] { const char* e = std::getenv("NFB_GROUPINT_TMA"); return !(e && e[0] == '0'); }();
  return on;
}

template <int FMT, int MT, int NT, bool TMA>
const char* launch_one(const GroupIntLinearParams& p, dim3 grid, cudaStream_t stream, const CUtensorMap& tm0, const CUtensorMap& tm1) {
  auto kernel = groupint_linear_kernel<FMT, MT, NT, TMA>;
  int dyn_bytes = 0;
  if (TMA) {
    constexpr int ROWS = 16 * MT;
    constexpr int NB = FMT == kW8G32 ? 2 : 1;
    const int scale_pitch = FMT == kW8G32 ? p.Kp / 32 : p.Kp / 64;
    dyn_bytes = max_i(ring_bytes(ROWS, NB), red_bytes(ROWS, 8 * NT)) + ((ROWS * (scale_pitch + 2) * 2 + 15) / 16) * 16 +
                kWarps * kStages * 8;
    if (dyn_bytes > 200 * 1024) return "groupint_linear: K is too large for the shared-memory scale rows";
    static int configured = 0;   // per instantiation: the largest size the attribute was raised to
    if (dyn_bytes > configured) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_bytes) != cudaSuccess)
        return "groupint_linear: cannot raise the dynamic shared memory limit";
      configured = dyn_bytes;
    }
  }
  kernel<<<grid, kThreads, dyn_bytes, stream>>>(p, tm0, tm1);
  return cudaGetLastError() == cudaSuccess ? nullptr : "groupint_linear: launch failed";
}

template <int FMT, int MT, bool TMA>
const char* launch_nt(const GroupIntLinearParams& p, dim3 grid, cudaStream_t stream, const CUtensorMap& tm0, const CUtensorMap& tm1) {
  if (p.T <= 8) return launch_one<FMT, MT, 1, TMA>(p, grid, stream, tm0, tm1);
  if (p.T <= 16) return launch_one<FMT, MT, 2, TMA>(p, grid, stream, tm0, tm1);
  return launch_one<FMT, MT, 4, TMA>(p, grid, stream, tm0, tm1);
}

template <int FMT>
const char* launch_mt(const GroupIntLinearParams& p, cudaStream_t stream) {
  int n_max = p.w[0].N;
  if (p.n_weights == 2 && p.w[1].N > n_max) n_max = p.w[1].N;
  // 32-row tiles reuse each activation fragment twice; 16-row tiles double the CTA count when rows are scarce
  const bool wide = n_max % 32 == 0 && (n_max / 32) * p.n_weights >= 2 * 148;
  const dim3 grid(wide ? n_max / 32 : n_max / 16, p.n_weights);
  CUtensorMap tm[2] = {};
  if constexpr (FMT == kQ4G64 || FMT == kW8G32) {
    bool ok = tma_enabled();
    const uint64_t pitch = FMT == kW8G32 ? p.Kp : p.Kp / 2;
    for (int i = 0; ok && i < p.n_weights; ++i)
      ok = (reinterpret_cast<uintptr_t>(p.w[i].base) & 15) == 0 &&
           make_tmap_2d(&tm[i], TmapDtype::U8, p.w[i].base, static_cast<uint64_t>(p.w[i].N), pitch, pitch, wide ? 32 : 16,
                        kBoxBytes, false);
    if (ok) {
      if (p.n_weights == 1) tm[1] = tm[0];
      return wide ? launch_nt<FMT, 2, true>(p, grid, stream, tm[0], tm[1]) : launch_nt<FMT, 1, true>(p, grid, stream, tm[0], tm[1]);
    }
  }
  return wide ? launch_nt<FMT, 2, false>(p, grid, stream, tm[0], tm[1]) : launch_nt<FMT, 1, false>(p, grid, stream, tm[0], tm[1]);
}

}  // namespace

const char* groupint_linear(const GroupIntLinearParams& p, cudaStream_t stream) {
  if (p.T < 1 || p.T > 32) return "groupint_linear: 1..32 tokens per launch";
  if (p.K <= 0 || p.K % 64 != 0) return "groupint_linear: K must be a positive multiple of 64";
  if (p.Kp != (p.K + 127) / 128 * 128) return "groupint_linear: Kp must be K rounded up to 128";
  if (p.n_weights < 1 || p.n_weights > 2) return "groupint_linear: one weight or a pair";
  if (p.ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(p.x) & 15) != 0) return "groupint_linear: x must be 16-byte aligned per row";
  for (int i = 0; i < p.n_weights; ++i) {
    const GroupIntWeight& w = p.w[i];
    if (w.N <= 0 || w.N % 16 != 0) return "groupint_linear: rows must be a multiple of 16";
    if (w.base == nullptr || w.scale == nullptr || w.out == nullptr) return "groupint_linear: missing plane";
    if ((reinterpret_cast<uintptr_t>(w.base) & 7) != 0 || (reinterpret_cast<uintptr_t>(w.scale) & 1) != 0)
      return "groupint_linear: planes must be 8-byte aligned";
    if ((p.fmt == kQ5G64 || p.fmt == kQ6G64) && (w.high == nullptr || (reinterpret_cast<uintptr_t>(w.high) & 3) != 0))
      return "groupint_linear: high-bit plane missing or misaligned";
  }
  switch (p.fmt) {
    case kQ4G64: return launch_mt<kQ4G64>(p, stream);
    case kQ5G64: return launch_mt<kQ5G64>(p, stream);
    case kQ6G64: return launch_mt<kQ6G64>(p, stream);
    case kW8G32: return launch_mt<kW8G32>(p, stream);
    default: return "groupint_linear: unknown format";
  }
}

}  // namespace nfb
