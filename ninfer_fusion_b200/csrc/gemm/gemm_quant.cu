// Weight-stationary GEMMs over quantised weights for sm_100a:  out[T, N] = x[T, K] * W[N, K]^T
//
//   kQFp8Row : W = e4m3 codes * fp32 row scale, activations quantised per token to e4m3
//              (tcgen05.mma kind::f8f6f4, scales applied in the epilogue);
//   kQNvfp4  : W = e2m1 codes * e4m3 scale per 16 values / d_w, activations quantised to the
//              same block format (tcgen05.mma kind::mxf4nvf4.block_scale: the scale factors
//              live in TMEM, copied there from shared memory with tcgen05.cp, and the tensor
//              core applies them per 16-element block).
//
// Shape of the kernel = the bf16 kernel (gemm_bf16.cu): 128 weight rows are the UMMA A operand,
// TN tokens the N operand, TMA -> 128B-swizzled shared memory (one k-block = 128 bytes of K:
// 128 fp8 or 256 fp4 values), accumulators in TMEM, tcgen05.ld epilogue with plain store,
// residual add or SwiGLU, optional in-cluster split-K through DSMEM.  For SwiGLU the weight rows
// are stored tile-interleaved ([64 gate rows ; 64 up rows] per 128-row tile) so that the scale
// planes stay ordinary 128-row tiles.
//
// The nvfp4 scale planes use the 128x4 tile order of the artifact format
// (docs/maintainer/storage-layouts.md:254-298): tile (row/128, k/64) holds 512 bytes,
// byte (r%32)*16 + (r/32)*4 + j = scale of row r, 16-value block j.  That is exactly the image
// tcgen05.cp.32x128b.warpx4 expects, so a tile goes global -> shared (bulk copy) -> TMEM untouched.
//
// Reference: src/ops/linear/nvfp4/nvfp4_w4a4_tma.cuh (mma.sync mxf4nvf4 on sm_120a, refused on
// sm_100a), src/ops/linear/fp8/fp8_a8_mma.cuh (mma.sync f8f6f4 with row-scale epilogue).
#include "gemm_quant.h"
#include "nvfp4_act.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "../kv/codec.cuh"

namespace nfb {

namespace {

constexpr int kTileN = 128;
constexpr int kKBytes = 128;  // bytes of K per k-block = one swizzle row
constexpr int kWTileBytes = kTileN * kKBytes;
constexpr int kSfTileBytes = 512;  // 128 rows x 4 scales

// DEEP = the whole grid fits in one wave: one CTA per SM with a deep pipeline.  Otherwise the pipeline is shallow
// enough for two CTAs per SM, so that a grid of up to two waves is resident at once.
template <int TN, int QT, bool DEEP>
struct QCfg {
  static constexpr bool kBlockScaled = QT == kQNvfp4;
  static constexpr int kXTileBytes = TN * kKBytes;
  static constexpr int kSfaBytes = kBlockScaled ? 4 * kSfTileBytes : 0;                     // 4 MMA-K steps per k-block
  static constexpr int kSfbBytes = kBlockScaled ? (TN <= 128 ? 4 : 8) * kSfTileBytes : 0;  // 1 or 2 token tiles
  static constexpr int kStageBytes = kWTileBytes + kXTileBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStages = TN <= 32 ? (DEEP ? 8 : 4) : (TN == 64 ? (DEEP ? 6 : 3) : (TN == 128 ? 5 : 3));
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kSfaCol = TN;           // TMEM columns: [0, TN) accumulator, then SFA, then SFB
  static constexpr int kSfbCol = TN + 16;
  static constexpr int kUsedCols = kBlockScaled ? TN + 16 + (TN <= 128 ? 16 : 32) : TN;
  static constexpr int kTmemCols = kUsedCols <= 32 ? 32 : (kUsedCols <= 64 ? 64 : (kUsedCols <= 128 ? 128 : (kUsedCols <= 256 ? 256 : 512)));
};

// Shared-memory descriptor of a 32-row x 16-byte scale image (no swizzle, rows 16 bytes apart,
// 8-row groups 128 bytes apart) for tcgen05.cp.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;  // SBO
  d |= static_cast<uint64_t>(1) << 46;         // descriptor version
  return d;
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
// Instruction descriptor of kind::mxf4nvf4: e2m1 x e2m1, ue4m3 scales, K-major, K = 64 per instruction.
__host__ __device__ constexpr uint32_t idesc_nvfp4(int M, int N) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}

struct QParams {
  int T, N, K;
  int num_kb, kb_per_split, cluster;
  int k_tiles;               // K / 64: scale tiles per row tile
  const uint8_t* w_sf;       // nvfp4: weight scale plane
  const uint8_t* x_sf;       // nvfp4: activation scale plane
  const float* w_scale;      // fp8: [N]
  const float* x_scale;      // fp8: [T]
  float out_scale;           // nvfp4: 1 / d_w
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* resid;
  long long ldr;
  int* status;
  // tensor-parallel epilogues (see gemm.h: kEpiPushPartial, kEpiPushAll)
  float* peer_recv[kMaxRanks];
  unsigned int* peer_flag[kMaxRanks];
  int rank, world, slice_cols, T_cap;
  const unsigned int* call_idx;
  // SwiGLU epilogue: also write the activation as the NEXT GEMM's nvfp4 operand (codes [T][N / 4], scale plane);
  // nullptr = bf16 output only
  uint8_t* next_codes;
  uint8_t* next_sf;
};

template <int TN, int QT, int EPI, bool DEEP>
__global__ void __launch_bounds__(128) gemm_q_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                                      const __grid_constant__ CUtensorMap tmap_x, const QParams p) {
  using Cfg = QCfg<TN, QT, DEEP>;
  constexpr int kStages = Cfg::kStages;
  constexpr bool kBS = Cfg::kBlockScaled;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_accum;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int peer_ok[8];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int t0 = blockIdx.y * TN;
  const int n0 = blockIdx.x * kTileN;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(p.num_kb, kb_begin + p.kb_per_split);
  const int num_it = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int r = 0; r < 8; ++r) peer_ok[r] = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_accum), 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_base_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_launch_next();

  if (warp == 0) {
    if (elect_one()) {
      // ---------------- TMA producer ----------------
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      bool waited_prior = false;
      int it = 0;
      for (; it < num_it; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (it >= kStages &&
            !mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, kStatusEmptyWaitTimeout))
          break;
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t dst = smem_base + s * Cfg::kStageBytes;
        const int kb = kb_begin + it;
        const int kx = kb * kKBytes;
        mbar_expect_tx(full, Cfg::kStageBytes);
        tma_load_2d(dst, &tmap_w, full, kx, n0, pol_w);
        tma_load_2d(dst + 64 * 128, &tmap_w, full, kx, n0 + 64, pol_w);
        if constexpr (kBS) {
          const uint8_t* sfa = p.w_sf + (static_cast<long long>(blockIdx.x) * p.k_tiles + 4 * kb) * kSfTileBytes;
          bulk_load(dst + kWTileBytes + Cfg::kXTileBytes, sfa, Cfg::kSfaBytes, full);
        }
        if (!waited_prior) {
          pdl_wait_prior();  // activations (and their scales) come from the previous kernel
          waited_prior = true;
        }
        tma_load_2d(dst + kWTileBytes, &tmap_x, full, kx, t0, pol_x);
        if constexpr (kBS) {
          const uint32_t sfb_dst = dst + kWTileBytes + Cfg::kXTileBytes + Cfg::kSfaBytes;
          const long long tile0 = t0 / 128;
          bulk_load(sfb_dst, p.x_sf + (tile0 * p.k_tiles + 4 * kb) * kSfTileBytes, 4 * kSfTileBytes, full);
          if constexpr (TN > 128)
            bulk_load(sfb_dst + 4 * kSfTileBytes, p.x_sf + ((tile0 + 1) * p.k_tiles + 4 * kb) * kSfTileBytes,
                      4 * kSfTileBytes, full);
        }
      }
      if (abort_flag) {
        const int first = it > kStages ? it - kStages : 0;
        for (int j = first; j < it; ++j) {
          const uint32_t bar = smem_u32(&bar_full[j % kStages]);
          const uint32_t ph = (j / kStages) & 1;
          for (uint32_t spin = 0; spin < (1u << 20); ++spin)
            if (mbar_try_wait(bar, ph)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = kBS ? idesc_nvfp4(kTileN, TN) : umma_idesc(kTileN, TN, 0, 0);
      bool ok = true;
      for (int it = 0; it < num_it; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag, p.status, kStatusTmaWaitTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
        const uint64_t a_desc = umma_desc_k_sw128(a_addr);
        const uint64_t b_desc = umma_desc_k_sw128(a_addr + kWTileBytes);
        if constexpr (kBS) {
          const uint32_t sfa_s = a_addr + kWTileBytes + Cfg::kXTileBytes;
          const uint32_t sfb_s = sfa_s + Cfg::kSfaBytes;
          constexpr int kSfbStep = TN <= 128 ? 4 : 8;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tc_cp_sf(tmem_base + Cfg::kSfaCol + 4 * k, sf_desc(sfa_s + k * kSfTileBytes));
            tc_cp_sf(tmem_base + Cfg::kSfbCol + kSfbStep * k, sf_desc(sfb_s + k * kSfTileBytes));
            if constexpr (TN > 128)
              tc_cp_sf(tmem_base + Cfg::kSfbCol + kSfbStep * k + 4, sf_desc(sfb_s + (4 + k) * kSfTileBytes));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_nvfp4(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + Cfg::kSfaCol + 4 * k,
                         tmem_base + Cfg::kSfbCol + kSfbStep * k, (it > 0 || k > 0) ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f8f6f4(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_empty[s]));
      }
      if (ok) tc_commit(smem_u32(&bar_accum));
    }
    __syncwarp();
  }

  // ---------------- epilogue ----------------
  pdl_wait_prior();
  bool have_acc = true;
  if (num_it > 0) have_acc = mbar_wait(smem_u32(&bar_accum), 0, &abort_flag, p.status, kStatusAccumWaitTimeout);
  tc_fence_after();
  int epilogue_ok = __syncthreads_and(have_acc && !abort_flag);
  const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  constexpr int kChunk = 16;

  // in-cluster split-K: peers hand their fp32 tiles to the leader through DSMEM (see gemm_bf16.cu)
  const int S = p.cluster;
  const uint32_t crank = S > 1 ? blockIdx.z : 0;
  const float* peer_s = reinterpret_cast<const float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
  if (S > 1) {
    cluster_sync_all();
    if (crank != 0) {
      if (epilogue_ok) {
        const uint32_t local = smem_base + ((crank - 1) * TN * 128 + warp * 32 + lane) * 4;
        const uint32_t remote = mapa_shared(local, 0);
        for (int c = 0; c < TN; c += kChunk) {
          uint32_t v[kChunk];
          tmem_ld_x16(lane_taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < kChunk; ++j) st_shared_cluster_u32(remote + (c + j) * 512, num_it > 0 ? v[j] : 0u);
        }
      }
      if (threadIdx.x == 0) st_shared_cluster_u32(mapa_shared(smem_u32(&peer_ok[crank]), 0), epilogue_ok ? 1u : 0u);
    }
    cluster_sync_all();
    if (crank != 0) {
      epilogue_ok = 0;
    } else {
      for (int r = 1; r < S; ++r) epilogue_ok &= peer_ok[r];
    }
  }
  const int n = n0 + warp * 32 + lane;
  float row_scale = kBS ? p.out_scale : ((n < p.N) ? p.w_scale[n] : 0.f);
  auto load_acc = [&](int c, float* acc) {
    uint32_t v[kChunk];
    tmem_ld_x16(lane_taddr + c, v);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < kChunk; ++j) acc[j] = num_it > 0 ? __uint_as_float(v[j]) : 0.f;
    for (int r = 1; r < S; ++r) {
#pragma unroll
      for (int j = 0; j < kChunk; ++j) acc[j] += peer_s[((r - 1) * TN + c + j) * 128 + warp * 32 + lane];
    }
#pragma unroll
    for (int j = 0; j < kChunk; ++j) {
      float sc = row_scale;
      if constexpr (!kBS) sc *= (t0 + c + j < p.T) ? p.x_scale[t0 + c + j] : 0.f;
      acc[j] *= sc;
    }
  };

  if (epilogue_ok) {
    if constexpr (EPI == kEpiSwiglu) {
      // rows are tile-interleaved: lanes 0..63 = gate rows, lanes 64..127 = the matching up rows
      float* up_s = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))) + (S - 1) * TN * 128;
      float* act_s = up_s + TN * 64;   // [TN][64] activations for the fused quantiser (behind the up rows)
      if (warp >= 2) {
        const int r = (warp - 2) * 32 + lane;
        for (int c = 0; c < TN; c += kChunk) {
          if (t0 + c >= p.T) break;
          float v[kChunk];
          load_acc(c, v);
#pragma unroll
          for (int j = 0; j < kChunk; ++j) up_s[(c + j) * 64 + r] = v[j];
        }
      }
      __syncthreads();
      if (warp < 2) {
        const int r = warp * 32 + lane;
        const int col = blockIdx.x * 64 + r;  // output column
        for (int c = 0; c < TN; c += kChunk) {
          if (t0 + c >= p.T) break;
          float v[kChunk];
          load_acc(c, v);
#pragma unroll
          for (int m = 0; m < kChunk / 2; ++m) {
            float a[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int j = 2 * m + h;
              const float g = v[j];
              a[h] = g / (1.f + __expf(-g)) * up_s[(c + j) * 64 + r];
            }
            if (p.next_codes != nullptr) {   // (same rounding as the bf16 store below: the quantiser reads bf16)
              act_s[(c + 2 * m) * 64 + r] = __bfloat162float(__float2bfloat16(a[0]));
              act_s[(c + 2 * m + 1) * 64 + r] = __bfloat162float(__float2bfloat16(a[1]));
            }
            const float send = (lane & 1) ? a[0] : a[1];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
            const int t = t0 + c + 2 * m + (lane & 1);
            const int ce = col & ~1;
            if (t < p.T && ce < p.N / 2) {
              const uint32_t packed = (lane & 1) ? pack_bf16x2(recv, a[1]) : pack_bf16x2(a[0], recv);
              *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.ldo + ce) = packed;
            }
          }
        }
      }
      if (p.next_codes != nullptr) {
        // the activation tile (TN tokens x 64 columns) as the next GEMM's nvfp4 operand: one (token, 16-column
        // block) per thread, the same bits the stand-alone quantiser would write from the bf16 tensor
        __syncthreads();
        const int K_next = p.N / 2;
        for (int u = threadIdx.x; u < TN * 4; u += 128) {
          const int tt = u >> 2, blk = u & 3;
          if (t0 + tt >= p.T) continue;
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = act_s[tt * 64 + blk * 16 + i];
          nvfp4_store_block(v, t0 + tt, blockIdx.x * 4 + blk, K_next, p.next_codes, p.next_sf);
        }
      }
    } else if constexpr (EPI == kEpiPushAll || EPI == kEpiPushPartial) {
      // the scaled fp32 tile goes to peer memory: to EVERY rank's [parity][src][T_cap][N] buffer (one-shot
      // all-reduce) or to the OWNER of this column slice [src][T][N/world] (reduce-scatter)
      for (int c = 0; c < TN; c += kChunk) {
        if (t0 + c >= p.T) break;
        float v[kChunk];
        load_acc(c, v);
        if constexpr (EPI == kEpiPushAll) {
          const unsigned int par = *p.call_idx & 1u;
          const long long base = ((static_cast<long long>(par) * p.world + p.rank) * p.T_cap) * p.N + n;
          for (int r = 0; r < p.world; ++r) {
            float* dst = p.peer_recv[r] + base;
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int t = t0 + c + j;
              if (t < p.T && n < p.N) dst[static_cast<long long>(t) * p.N] = v[j];
            }
          }
        } else {
          const int owner = n0 / p.slice_cols;
          float* dst = p.peer_recv[owner] + static_cast<long long>(p.rank) * p.T * p.slice_cols + (n - owner * p.slice_cols);
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const int t = t0 + c + j;
            if (t < p.T && n < p.N) dst[static_cast<long long>(t) * p.slice_cols] = v[j];
          }
        }
      }
      // the block barrier orders every thread's peer stores before the signalling threads, whose system-scope
      // fence + release is cumulative over them
      __syncthreads();
      if constexpr (EPI == kEpiPushAll) {
        if (threadIdx.x < p.world) {
          __threadfence_system();
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.peer_flag[threadIdx.x]) : "memory");
        }
      } else {
        if (threadIdx.x == 0) {
          __threadfence_system();
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.peer_flag[n0 / p.slice_cols]) : "memory");
        }
      }
    } else {
      for (int c = 0; c < TN; c += kChunk) {
        if (t0 + c >= p.T) break;
        float v[kChunk];
        load_acc(c, v);
        __nv_bfloat162 r2[kChunk / 2];
        if constexpr (EPI == kEpiResidual) {
#pragma unroll
          for (int m = 0; m < kChunk / 2; ++m) {
            const int t = t0 + c + 2 * m + (lane & 1);
            const int ne = n & ~1;
            r2[m] = (t < p.T && ne < p.N)
                        ? *reinterpret_cast<const __nv_bfloat162*>(p.resid + static_cast<long long>(t) * p.ldr + ne)
                        : __nv_bfloat162();
          }
        }
#pragma unroll
        for (int m = 0; m < kChunk / 2; ++m) {
          const float a0 = v[2 * m], a1 = v[2 * m + 1];
          const float send = (lane & 1) ? a0 : a1;
          const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
          const int t = t0 + c + 2 * m + (lane & 1);
          const int ne = n & ~1;
          if (t < p.T && ne < p.N) {
            float lo = (lane & 1) ? recv : a0;
            float hi = (lane & 1) ? a1 : recv;
            if constexpr (EPI == kEpiResidual) {
              lo += __bfloat162float(r2[m].x);
              hi += __bfloat162float(r2[m].y);
            }
            *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.ldo + ne) = pack_bf16x2(lo, hi);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// activation quantisers
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_act_fp8_kernel(const __nv_bfloat16* x, long long ldx, int K, uint8_t* codes,
                                                            float* scale) {
  __shared__ float red[8];
  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  const __nv_bfloat16* row = x + static_cast<long long>(t) * ldx;
  const int nvec = K / 8;
  float amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += 256) {
    const uint4 r = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(__bfloat162float(p2[i].x)), fabsf(__bfloat162float(p2[i].y))));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float sc = fmaxf(amax / 448.f, 1e-12f);
  if (threadIdx.x == 0) scale[t] = sc;
  for (int v = threadIdx.x; v < nvec; v += 256) {
    const uint4 r = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&r);
    uint2 o = make_uint2(0u, 0u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = float_to_e4m3(__fdiv_rn(__bfloat162float(p2[i].x), sc));
      const uint32_t hi = float_to_e4m3(__fdiv_rn(__bfloat162float(p2[i].y), sc));
      const uint32_t pair = lo | (hi << 8);
      if (i < 2) o.x |= pair << (16 * i); else o.y |= pair << (16 * (i - 2));
    }
    *reinterpret_cast<uint2*>(codes + static_cast<long long>(t) * K + v * 8) = o;
  }
}

__global__ void __launch_bounds__(256) quant_act_nvfp4_kernel(const __nv_bfloat16* x, long long ldx, int K, uint8_t* codes,
                                                              uint8_t* sf_plane) {
  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  const int g = blockIdx.y * 256 + threadIdx.x;  // 16-value block index
  if (g * 16 >= K) return;
  const __nv_bfloat16* src = x + static_cast<long long>(t) * ldx + g * 16;
  const uint4 r0 = *reinterpret_cast<const uint4*>(src);
  const uint4 r1 = *reinterpret_cast<const uint4*>(src + 8);
  float v[16];
  const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&r0);
  const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __bfloat162float(p0[i].x); v[2 * i + 1] = __bfloat162float(p0[i].y);
    v[8 + 2 * i] = __bfloat162float(p1[i].x); v[8 + 2 * i + 1] = __bfloat162float(p1[i].y);
  }
  nvfp4_store_block(v, t, g, K, codes, sf_plane);
}

// ------------------------------------------------------------------------------------------------------------
// Persistent prefill kernel for quantised weights: the same role split as the bf16 one (gemm_bf16.cu) -- warp 0 TMA,
// warp 1 MMA with the accumulator alternating between two TMEM column ranges, warps 2..5 epilogue -- so the epilogue
// of tile i overlaps the main loop of tile i + 1.  With fp8 / nvfp4 the main loop is 2-4 x shorter than in bf16 while
// the epilogue is the same size, so the one-tile-per-CTA kernel spends most of its time in epilogues.
//   fp8 row-scale: 256-token tiles, accumulators at TMEM columns [0, 256) and [256, 512)
//   nvfp4:         128-token tiles, accumulators at [0, 128) and [128, 256), scale factors at [256, 288)
template <int QT>
struct QPersist {
  static constexpr bool kBS = QT == kQNvfp4;
  static constexpr int TN = kBS ? 128 : 256;
  static constexpr int kXTileBytes = TN * kKBytes;
  static constexpr int kSfaBytes = kBS ? 4 * kSfTileBytes : 0;
  static constexpr int kSfbBytes = kBS ? 4 * kSfTileBytes : 0;
  static constexpr int kStageBytes = kWTileBytes + kXTileBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStages = kBS ? 5 : 4;
  static constexpr int kExchangeBytes = 2 * 16 * 64 * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kExchangeBytes + 1024;
  static constexpr int kSfaCol = 2 * TN;
  static constexpr int kSfbCol = 2 * TN + 16;
};
constexpr int kQPersistThreads = 192;

__device__ __forceinline__ void q_epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int QT, int EPI>
__global__ void __launch_bounds__(kQPersistThreads, 1) gemm_q_persist_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                                                              const __grid_constant__ CUtensorMap tmap_x,
                                                                              const QParams p) {
  static_assert(EPI == kEpiStore || EPI == kEpiResidual || EPI == kEpiSwiglu, "persistent kernel: plain epilogues only");
  using Cfg = QPersist<QT>;
  constexpr int TN = Cfg::TN;
  constexpr int kStages = Cfg::kStages;
  constexpr bool kBS = Cfg::kBS;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int epi_verdict[4];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int n_w_tiles = (p.N + kTileN - 1) / kTileN;
  const int n_t_tiles = (p.T + TN - 1) / TN;
  const int n_tiles = n_w_tiles * n_t_tiles;
  const int num_kb = p.num_kb;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_launch_next();

  if (warp == 0) {
    if (elect_one()) {
      // ---------------- TMA producer ----------------
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      bool waited_prior = false;
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !*abortp; tile += gridDim.x) {
        const int w_tile = tile / n_t_tiles;
        const int n0 = w_tile * kTileN;
        const int t0 = (tile % n_t_tiles) * TN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (it >= kStages &&
              !mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, kStatusEmptyWaitTimeout)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t dst = smem_base + s * Cfg::kStageBytes;
          const int kx = kb * kKBytes;
          mbar_expect_tx(full, Cfg::kStageBytes);
          tma_load_2d(dst, &tmap_w, full, kx, n0, pol_w);
          tma_load_2d(dst + 64 * 128, &tmap_w, full, kx, n0 + 64, pol_w);
          if constexpr (kBS) {
            const uint8_t* sfa = p.w_sf + (static_cast<long long>(w_tile) * p.k_tiles + 4 * kb) * kSfTileBytes;
            bulk_load(dst + kWTileBytes + Cfg::kXTileBytes, sfa, Cfg::kSfaBytes, full);
          }
          if (!waited_prior) {
            pdl_wait_prior();  // activations (and their scales) come from the previous kernel
            waited_prior = true;
          }
          tma_load_2d(dst + kWTileBytes, &tmap_x, full, kx, t0, pol_x);
          if constexpr (kBS) {
            const uint32_t sfb_dst = dst + kWTileBytes + Cfg::kXTileBytes + Cfg::kSfaBytes;
            const long long tile0 = t0 / 128;
            bulk_load(sfb_dst, p.x_sf + (tile0 * p.k_tiles + 4 * kb) * kSfTileBytes, 4 * kSfTileBytes, full);
          }
        }
        if (!ok) break;
      }
      if (*abortp) {
        const uint32_t first = it > kStages ? it - kStages : 0;
        for (uint32_t j = first; j < it; ++j) {
          const uint32_t bar = smem_u32(&bar_full[j % kStages]);
          const uint32_t ph = (j / kStages) & 1;
          for (uint32_t spin = 0; spin < (1u << 20); ++spin)
            if (mbar_try_wait(bar, ph)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = kBS ? idesc_nvfp4(kTileN, TN) : umma_idesc(kTileN, TN, 0, 0);
      uint32_t it = 0;
      int tile_i = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !*abortp; tile += gridDim.x, ++tile_i) {
        const int a = tile_i & 1;
        const uint32_t aph = (tile_i >> 1) & 1;
        if (tile_i >= 2 &&
            !mbar_wait(smem_u32(&bar_acc_empty[a]), aph ^ 1, &abort_flag, p.status, kStatusAccumWaitTimeout))
          break;
        tc_fence_after();
        const uint32_t acc = tmem_base + a * TN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag, p.status, kStatusTmaWaitTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
          const uint64_t a_desc = umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + kWTileBytes);
          if constexpr (kBS) {
            const uint32_t sfa_s = a_addr + kWTileBytes + Cfg::kXTileBytes;
            const uint32_t sfb_s = sfa_s + Cfg::kSfaBytes;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              tc_cp_sf(tmem_base + Cfg::kSfaCol + 4 * k, sf_desc(sfa_s + k * kSfTileBytes));
              tc_cp_sf(tmem_base + Cfg::kSfbCol + 4 * k, sf_desc(sfb_s + k * kSfTileBytes));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma_nvfp4(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + Cfg::kSfaCol + 4 * k,
                           tmem_base + Cfg::kSfbCol + 4 * k, (kb > 0 || k > 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma_f8f6f4(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(smem_u32(&bar_empty[s]));
        }
        if (!ok) break;
        tc_commit(smem_u32(&bar_acc_full[a]));
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps ----------------
    pdl_wait_prior();
    const int lg = warp & 3;
    constexpr int kChunk = 16;
    float* up_s = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)) + kStages * Cfg::kStageBytes);
    int tile_i = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_i) {
      const int a = tile_i & 1;
      const uint32_t ph = (tile_i >> 1) & 1;
      const bool have = mbar_wait(smem_u32(&bar_acc_full[a]), ph, &abort_flag, p.status, kStatusAccumWaitTimeout);
      if (lane == 0) epi_verdict[warp - 2] = (have && !*abortp) ? 1 : 0;
      q_epi_bar_sync();
      const bool go = epi_verdict[0] && epi_verdict[1] && epi_verdict[2] && epi_verdict[3];
      q_epi_bar_sync();
      if (!go) break;
      tc_fence_after();
      const int w_tile = tile / n_t_tiles;
      const int n0 = w_tile * kTileN;
      const int t0 = (tile % n_t_tiles) * TN;
      const uint32_t lane_taddr = tmem_base + a * TN + (static_cast<uint32_t>(lg * 32) << 16);
      const int n = n0 + lg * 32 + lane;
      const float row_scale = kBS ? p.out_scale : ((n < p.N) ? p.w_scale[n] : 0.f);
      auto load_acc = [&](int c, float* acc) {
        uint32_t v[kChunk];
        tmem_ld_x16(lane_taddr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < kChunk; ++j) {
          float sc = row_scale;
          if constexpr (!kBS) sc *= (t0 + c + j < p.T) ? p.x_scale[t0 + c + j] : 0.f;
          acc[j] = __uint_as_float(v[j]) * sc;
        }
      };
      if constexpr (EPI == kEpiSwiglu) {
        // rows are tile-interleaved: lane groups 0, 1 = gate rows, 2, 3 = the matching up rows
        const bool is_up = lg >= 2;
        const int r = (lg & 1) * 32 + lane;
        const int col = w_tile * 64 + r;
        for (int c = 0, ci = 0; c < TN; c += kChunk, ++ci) {
          float* buf = up_s + (ci & 1) * (kChunk * 64);
          float v[kChunk];
          load_acc(c, v);
          if (is_up) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) buf[j * 64 + r] = v[j];
          }
          q_epi_bar_sync();
          if (!is_up && t0 + c < p.T) {
#pragma unroll
            for (int m = 0; m < kChunk / 2; ++m) {
              float o2[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int j = 2 * m + h;
                const float g = v[j];
                o2[h] = g / (1.f + __expf(-g)) * buf[j * 64 + r];
              }
              const float send = (lane & 1) ? o2[0] : o2[1];
              const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
              const int t = t0 + c + 2 * m + (lane & 1);
              const int ce = col & ~1;
              if (t < p.T && ce < p.N / 2) {
                const uint32_t packed = (lane & 1) ? pack_bf16x2(recv, o2[1]) : pack_bf16x2(o2[0], recv);
                *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.ldo + ce) = packed;
              }
            }
          }
        }
      } else {
        for (int c = 0; c < TN; c += kChunk) {
          if (t0 + c >= p.T) break;
          float v[kChunk];
          load_acc(c, v);
          __nv_bfloat162 r2[kChunk / 2];
          if constexpr (EPI == kEpiResidual) {
#pragma unroll
            for (int m = 0; m < kChunk / 2; ++m) {
              const int t = t0 + c + 2 * m + (lane & 1);
              const int ne = n & ~1;
              r2[m] = (t < p.T && ne < p.N)
                          ? *reinterpret_cast<const __nv_bfloat162*>(p.resid + static_cast<long long>(t) * p.ldr + ne)
                          : __nv_bfloat162();
            }
          }
#pragma unroll
          for (int m = 0; m < kChunk / 2; ++m) {
            const float a0 = v[2 * m], a1 = v[2 * m + 1];
            const float send = (lane & 1) ? a0 : a1;
            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
            const int t = t0 + c + 2 * m + (lane & 1);
            const int ne = n & ~1;
            if (t < p.T && ne < p.N) {
              float lo = (lane & 1) ? recv : a0;
              float hi = (lane & 1) ? a1 : recv;
              if constexpr (EPI == kEpiResidual) {
                lo += __bfloat162float(r2[m].x);
                hi += __bfloat162float(r2[m].y);
              }
              *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.ldo + ne) = pack_bf16x2(lo, hi);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[a]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

int q_sm_count();

template <int QT, int EPI>
cudaError_t launch_q_persist(const CUtensorMap& tw, const CUtensorMap& tx, const QParams& kp, int n_tiles,
                             cudaStream_t stream, bool pdl) {
  auto kern = gemm_q_persist_kernel<QT, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, QPersist<QT>::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles < q_sm_count() ? n_tiles : q_sm_count());
  cfg.blockDim = dim3(kQPersistThreads);
  cfg.dynamicSmemBytes = QPersist<QT>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, kp);
}

template <int QT>
cudaError_t launch_q_persist_epi(int epi, const CUtensorMap& tw, const CUtensorMap& tx, const QParams& kp, int n_tiles,
                                 cudaStream_t stream, bool pdl) {
  switch (epi) {
    case kEpiResidual: return launch_q_persist<QT, kEpiResidual>(tw, tx, kp, n_tiles, stream, pdl);
    case kEpiSwiglu: return launch_q_persist<QT, kEpiSwiglu>(tw, tx, kp, n_tiles, stream, pdl);
    default: return launch_q_persist<QT, kEpiStore>(tw, tx, kp, n_tiles, stream, pdl);
  }
}

template <int TN, int QT, int EPI, bool DEEP>
cudaError_t launch_one(const CUtensorMap& tw, const CUtensorMap& tx, const QParams& kp, dim3 grid, cudaStream_t stream,
                       bool pdl) {
  using Cfg = QCfg<TN, QT, DEEP>;
  auto kern = gemm_q_kernel<TN, QT, EPI, DEEP>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (kp.cluster > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = kp.cluster;
    ++n_attr;
  }
  if (pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, kp);
}

int q_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}
bool q_is_deep(int tn, dim3 grid) {
  return tn <= 64 && static_cast<long long>(grid.x) * grid.y * grid.z <= q_sm_count();
}

template <int QT, int EPI>
cudaError_t launch_tn(int tn, const CUtensorMap& tw, const CUtensorMap& tx, const QParams& kp, dim3 grid,
                      cudaStream_t stream, bool pdl) {
  const bool deep = q_is_deep(tn, grid);
  switch (tn) {
    case 32: return deep ? launch_one<32, QT, EPI, true>(tw, tx, kp, grid, stream, pdl)
                         : launch_one<32, QT, EPI, false>(tw, tx, kp, grid, stream, pdl);
    case 64: return deep ? launch_one<64, QT, EPI, true>(tw, tx, kp, grid, stream, pdl)
                         : launch_one<64, QT, EPI, false>(tw, tx, kp, grid, stream, pdl);
    case 128: return launch_one<128, QT, EPI, false>(tw, tx, kp, grid, stream, pdl);
    default: return launch_one<256, QT, EPI, false>(tw, tx, kp, grid, stream, pdl);
  }
}

template <int QT>
cudaError_t launch_epi(int epi, int tn, const CUtensorMap& tw, const CUtensorMap& tx, const QParams& kp, dim3 grid,
                       cudaStream_t stream, bool pdl) {
  switch (epi) {
    case kEpiResidual: return launch_tn<QT, kEpiResidual>(tn, tw, tx, kp, grid, stream, pdl);
    case kEpiSwiglu: return launch_tn<QT, kEpiSwiglu>(tn, tw, tx, kp, grid, stream, pdl);
    case kEpiPushAll: return launch_tn<QT, kEpiPushAll>(tn, tw, tx, kp, grid, stream, pdl);
    case kEpiPushPartial: return launch_tn<QT, kEpiPushPartial>(tn, tw, tx, kp, grid, stream, pdl);
    default: return launch_tn<QT, kEpiStore>(tn, tw, tx, kp, grid, stream, pdl);
  }
}

struct Key {
  const void* base; uint64_t rows, cols, ld; uint32_t box;
  bool operator==(const Key& o) const { return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ k.rows; h = h * 1000003u ^ k.cols; h = h * 1000003u ^ k.ld;
    return h * 1000003u ^ k.box;
  }
};
bool cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box) {
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  Key key{base, rows, cols, ld, box};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  CUtensorMap m;
  if (!make_tmap_2d(&m, TmapDtype::U8, base, rows, cols, ld, box, kKBytes, true)) return false;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

int q_tile_tokens(int T) { return T <= 32 ? 32 : (T <= 64 ? 64 : (T <= 128 ? 128 : 256)); }

}  // namespace

int64_t nvfp4_act_scale_bytes(int64_t T, int64_t K) { return ((T + 255) / 256) * 2 * (K / 64) * kSfTileBytes; }

template <typename Kern, typename... Args>
cudaError_t launch_pdl(Kern kern, dim3 grid, cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = dim3(256); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

const char* quant_act_fp8(const __nv_bfloat16* x, int64_t ldx, int64_t T, int64_t K, uint8_t* codes, float* scale,
                          cudaStream_t stream, bool pdl) {
  if (T <= 0) return nullptr;
  if (K % 8 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(codes) & 7))
    return "quant_act_fp8: K and the row stride must be multiples of 8, pointers aligned";
  cudaError_t e = launch_pdl(quant_act_fp8_kernel, dim3(static_cast<unsigned>(T)), stream, pdl, x,
                             static_cast<long long>(ldx), static_cast<int>(K), codes, scale);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* quant_act_nvfp4(const __nv_bfloat16* x, int64_t ldx, int64_t T, int64_t K, uint8_t* codes, uint8_t* sf_plane,
                            cudaStream_t stream, bool pdl) {
  if (T <= 0) return nullptr;
  if (K % 64 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(codes) & 7))
    return "quant_act_nvfp4: K must be a multiple of 64, the row stride of 8, pointers aligned";
  dim3 grid(static_cast<unsigned>(T), static_cast<unsigned>((K / 16 + 255) / 256));
  cudaError_t e = launch_pdl(quant_act_nvfp4_kernel, grid, stream, pdl, x, static_cast<long long>(ldx),
                             static_cast<int>(K), codes, sf_plane);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* gemm_quant(const QGemmArgs& a) {
  if (a.T <= 0 || a.N <= 0 || a.K <= 0) return "gemm_quant: empty problem";
  const bool bs = a.qtype == kQNvfp4;
  if (a.qtype != kQFp8Row && !bs) return "gemm_quant: unknown weight format";
  const bool push = a.epi == kEpiPushAll || a.epi == kEpiPushPartial;
  if (a.epi != kEpiStore && a.epi != kEpiResidual && a.epi != kEpiSwiglu && !push) return "gemm_quant: unsupported epilogue";
  const int64_t k_bytes = bs ? a.K / 2 : a.K;
  if (bs ? (a.K % 256) : (a.K % 16)) return "gemm_quant: K must be a multiple of 256 (nvfp4) / 16 (fp8)";
  if ((a.ldw % 16) || (a.ldx % 16) || ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.x)) & 15))
    return "gemm_quant: operands and leading dimensions must be 16-byte aligned";
  if (a.w_scale == nullptr || a.x_scale == nullptr || (a.out == nullptr && !push)) return "gemm_quant: missing scale or output";
  if ((a.N & 1) || (a.ldo & 1)) return "gemm_quant: N and ldo must be even";
  if (a.epi == kEpiSwiglu && a.N % 128) return "gemm_quant: SwiGLU needs tile-interleaved rows (N multiple of 128)";
  if (a.epi == kEpiResidual && a.resid == nullptr) return "gemm_quant: residual epilogue without residual";
  const int tn = q_tile_tokens(static_cast<int>(a.T));
  QParams kp = {};
  kp.T = static_cast<int>(a.T); kp.N = static_cast<int>(a.N); kp.K = static_cast<int>(a.K);
  kp.num_kb = static_cast<int>((k_bytes + kKBytes - 1) / kKBytes);
  int splits = a.splits < 1 ? 1 : a.splits;
  if (splits > kp.num_kb) splits = kp.num_kb;
  kp.kb_per_split = (kp.num_kb + splits - 1) / splits;
  splits = (kp.num_kb + kp.kb_per_split - 1) / kp.kb_per_split;
  // leader's idle stages hold (S-1) peer tiles of TN*512 bytes (+ TN*256 for the SwiGLU exchange)
  const int stage_bytes = kWTileBytes + tn * kKBytes + (bs ? (tn <= 128 ? 8 : 12) * kSfTileBytes : 0);
  // (sized for the shallow pipeline: a split grid may or may not fit in one wave)
  const int stages = tn <= 32 ? 4 : (tn == 64 ? 3 : (tn == 128 ? 5 : 3));
  while (splits > 1 && ((splits - 1) * tn * 512 + tn * 256 > stages * stage_bytes || splits > 8 ||
                        (kp.num_kb + splits - 1) / splits * (splits - 1) >= kp.num_kb))
    --splits;
  kp.kb_per_split = (kp.num_kb + splits - 1) / splits;
  kp.cluster = splits;
  kp.k_tiles = static_cast<int>(a.K / 64);
  if (bs) {
    kp.w_sf = static_cast<const uint8_t*>(a.w_scale);
    kp.x_sf = static_cast<const uint8_t*>(a.x_scale);
    if ((reinterpret_cast<uintptr_t>(kp.w_sf) | reinterpret_cast<uintptr_t>(kp.x_sf)) & 15) return "gemm_quant: scale planes must be 16-byte aligned";
    kp.out_scale = 1.f / a.w_divisor;
  } else {
    kp.w_scale = static_cast<const float*>(a.w_scale);
    kp.x_scale = static_cast<const float*>(a.x_scale);
  }
  kp.out = static_cast<__nv_bfloat16*>(a.out); kp.ldo = a.ldo;
  kp.resid = static_cast<const __nv_bfloat16*>(a.resid); kp.ldr = a.ldr;
  kp.status = a.status;
  kp.next_codes = nullptr; kp.next_sf = nullptr;
  if (a.next_codes != nullptr) {
    if (a.epi != kEpiSwiglu || !bs || a.next_sf == nullptr || (a.N / 2) % 64 || a.T > 128)
      return "gemm_quant: the fused activation quantiser is for nvfp4 SwiGLU at decode sizes (N / 2 a multiple of 64)";
    kp.next_codes = static_cast<uint8_t*>(a.next_codes); kp.next_sf = static_cast<uint8_t*>(a.next_sf);
  }
  if (push) {
    if (a.world < 1 || a.world > kMaxRanks || a.rank < 0 || a.rank >= a.world) return "gemm_quant: bad rank/world";
    kp.rank = a.rank; kp.world = a.world;
    for (int r = 0; r < a.world; ++r) {
      if (a.peer_recv[r] == nullptr || a.peer_flag[r] == nullptr) return "gemm_quant: missing peer pointer";
      kp.peer_recv[r] = a.peer_recv[r]; kp.peer_flag[r] = a.peer_flag[r];
    }
    if (a.epi == kEpiPushAll) {
      if (a.call_idx == nullptr || a.T_cap < kp.T) return "gemm_quant: push-all needs the call counter and T <= T_cap";
      kp.call_idx = a.call_idx; kp.T_cap = a.T_cap;
    } else {
      if (kp.N % a.world || (kp.N / a.world) % kTileN) return "gemm_quant: N / world must be a multiple of 128";
      if (splits != 1) return "gemm_quant: the reduce-scatter epilogue takes no split-K";
      kp.slice_cols = kp.N / a.world;
    }
  }
  CUtensorMap tw, tx;
  if (!cached_tmap(&tw, a.w, a.N, k_bytes, a.ldw, 64)) return "gemm_quant: weight tensor map rejected";
  // prefill-sized problems with more tiles than SMs: persistent kernel (NFB_GEMM_PERSISTENT=0 switches it off)
  static const bool persistent_enabled = [] {
    const char* e = getenv("NFB_GEMM_PERSISTENT");
    return !(e != nullptr && e[0] == '0');
  }();
  if (persistent_enabled && tn == 256 && splits == 1 && !push) {
    const int ptn = bs ? 128 : 256;
    const long long n_tiles = static_cast<long long>((kp.N + kTileN - 1) / kTileN) * ((kp.T + ptn - 1) / ptn);
    if (n_tiles > q_sm_count()) {
      if (!cached_tmap(&tx, a.x, a.T, k_bytes, a.ldx, ptn)) return "gemm_quant: activation tensor map rejected";
      cudaError_t e = bs ? launch_q_persist_epi<kQNvfp4>(a.epi, tw, tx, kp, static_cast<int>(n_tiles), a.stream, a.pdl)
                         : launch_q_persist_epi<kQFp8Row>(a.epi, tw, tx, kp, static_cast<int>(n_tiles), a.stream, a.pdl);
      return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
    }
  }
  if (!cached_tmap(&tx, a.x, a.T, k_bytes, a.ldx, tn)) return "gemm_quant: activation tensor map rejected";
  dim3 grid((kp.N + kTileN - 1) / kTileN, (kp.T + tn - 1) / tn, splits);
  cudaError_t e = bs ? launch_epi<kQNvfp4>(a.epi, tn, tw, tx, kp, grid, a.stream, a.pdl)
                     : launch_epi<kQFp8Row>(a.epi, tn, tw, tx, kp, grid, a.stream, a.pdl);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
