// Weight-stationary bf16 GEMM for sm_100a:  out[T, N] = x[T, K] * W[N, K]^T.
//
// The weight matrix is the UMMA "A" operand (M = 128 weight rows per CTA), the
// activations are the "B" operand (UMMA N = TN tokens, 16..256), so one kernel
// template covers decode (T = 1..64: pure weight streaming) and prefill
// (T tiles of 256).  Operands arrive by TMA into 128-byte-swizzled shared
// memory, tcgen05.mma accumulates in TMEM, and the epilogue reads TMEM with
// tcgen05.ld and fuses: plain store (+bias), residual add, SwiGLU (gate and up
// rows of the fused [gate; up] parent are loaded as two 64-row boxes of one
// 128-row tile), or fp32 split-K partials.
//
// Covers the reference's linear / linear_add / linear_swiglu bf16 routes
// (include/ninfer/ops/linear.h, src/ops/linear/bf16/bf16_gemm_mma.cuh,
// src/ops/linear_swiglu/*, src/ops/linear_add/*), which are mma.sync kernels.
#include "gemm.h"

#include <mutex>
#include <unordered_map>

#include <cstdlib>

#include "../comm/peer_sync.cuh"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"

namespace nfb {

namespace {

constexpr int kBlockK = 64;           // bf16 elements per k-block = one 128-byte swizzle row
constexpr int kTileN = 128;           // weight rows per CTA (UMMA M)
constexpr int kWTileBytes = kTileN * 128;

// DEEP = one CTA per SM with a pipeline twice as deep: used when the whole grid fits in one wave, so that a
// grid of ~100 CTAs still keeps ~200 KB per SM in flight (the memory system needs ~30 MB in flight overall).
template <int TN, bool DEEP = false>
struct GemmCfg {
  // TN = 256 (prefill): the main loop already runs at the tensor rate, so what matters is hiding the epilogue
  // (9-24 us per tile against a 33 us main loop at K = 5120).  Two stages = 96 KB let two CTAs share an SM (and its
  // 512 TMEM columns): one drains its accumulator while the other feeds the tensor core.  A grid that fits in one
  // wave keeps the four-stage pipeline (DEEP).
  static constexpr int kStages =
      DEEP ? (TN <= 32 ? 10 : (TN == 256 ? 4 : 8)) : (TN <= 32 ? 5 : (TN == 64 ? 4 : (TN == 128 ? 6 : 2)));
  static constexpr int kXTileBytes = TN * 128;
  static constexpr int kStageBytes = kWTileBytes + kXTileBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;  // +1024: manual alignment
  static constexpr int kTmemCols = TN < 32 ? 32 : TN;
};

// Optional phase timeline (globaltimer, ns) of every CTA, for performance debugging: 8 stamps per CTA.
constexpr int kTraceStamps = 12;
constexpr int kTraceCtas = 4096;
__device__ unsigned long long g_gemm_trace[kTraceCtas * kTraceStamps];
bool g_trace_enabled = false;
// Timeline over SEVERAL launches (a whole layer, a captured graph): launch i of a traced run writes the stamps of
// its first kTimelineCtas CTAs into slot i % kTimelineSlots, so that the overlap of consecutive kernels under
// programmatic dependent launch can be read off one clock (globaltimer).
constexpr int kTimelineSlots = 64;
constexpr int kTimelineCtas = 256;
__device__ unsigned long long g_gemm_timeline[kTimelineSlots * kTimelineCtas * kTraceStamps];
int g_timeline_next = -1;   // < 0: off; else the slot of the next launch

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct KernelParams {
  int trace;
  int T, N, K;
  int kb_per_split;    // k-blocks handled by one blockIdx.z
  int num_kb;          // ceil(K / 64)
  int swiglu_half;     // N/2 for the SwiGLU epilogue, else 0
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* resid;
  long long ldr;
  const float* bias;
  int act;  // kActNone / kActGeluTanh / kActGeluErf, applied after the bias (kEpiStore only)
  float* partial;      // [splits, T, N] fp32
  int* status;
  // kEpiPushPartial: tensor-parallel reduce-scatter by peer stores
  float* peer_recv[kMaxRanks];
  unsigned int* peer_flag[kMaxRanks];
  int rank, slice_cols;
  // in-cluster split-K: `cluster` CTAs along z share one output tile and reduce through DSMEM
  int cluster;
  // kEpiPushAll: one-shot all-reduce by push into [parity][src_rank][T_cap][N] on every rank
  int world, T_cap;
  const unsigned int* call_idx;  // device counter of finished reduce calls; its parity picks the buffer
  // kEpiRsAg: reduce-scatter into the owner, owner-side reduction, all-gather of the new residual tile
  __nv_bfloat16* peer_x[kMaxRanks];
  long long ld_resid;
  float* peer_ss[kMaxRanks];
  unsigned int* peer_xflag[kMaxRanks];
  uint2* peer_recv_ll[kMaxRanks];   // [src][T_cap][N / world] (fp32 bits, epoch)
  RsState* rs_state;
  int rs_phase;
  // gathered consumer (kEpiStore / kEpiSwiglu): wait for the residual tiles, RMS norm as an epilogue row scale
  const unsigned int* g_flag;
  const unsigned int* g_target;
  const float* g_ss;
  int g_tiles;
  float g_inv_n, g_eps;
  // kEpiStore: decode conv + SiLU + history roll on columns [0, conv_C)
  const __nv_bfloat16* conv_w;
  __nv_bfloat16* conv_state;
  const int* conv_slot;
  __nv_bfloat16* conv_out;
  int conv_C;
  // L2 prefetch hint for the next kernel's weights: each CTA asks for `pf_per_cta` bytes of [pf_ptr, pf_ptr + pf_bytes)
  const uint8_t* pf_ptr;
  long long pf_bytes;
  int pf_per_cta;
};

// GELU in the two forms vision towers use: tanh approximation (transformer blocks) and exact erf (merger).
__device__ __forceinline__ float gelu(float x, int mode) {
  if (mode == kActGeluTanh) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}

template <int TN, int EPI, bool DEEP>
__global__ void __launch_bounds__(128) gemm_ws_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                                       const __grid_constant__ CUtensorMap tmap_x,
                                                       const KernelParams p) {
  using Cfg = GemmCfg<TN, DEEP>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_accum;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int peer_ok[kMaxRanks];
  __shared__ float row_s[TN];   // per token: RMS factor (gathered consumer) or the tile's sum of squares (kEpiRsAg)
  __shared__ int rs_ok;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int cta_linear = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  auto stamp = [&](int i) {
    if (p.trace && threadIdx.x == 0) {
      const unsigned long long now = globaltimer_ns();
      if (cta_linear < kTraceCtas) g_gemm_trace[cta_linear * kTraceStamps + i] = now;
      if (p.trace > 1 && cta_linear < kTimelineCtas)
        g_gemm_timeline[((p.trace - 2) * kTimelineCtas + cta_linear) * kTraceStamps + i] = now;
    }
  };
  stamp(0);

  const int t0 = blockIdx.y * TN;
  const int n0 = (EPI == kEpiSwiglu) ? blockIdx.x * 64 : blockIdx.x * kTileN;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(p.num_kb, kb_begin + p.kb_per_split);
  // (phase 2 of kEpiRsAg runs no GEMM: the tiles were left in the receive buffers by phase 1)
  const int num_it = (EPI == kEpiRsAg && p.rs_phase == 2) ? 0 : kb_end - kb_begin;
  const bool gathered = (EPI == kEpiStore || EPI == kEpiSwiglu) && p.g_flag != nullptr;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int r = 0; r < kMaxRanks; ++r) peer_ok[r] = 0;
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
  stamp(1);

  // Let the next kernel in the stream begin its own prologue / weight prefetch.
  pdl_launch_next();

  if (warp == 0) {
    if (elect_one()) {
      // ---------------- TMA producer ----------------
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const int row_a = n0;
      const int row_b = (EPI == kEpiSwiglu) ? p.swiglu_half + n0 : n0 + 64;
      // Weights do not depend on the previous kernel: fill EVERY stage with them before waiting for it, so that the
      // whole pipeline (not one stage) is in flight while the previous kernel drains.  Only then the activations:
      // after the previous kernel (plain input), or after the owner ranks have pushed their residual tiles into
      // this rank's buffer (gathered input; bounded wait).
      const int pre = num_it < kStages ? num_it : kStages;
      for (int j = 0; j < pre; ++j) {
        const uint32_t full = smem_u32(&bar_full[j]);
        const uint32_t dst = smem_base + j * Cfg::kStageBytes;
        const int kx = (kb_begin + j) * kBlockK;
        mbar_expect_tx(full, Cfg::kStageBytes);
        tma_load_2d(dst, &tmap_w, full, kx, row_a, pol_w);
        tma_load_2d(dst + 64 * 128, &tmap_w, full, kx, row_b, pol_w);
      }
      pdl_wait_prior();
      if (gathered) {
        const uint32_t target = __ldcg(p.g_target);
        // on a time-out the loads below are still issued (the data is stale, the status word says so): every
        // barrier that was armed above must complete before the CTA may leave
        if (!wait_counter(p.g_flag, target, p.status)) abort_flag = 1;
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      for (int j = 0; j < pre; ++j)
        tma_load_2d(smem_base + j * Cfg::kStageBytes + kWTileBytes, &tmap_x, smem_u32(&bar_full[j]),
                    (kb_begin + j) * kBlockK, t0, pol_x);
      int it = pre;
      for (; it < num_it; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, kStatusEmptyWaitTimeout)) break;
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t dst = smem_base + s * Cfg::kStageBytes;
        const int kx = (kb_begin + it) * kBlockK;
        mbar_expect_tx(full, Cfg::kStageBytes);
        tma_load_2d(dst, &tmap_w, full, kx, row_a, pol_w);
        tma_load_2d(dst + 64 * 128, &tmap_w, full, kx, row_b, pol_w);
        tma_load_2d(dst + kWTileBytes, &tmap_x, full, kx, t0, pol_x);
      }
      if (abort_flag) {
        // Unwinding: let copies that were already issued land before the CTA exits.
        const int first = it > kStages ? it - kStages : 0;
        for (int j = first; j < it; ++j) {
          const uint32_t bar = smem_u32(&bar_full[j % kStages]);
          const uint32_t ph = (j / kStages) & 1;
          for (uint32_t spin = 0; spin < (1u << 20); ++spin)
            if (mbar_try_wait(bar, ph)) break;
        }
      } else if (p.pf_per_cta > 0) {
        // own loads are all in flight: pull this CTA's share of the next kernel's weights into L2
        const long long off = static_cast<long long>(cta_linear) * p.pf_per_cta;
        if (off < p.pf_bytes) {
          const long long n = min(static_cast<long long>(p.pf_per_cta), p.pf_bytes - off) & ~15LL;
          if (n > 0)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.pf_ptr + off), "r"(static_cast<uint32_t>(n))
                         : "memory");
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = umma_idesc(kTileN, TN, 1, 1);
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
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k) {
          // advance 16 elements (32 bytes) along K inside the swizzle atom: +2 in 16-byte units
          tc_mma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_empty[s]));
      }
      if (ok) tc_commit(smem_u32(&bar_accum));
    }
    __syncwarp();
  }

  // ---------------- epilogue: all four warps, warp w owns TMEM lanes 32w..32w+31 ----------------
  pdl_wait_prior();
  // kEpiRsAg: the bookkeeping word of this CTA's tile (its epoch) is fetched now, so that the latency hides under
  // the main loop
  uint32_t epoch_pre = 0;
  if constexpr (EPI == kEpiRsAg) {
    if (p.cluster <= 1 || blockIdx.z == 0) epoch_pre = p.rs_state->tile_epoch[blockIdx.x * kRsMaxTokenTiles + blockIdx.y];
  }
  if constexpr (EPI == kEpiStore) {
    // decode conv tiles: pull this thread's history columns towards L2 now (fire and forget), so that the
    // dependent slot -> history loads of the epilogue do not each pay a trip to HBM after the main loop
    if (p.conv_state != nullptr && n0 < p.conv_C && (p.cluster <= 1 || blockIdx.z == 0)) {
      const int n = n0 + threadIdx.x;
      for (int t = t0; t < min(p.T, t0 + TN); ++t) {
        const __nv_bfloat16* st = p.conv_state + static_cast<long long>(p.conv_slot[t]) * 3 * p.conv_C + n;
        if ((threadIdx.x & 31) == 0) {   // one request per 64-byte run of a warp's channels
#pragma unroll
          for (int j = 0; j < 3; ++j) asm volatile("prefetch.global.L2 [%0];" ::"l"(st + j * p.conv_C));
        }
      }
    }
  }
  bool have_acc = true;
  if (num_it > 0) {
    have_acc = mbar_wait(smem_u32(&bar_accum), 0, &abort_flag, p.status, kStatusAccumWaitTimeout);
  }
  tc_fence_after();
  // One CTA-wide verdict, so the barriers inside the epilogue are never divergent.
  int epilogue_ok = __syncthreads_and(have_acc && !abort_flag);
  stamp(2);
  const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  constexpr int kChunk = 16;

  // ---------------- in-cluster split-K: peers hand their fp32 tiles to the leader through DSMEM ----------------
  const int S = p.cluster;
  const uint32_t crank = S > 1 ? blockIdx.z : 0;
  // leader-side landing zone in the (now idle) pipeline stages: [S-1][TN][128] floats
  const float* peer_s = reinterpret_cast<const float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
  if (S > 1) {
    // #1: every CTA of the cluster has retired its MMAs, so the leader's stages may be overwritten
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
    stamp(3);
    // #2: peers' tiles (release) are visible to the leader (acquire)
    cluster_sync_all();
    stamp(4);
    if (crank != 0) {
      epilogue_ok = 0;  // only the leader writes the output
    } else {
      for (int r = 1; r < S; ++r) epilogue_ok &= peer_ok[r];
    }
  }
  if (gathered) {
    // RMS factor of every token of the tile from the per-tile sums of squares that travelled with the residual
    if (threadIdx.x == 0) (void)ld_acquire_sys(p.g_flag);
    __syncthreads();
    for (int t = threadIdx.x; t < TN; t += 128) {
      // the whole table row in independent 16-byte loads (entries past the last tile are never written: zero)
      float ss = 0.f;
      if (t0 + t < p.T) {
        const float4* rowp = reinterpret_cast<const float4*>(p.g_ss + static_cast<long long>(t0 + t) * kRsSsStride);
        float4 q[kRsSsStride / 4];
#pragma unroll
        for (int j = 0; j < kRsSsStride / 4; ++j) q[j] = __ldcg(rowp + j);
#pragma unroll
        for (int j = 0; j < kRsSsStride / 4; ++j) ss += (q[j].x + q[j].y) + (q[j].z + q[j].w);
      }
      row_s[t] = rsqrtf(ss * p.g_inv_n + p.g_eps);
    }
    __syncthreads();
  }
  // accumulator chunk = own TMEM columns + the peers' contributions, summed in rank order
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
    if (gathered) {
#pragma unroll
      for (int j = 0; j < kChunk; ++j) acc[j] *= row_s[c + j];
    }
  };

  if (epilogue_ok) {
    if constexpr (EPI == kEpiSwiglu) {
      // lanes 0..63 hold gate rows, lanes 64..127 the matching up rows.
      float* up_s = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))) +
                    (S - 1) * TN * 128;  // [TN][64], behind the peers' landing zone
      if (warp >= 2) {
        const int r = (warp - 2) * 32 + lane;
        for (int c = 0; c < TN; c += kChunk) {
          float v[kChunk];
          load_acc(c, v);
#pragma unroll
          for (int j = 0; j < kChunk; ++j) up_s[(c + j) * 64 + r] = v[j];
        }
      }
      __syncthreads();
      if (warp < 2) {
        const int r = warp * 32 + lane;
        const int n = n0 + r;
        for (int c = 0; c < TN; c += kChunk) {
          float v[kChunk];
          load_acc(c, v);
#pragma unroll
          for (int m = 0; m < kChunk / 2; ++m) {
            float a[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int j = 2 * m + h;
              const float g = v[j];
              const float u = up_s[(c + j) * 64 + r];
              a[h] = g / (1.f + __expf(-g)) * u;
            }
            const float send = (lane & 1) ? a[0] : a[1];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
            const int t = t0 + c + 2 * m + (lane & 1);
            const int ne = n & ~1;
            if (t < p.T && ne < p.swiglu_half) {
              const uint32_t packed = (lane & 1) ? pack_bf16x2(recv, a[1]) : pack_bf16x2(a[0], recv);
              *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.ldo + ne) = packed;
            }
          }
        }
      }
    } else if constexpr (EPI == kEpiPushPartial) {
      // reduce-scatter by push: this tile's columns belong to one owner rank; the fp32 partial goes into the
      // owner's receive buffer [src_rank][split][T][slice_cols].  The tile passes through shared memory (the idle
      // pipeline stages), up to 128 token rows at a time, so that the stores are 16 bytes wide and every token row
      // of the tile is one contiguous 512-byte run, instead of 4-byte stores in 128-byte runs.
      const int owner = n0 / p.slice_cols;
      constexpr int kRowPad = kTileN + 4;
      constexpr int kRows = TN < 128 ? TN : 128;
      float* tile_s = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
      const int col = (threadIdx.x & 3) * 32;
      float* dst = p.peer_recv[owner] + (static_cast<long long>(p.rank) * gridDim.z + blockIdx.z) * p.T * p.slice_cols +
                   (n0 + col - owner * p.slice_cols);
      for (int h = 0; h < TN; h += kRows) {
        if (t0 + h >= p.T) break;
        for (int c = h; c < h + kRows; c += kChunk) {
          if (t0 + c >= p.T) break;
          float v[kChunk];
          load_acc(c, v);
#pragma unroll
          for (int j = 0; j < kChunk; ++j) tile_s[(c - h + j) * kRowPad + warp * 32 + lane] = v[j];
        }
        __syncthreads();
        for (int r = threadIdx.x >> 2; r < kRows; r += 32) {
          const int t = t0 + h + r;
          if (t >= p.T) continue;
          const float4* src4 = reinterpret_cast<const float4*>(tile_s + r * kRowPad + col);
          float4* dst4 = reinterpret_cast<float4*>(dst + static_cast<long long>(t) * p.slice_cols);
#pragma unroll
          for (int q = 0; q < 8; ++q) dst4[q] = src4[q];
        }
        __syncthreads();   // (orders the peer stores before the signalling thread; frees the staging tile)
      }
      // publish: the signalling thread's release (system scope) is cumulative over the stores the barrier ordered
      if (threadIdx.x == 0) red_release_sys_add(p.peer_flag[owner], 1u);
    } else if constexpr (EPI == kEpiRsAg) {
      const int owner = n0 / p.slice_cols;
      const bool pushes = p.rs_phase != 2;
      const bool reduces = p.rs_phase != 1;
      // Every call of this tile carries the next epoch: the tile's fp32 values travel as (value, epoch) pairs, so
      // the reader sees from the data itself when a tile is complete.  No fence and no counter sit between the
      // writer's stores and the reader's loads (16-byte stores are not torn).  Every tile of one state object is
      // written once per call, so all tiles carry the same epoch.
      unsigned int* epoch_word = &p.rs_state->tile_epoch[blockIdx.x * kRsMaxTokenTiles + blockIdx.y];
      const uint32_t epoch = epoch_pre + 1u;
      // The fp32 tile goes through shared memory (behind the split-K landing zone of the idle pipeline stages) so
      // that the push works on token rows: a quarter row (32 columns) per thread, 16-byte accesses, long
      // contiguous runs per token towards the owner.
      constexpr int kRowPad = kTileN + 4;   // floats per row: shifts consecutive rows by four banks
      float* tile_s = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))) + (S - 1) * TN * 128;
      if (pushes) {
        for (int c = 0; c < TN; c += kChunk) {
          if (t0 + c >= p.T) break;
          float v[kChunk];
          load_acc(c, v);
#pragma unroll
          for (int j = 0; j < kChunk; ++j) tile_s[(c + j) * kRowPad + warp * 32 + lane] = v[j];
        }
      }
      if (threadIdx.x == 0) rs_ok = 1;
      __syncthreads();
      if (pushes) {
        // hop 1: rows of the tile into the owner's receive buffer [src][T_cap][slice] of (value, epoch) pairs --
        // the owner's own tiles take the same road (into its own buffer), so that the reduction below reads every
        // contribution the same way and can run on any CTA
        const int col = (threadIdx.x & 3) * 32;
        const int n_local = n0 + col - owner * p.slice_cols;
        uint2* dst = p.peer_recv_ll[owner] + static_cast<long long>(p.rank) * p.T_cap * p.slice_cols + n_local;
        for (int r = threadIdx.x >> 2; r < TN; r += 32) {
          const int t = t0 + r;
          if (t >= p.T) continue;
          const float4* src4 = reinterpret_cast<const float4*>(tile_s + r * kRowPad + col);
          uint4* dst4 = reinterpret_cast<uint4*>(dst + static_cast<long long>(t) * p.slice_cols);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 f = src4[q];
            dst4[2 * q] = make_uint4(__float_as_uint(f.x), epoch, __float_as_uint(f.y), epoch);
            dst4[2 * q + 1] = make_uint4(__float_as_uint(f.z), epoch, __float_as_uint(f.w), epoch);
          }
        }
        stamp(7);
      }
      // hop 2, spread over the grid: this rank owns T x slice_cols values; they are cut into units of one token x
      // eight columns, one unit per thread, and dealt to the leading CTAs of the grid.  A thread has the 64 bytes
      // of all `world` contributions in flight at once, so a unit costs one round of polling instead of one per
      // contribution (a tile's owner CTA reducing its whole tile alone needed 2 x (world - 1) dependent rounds).
      const int n_ctas = gridDim.x * gridDim.y;                       // (split-K helpers never get here)
      const int cta = blockIdx.x + gridDim.x * blockIdx.y;
      const int groups = p.slice_cols / 8;                            // 8-column groups per token
      const int units = p.T * groups;
      const int n_red = min(n_ctas, (units + 127) / 128);
      if (reduces && cta < n_red) {
        stamp(8);
        __nv_bfloat16* my_x = p.peer_x[p.rank];
        const uint2* recv = p.peer_recv_ll[p.rank];
        for (int u0 = cta * 128; u0 < units; u0 += n_red * 128) {    // uniform trip count per CTA
          const int u = u0 + threadIdx.x;
          const bool live0 = u < units;
          const int t = live0 ? u / groups : 0;
          const int cg = live0 ? u % groups : 0;
          const int n_first = p.rank * p.slice_cols + cg * 8;         // first output column of the unit
          bool live = live0;
          float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          uint4 rv = make_uint4(0, 0, 0, 0);
          if (live) {
            rv = *reinterpret_cast<const uint4*>(my_x + static_cast<long long>(t) * p.ld_resid + n_first);
            uint4 v[kMaxRanks][4];
            bool here = false;
            for (uint32_t spin = 0; spin < kPeerPollLimit && !here; ++spin) {
              here = true;
#pragma unroll
              for (int src = 0; src < kMaxRanks; ++src) {
                if (src >= p.world) break;
                const uint4* sp = reinterpret_cast<const uint4*>(recv + (static_cast<long long>(src) * p.T_cap + t) * p.slice_cols + cg * 8);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  v[src][q] = ld_volatile_v4(sp + q);
                  here = here && v[src][q].y == epoch && v[src][q].w == epoch;
                }
              }
              if (!here) {
                if ((spin & 1023u) == 1023u && p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) break;
                if (spin > 64) __nanosleep(100);
              }
            }
            if (!here) {   // bounded: record it and let the step fail on the host instead of hanging
              report_status(p.status, kStatusPeerWaitTimeout);
              rs_ok = 0;
              live = false;
            }
#pragma unroll
            for (int src = 0; src < kMaxRanks; ++src) {   // rank order, the same on every rank
              if (src >= p.world) break;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                a[2 * q] += __uint_as_float(v[src][q].x);
                a[2 * q + 1] += __uint_as_float(v[src][q].z);
              }
            }
          }
          float ss = 0.f;
          if (live) {
            const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
            uint4 o;
            uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              op[e] = pack_bf16x2(a[2 * e] + __bfloat162float(rp[e].x), a[2 * e + 1] + __bfloat162float(rp[e].y));
              const __nv_bfloat162 ob = *reinterpret_cast<const __nv_bfloat162*>(&op[e]);
              const float f0 = __bfloat162float(ob.x), f1 = __bfloat162float(ob.y);
              ss += f0 * f0 + f1 * f1;
            }
            const long long at = static_cast<long long>(t) * p.ld_resid + n_first;
            for (int rk = 0; rk < p.world; ++rk)   // all-gather by push (own copy included)
              *reinterpret_cast<uint4*>(p.peer_x[rk] + at) = o;
          }
          // the sixteen threads of one (token, 128-column tile): its sum of squares (a dead unit adds zero)
#pragma unroll
          for (int o2 = 1; o2 < 16; o2 <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
          if (live && (threadIdx.x & 15) == 0) {
            const int tile_global = n_first / kTileN;
            for (int rk = 0; rk < p.world; ++rk)
              p.peer_ss[rk][static_cast<long long>(t) * kRsSsStride + tile_global] = ss;
          }
        }
        stamp(9);
        __syncthreads();
        stamp(10);
        // the block barrier orders every thread's peer stores before the signalling threads, whose release (system
        // scope) is cumulative over them: no separate fence
        if (rs_ok && threadIdx.x < p.world) red_release_sys_add(p.peer_xflag[threadIdx.x], 1u);
        stamp(11);
      }
      if (threadIdx.x == 0 && p.rs_phase != 1) *epoch_word = epoch;
      // what the next consumer of the residual stream has to wait for: one arrival per reducing CTA of every rank
      if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && p.rs_phase != 1)
        p.rs_state->x_expected += static_cast<unsigned int>(n_red * p.world);
    } else {
      const int n = n0 + warp * 32 + lane;
      const float bias = ((EPI == kEpiStore || EPI == kEpiResidual) && p.bias != nullptr && n < p.N) ? p.bias[n] : 0.f;
      // tiles of conv channels (kEpiStore at decode): taps + SiLU + history roll here, activation to conv_out
      const bool conv_tile = EPI == kEpiStore && p.conv_state != nullptr && n0 < p.conv_C;
      float cw[4] = {0.f, 0.f, 0.f, 0.f};
      if (conv_tile) {
        const uint2 wv = *reinterpret_cast<const uint2*>(p.conv_w + static_cast<long long>(n) * 4);
        const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) cw[j] = __bfloat162float(wp[j]);
      }
      __nv_bfloat16* const outp = conv_tile ? p.conv_out : p.out;
      const long long ldo = conv_tile ? p.conv_C : p.ldo;
      for (int c = 0; c < TN; c += kChunk) {
        if (t0 + c >= p.T) break;
        float v[kChunk];
        load_acc(c, v);
        if (conv_tile) {
          // all history columns of the chunk's tokens first (48 independent loads), then taps and the roll
          long long at[kChunk];
          __nv_bfloat16 h[kChunk][3];
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const int t = t0 + c + j;
            at[j] = t < p.T ? static_cast<long long>(p.conv_slot[t]) * 3 * p.conv_C + n : -1;
          }
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            if (at[j] >= 0) {
              h[j][0] = p.conv_state[at[j]];
              h[j][1] = p.conv_state[at[j] + p.conv_C];
              h[j][2] = p.conv_state[at[j] + 2 * p.conv_C];
            }
          }
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            if (at[j] >= 0) {
              const __nv_bfloat16 xb = __float2bfloat16(v[j] + bias);   // the projection's bf16 value
              float a = 0.f;
              a += cw[0] * __bfloat162float(h[j][0]);
              a += cw[1] * __bfloat162float(h[j][1]);
              a += cw[2] * __bfloat162float(h[j][2]);
              a += cw[3] * __bfloat162float(xb);
              p.conv_state[at[j]] = h[j][1];
              p.conv_state[at[j] + p.conv_C] = h[j][2];
              p.conv_state[at[j] + 2 * p.conv_C] = xb;
              v[j] = a / (1.f + __expf(-a)) - bias;   // (the bias is added back below; it is zero for these tiles)
            }
          }
        }
        if constexpr (EPI == kEpiPartial) {
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const int t = t0 + c + j;
            if (t < p.T && n < p.N)
              p.partial[(static_cast<long long>(blockIdx.z) * p.T + t) * p.N + n] = v[j];
          }
        } else if constexpr (EPI == kEpiPushAll) {
          // one-shot all-reduce by push: the fp32 tile goes to EVERY rank's receive buffer
          // [parity][src_rank][T_cap][N]; the reader sums the W sources in rank order.
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
          // The residual may alias the output (in-place update): fetch the whole chunk's residual values
          // before the first store, otherwise every load would have to wait for the previous store.
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
            float a0 = v[2 * m] + bias;
            float a1 = v[2 * m + 1] + bias;
            if constexpr (EPI == kEpiStore) {
              if (p.act != kActNone) {
                a0 = gelu(a0, p.act);
                a1 = gelu(a1, p.act);
              }
            }
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
              *reinterpret_cast<uint32_t*>(outp + static_cast<long long>(t) * ldo + ne) = pack_bf16x2(lo, hi);
            }
          }
        }
      }
      if constexpr (EPI == kEpiPushAll) {
        __syncthreads();
        if (threadIdx.x < p.world) {
          __threadfence_system();
          unsigned int* flag = p.peer_flag[threadIdx.x];
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
        }
      }
    }
  }

  stamp(5);
  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::kTmemCols);
  stamp(6);
}

int device_sm_count();

// ------------------------------------------------------------------------------------------------------------
// Persistent prefill kernel (TN = 256): one CTA per SM walks output tiles, with the roles split over six warps so
// that the epilogue of tile i overlaps the main loop of tile i + 1:
//   warp 0  TMA producer (4 stages of 16 KB weights + 32 KB tokens, one running stage counter across tiles)
//   warp 1  MMA issuer; the fp32 accumulator alternates between TMEM columns [0, 256) and [256, 512)
//   warps 2..5  epilogue: warp w drains TMEM lanes 32 (w % 4) ..; tcgen05.ld -> bias / GELU / residual / SwiGLU -> bf16
// The non-persistent kernel spends 9-24 us per tile in an epilogue that nothing overlaps (main loop 33 us at
// K = 5120); here the tensor core only waits for the first tile's pipeline fill.  Tiles are numbered token-tile
// fastest, so the CTAs running at one time share a few weight tiles and all token tiles through L2.
constexpr int kPersistTN = 256;
constexpr int kPersistStages = 4;
constexpr int kPersistThreads = 192;
constexpr int kPersistStageBytes = kWTileBytes + kPersistTN * 128;
constexpr int kPersistExchangeBytes = 2 * 16 * 64 * 4;   // SwiGLU: two 16-column chunks of up values
constexpr int kPersistSmemBytes = kPersistStages * kPersistStageBytes + kPersistExchangeBytes + 1024;

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int EPI>
__global__ void __launch_bounds__(kPersistThreads, 1) gemm_persist_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                                                           const __grid_constant__ CUtensorMap tmap_x,
                                                                           const KernelParams p) {
  static_assert(EPI == kEpiStore || EPI == kEpiResidual || EPI == kEpiSwiglu, "persistent kernel: plain epilogues only");
  constexpr int TN = kPersistTN;
  constexpr int kStages = kPersistStages;
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
  const int w_rows = (EPI == kEpiSwiglu) ? 64 : kTileN;                 // output rows per tile
  const int n_w_tiles = (EPI == kEpiSwiglu) ? (p.swiglu_half + 63) / 64 : (p.N + kTileN - 1) / kTileN;
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
        const int n0 = (tile / n_t_tiles) * w_rows;
        const int t0 = (tile % n_t_tiles) * TN;
        const int row_a = n0;
        const int row_b = (EPI == kEpiSwiglu) ? p.swiglu_half + n0 : n0 + 64;
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
          const uint32_t dst = smem_base + s * kPersistStageBytes;
          const int kx = kb * kBlockK;
          mbar_expect_tx(full, kPersistStageBytes);
          tma_load_2d(dst, &tmap_w, full, kx, row_a, pol_w);
          tma_load_2d(dst + 64 * 128, &tmap_w, full, kx, row_b, pol_w);
          if (!waited_prior) {
            pdl_wait_prior();  // activations are produced by the previous kernel
            waited_prior = true;
          }
          tma_load_2d(dst + kWTileBytes, &tmap_x, full, kx, t0, pol_x);
        }
        if (!ok) break;
      }
      if (*abortp) {
        // Unwinding: let copies that were already issued land before the CTA exits.
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
      constexpr uint32_t idesc = umma_idesc(kTileN, TN, 1, 1);
      uint32_t it = 0;
      int tile_i = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !*abortp; tile += gridDim.x, ++tile_i) {
        const int a = tile_i & 1;
        const uint32_t aph = (tile_i >> 1) & 1;
        // the epilogue has drained this accumulator's previous tile
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
          const uint32_t a_addr = smem_base + s * kPersistStageBytes;
          const uint64_t a_desc = umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + kWTileBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k)
            tc_mma_f16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(smem_u32(&bar_empty[s]));
        }
        if (!ok) break;
        tc_commit(smem_u32(&bar_acc_full[a]));
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps ----------------
    pdl_wait_prior();   // the residual may be written by the previous kernel
    const int lg = warp & 3;   // TMEM lane group this warp may read
    constexpr int kChunk = 16;
    float* up_s = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)) + kStages * kPersistStageBytes);
    int tile_i = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_i) {
      const int a = tile_i & 1;
      const uint32_t ph = (tile_i >> 1) & 1;
      const bool have = mbar_wait(smem_u32(&bar_acc_full[a]), ph, &abort_flag, p.status, kStatusAccumWaitTimeout);
      // one verdict for the four warps, so that the chunk barriers below are never divergent
      if (lane == 0) epi_verdict[warp - 2] = (have && !*abortp) ? 1 : 0;
      epi_bar_sync();
      const bool go = epi_verdict[0] && epi_verdict[1] && epi_verdict[2] && epi_verdict[3];
      epi_bar_sync();   // everybody has read the verdict before the next tile overwrites it
      if (!go) break;
      tc_fence_after();
      const int n0 = (tile / n_t_tiles) * w_rows;
      const int t0 = (tile % n_t_tiles) * TN;
      const uint32_t lane_taddr = tmem_base + a * TN + (static_cast<uint32_t>(lg * 32) << 16);
      if constexpr (EPI == kEpiSwiglu) {
        // lane groups 0, 1 hold gate rows, 2, 3 the matching up rows; up values cross in 16-column chunks
        const bool is_up = lg >= 2;
        const int r = (lg & 1) * 32 + lane;
        const int n = n0 + r;
        for (int c = 0, ci = 0; c < TN; c += kChunk, ++ci) {
          float* buf = up_s + (ci & 1) * (kChunk * 64);
          uint32_t v[kChunk];
          tmem_ld_x16(lane_taddr + c, v);
          tmem_ld_wait();
          if (is_up) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) buf[j * 64 + r] = __uint_as_float(v[j]);
          }
          epi_bar_sync();
          if (!is_up && t0 + c < p.T) {
#pragma unroll
            for (int m = 0; m < kChunk / 2; ++m) {
              float o2[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int j = 2 * m + h;
                const float g = __uint_as_float(v[j]);
                o2[h] = g / (1.f + __expf(-g)) * buf[j * 64 + r];
              }
              const float send = (lane & 1) ? o2[0] : o2[1];
              const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
              const int t = t0 + c + 2 * m + (lane & 1);
              const int ne = n & ~1;
              if (t < p.T && ne < p.swiglu_half) {
                const uint32_t packed = (lane & 1) ? pack_bf16x2(recv, o2[1]) : pack_bf16x2(o2[0], recv);
                *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.ldo + ne) = packed;
              }
            }
          }
        }
      } else {
        const int n = n0 + lg * 32 + lane;
        const float bias = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.f;
        for (int c = 0; c < TN; c += kChunk) {
          if (t0 + c >= p.T) break;
          uint32_t v[kChunk];
          tmem_ld_x16(lane_taddr + c, v);
          tmem_ld_wait();
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
            float a0 = __uint_as_float(v[2 * m]) + bias;
            float a1 = __uint_as_float(v[2 * m + 1]) + bias;
            if constexpr (EPI == kEpiStore) {
              if (p.act != kActNone) {
                a0 = gelu(a0, p.act);
                a1 = gelu(a1, p.act);
              }
            }
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
      // this warp is done with the accumulator: hand it back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[a]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <int EPI>
cudaError_t launch_persist(const CUtensorMap& tw, const CUtensorMap& tx, const KernelParams& kp, int n_tiles,
                           cudaStream_t stream, bool pdl) {
  auto kern = gemm_persist_kernel<EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPersistSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles < device_sm_count() ? n_tiles : device_sm_count());
  cfg.blockDim = dim3(kPersistThreads);
  cfg.dynamicSmemBytes = kPersistSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, kp);
}

template <int TN, int EPI, bool DEEP>
cudaError_t launch_one(const CUtensorMap& tw, const CUtensorMap& tx, const KernelParams& kp, dim3 grid,
                       cudaStream_t stream, bool pdl) {
  using Cfg = GemmCfg<TN, DEEP>;
  auto kern = gemm_ws_kernel<TN, EPI, DEEP>;
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

int device_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

// One CTA per SM with the deep pipeline when the whole grid fits in one wave.  NFB_GEMM_DEEP=0 keeps the shallow
// pipeline (about 100 KB per CTA) for every size, so that the CTAs of two consecutive kernels fit on one SM and the
// next kernel's weight prefetch (programmatic dependent launch) can run under the current kernel.
bool deep_enabled() {
  static const bool enabled = [] {
    const char* e = getenv("NFB_GEMM_DEEP");
    return !(e != nullptr && e[0] == '0');
  }();
  return enabled;
}
bool use_deep(int tn, long long ctas) { return deep_enabled() && tn <= 64 && ctas <= device_sm_count(); }

template <int EPI>
cudaError_t launch_tn(int TN, const CUtensorMap& tw, const CUtensorMap& tx, const KernelParams& kp,
                      dim3 grid, cudaStream_t stream, bool pdl) {
  const bool deep = use_deep(TN, static_cast<long long>(grid.x) * grid.y * grid.z);
  switch (TN) {
    case 16: return deep ? launch_one<16, EPI, true>(tw, tx, kp, grid, stream, pdl)
                         : launch_one<16, EPI, false>(tw, tx, kp, grid, stream, pdl);
    case 32: return deep ? launch_one<32, EPI, true>(tw, tx, kp, grid, stream, pdl)
                         : launch_one<32, EPI, false>(tw, tx, kp, grid, stream, pdl);
    case 64: return deep ? launch_one<64, EPI, true>(tw, tx, kp, grid, stream, pdl)
                         : launch_one<64, EPI, false>(tw, tx, kp, grid, stream, pdl);
    case 128: return launch_one<128, EPI, false>(tw, tx, kp, grid, stream, pdl);
    default:
      return static_cast<long long>(grid.x) * grid.y * grid.z <= device_sm_count()
                 ? launch_one<256, EPI, true>(tw, tx, kp, grid, stream, pdl)
                 : launch_one<256, EPI, false>(tw, tx, kp, grid, stream, pdl);
  }
}

// Tensor maps are pure functions of (pointer, shape, box): cache them so the
// eager path does not re-encode on every call.
struct TmapKey {
  const void* base; uint64_t rows, cols, ld; uint32_t box_rows;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ k.rows; h = h * 1000003u ^ k.cols; h = h * 1000003u ^ k.ld;
    return h * 1000003u ^ k.box_rows;
  }
};
bool cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{base, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  CUtensorMap m;
  if (!make_tmap_2d(&m, TmapDtype::BF16, base, rows, cols, ld, box_rows, kBlockK, true)) return false;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

}  // namespace

void gemm_trace_enable(bool on) { g_trace_enabled = on; }
void gemm_timeline_begin() {
  g_trace_enabled = true;
  g_timeline_next = 0;
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_gemm_timeline) == cudaSuccess) cudaMemset(p, 0, sizeof(unsigned long long) * kTimelineSlots * kTimelineCtas * kTraceStamps);
}
int gemm_timeline_end(unsigned long long* host, int* n_slots, int* n_ctas) {
  g_trace_enabled = false;
  const int used = g_timeline_next < 0 ? 0 : (g_timeline_next < kTimelineSlots ? g_timeline_next : kTimelineSlots);
  g_timeline_next = -1;
  *n_slots = kTimelineSlots;
  *n_ctas = kTimelineCtas;
  if (host != nullptr)
    cudaMemcpyFromSymbol(host, g_gemm_timeline, sizeof(unsigned long long) * kTimelineSlots * kTimelineCtas * kTraceStamps);
  return used;
}
int gemm_trace_read(unsigned long long* host, int n_ctas) {
  if (n_ctas > kTraceCtas) n_ctas = kTraceCtas;
  cudaMemcpyFromSymbol(host, g_gemm_trace, sizeof(unsigned long long) * n_ctas * kTraceStamps);
  return kTraceStamps;
}

int gemm_tile_tokens(int T) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  if (T <= 128) return 128;
  return 256;
}

// Largest in-cluster split for a token tile: the leader needs (S-1) * TN * 512 bytes for the peers'
// fp32 tiles plus TN * 256 bytes for the SwiGLU exchange inside its idle pipeline stages.
int gemm_max_cluster(int tn) {
  switch (tn) {
    case 16: return 8;
    case 32: return 6;   // 5 stages x 20.5 KB hold 5 peer tiles of 16 KB plus the 8 KB SwiGLU exchange
    case 64: return 2;
    case 128: return 2;
    default: return 1;
  }
}

// How many clusters of `s` CTAs (along z) of one kernel instance can be resident at once.  A cluster lives inside
// one GPC, so this is not sm_count / s: with one CTA per SM, 17 clusters of 8 or 34 clusters of 4 do not fit and
// the grid runs in two waves.  Asked from the runtime once per (kernel, cluster size) and cached.
template <int TN, int EPI, bool DEEP>
int occupancy_clusters(int s) {
  using Cfg = GemmCfg<TN, DEEP>;
  auto kern = gemm_ws_kernel<TN, EPI, DEEP>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, s);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = s;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

template <int EPI>
int occupancy_clusters_tn(int tn, bool deep, int s) {
  switch (tn) {
    case 16: return deep ? occupancy_clusters<16, EPI, true>(s) : occupancy_clusters<16, EPI, false>(s);
    case 32: return deep ? occupancy_clusters<32, EPI, true>(s) : occupancy_clusters<32, EPI, false>(s);
    case 64: return deep ? occupancy_clusters<64, EPI, true>(s) : occupancy_clusters<64, EPI, false>(s);
    default: return 0;
  }
}

// 0 = unknown (no device, query failed): the caller then falls back to the SM-count estimate.
int max_active_clusters(int tn, int epi, bool deep, int s) {
  static std::mutex mu;
  static std::unordered_map<int, int> cache;
  const int key = ((tn * 16 + epi) * 2 + (deep ? 1 : 0)) * 16 + s;
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  int n = 0;
  switch (epi) {
    case kEpiStore: n = occupancy_clusters_tn<kEpiStore>(tn, deep, s); break;
    case kEpiResidual: n = occupancy_clusters_tn<kEpiResidual>(tn, deep, s); break;
    case kEpiSwiglu: n = occupancy_clusters_tn<kEpiSwiglu>(tn, deep, s); break;
    case kEpiPushAll: n = occupancy_clusters_tn<kEpiPushAll>(tn, deep, s); break;
    case kEpiRsAg: n = occupancy_clusters_tn<kEpiRsAg>(tn, deep, s); break;
    default: n = 0;
  }
  cache.emplace(key, n);
  return n;
}

int gemm_pick_splits(int T, int N, int K, int epi, int sm_count) {
  const int tn = gemm_tile_tokens(T);
  const int rows = epi == kEpiSwiglu ? N / 2 : N;
  const int tile_rows = epi == kEpiSwiglu ? 64 : kTileN;
  const int tiles = ((rows + tile_rows - 1) / tile_rows) * ((T + tn - 1) / tn);
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  const bool in_cluster = epi != kEpiPartial && epi != kEpiPushPartial;
  if (T > 256) return 1;
  if (!in_cluster) {
    const int slots = sm_count * (tn <= 64 ? 2 : 1);
    if (tiles >= slots) return 1;
    int s = slots / tiles;
    if (s > 8) s = 8;
    while (s > 1 && num_kb / s < 8) --s;
    const int per = (num_kb + s - 1) / s;
    return (num_kb + per - 1) / per;
  }
  // in-cluster split: aim for ONE wave of deep-pipeline CTAs (<= sm_count CTAs, one per SM)
  if (tiles >= sm_count || tn > 64) return 1;
  int s = sm_count / tiles;
  if (s > 8) s = 8;
  if (tn == 64 && s > 6) s = 6;
  if (tn == 64 && epi == kEpiRsAg && s > 5) s = 5;   // its row staging tile shares the pipeline stages
  if (!deep_enabled() && s > gemm_max_cluster(tn)) s = gemm_max_cluster(tn);
  // the largest split whose clusters are all resident at once (one wave), that leaves every split at least eight
  // k-blocks and no split empty
  for (; s > 1; --s) {
    if (num_kb / s < 8) continue;
    if ((num_kb + s - 1) / s * (s - 1) >= num_kb) continue;
    const bool deep = use_deep(tn, static_cast<long long>(tiles) * s);
    if (!deep && s > gemm_max_cluster(tn)) continue;
    const int fit = max_active_clusters(tn, epi, deep, s);
    if (fit > 0 && fit < tiles) continue;
    break;
  }
  return s < 1 ? 1 : s;
}

const char* gemm_bf16(const GemmArgs& a) {
  if (a.T <= 0 || a.N <= 0 || a.K <= 0) return "gemm_bf16: empty problem";
  if ((a.K % 8) || (a.ldw % 8) || (a.ldx % 8)) return "gemm_bf16: K and leading dims must be multiples of 8";
  if ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.x)) & 15)
    return "gemm_bf16: operands must be 16-byte aligned";
  if ((a.N & 1) || (a.ldo & 1)) return "gemm_bf16: N and ldo must be even";
  const int tn = gemm_tile_tokens(static_cast<int>(a.T));
  const bool global_split = a.epi == kEpiPartial || a.epi == kEpiPushPartial;
  KernelParams kp = {};
  kp.trace = g_trace_enabled ? 1 : 0;
  if (g_trace_enabled && g_timeline_next >= 0) kp.trace = 2 + (g_timeline_next++ % kTimelineSlots);
  kp.T = static_cast<int>(a.T); kp.N = static_cast<int>(a.N); kp.K = static_cast<int>(a.K);
  kp.num_kb = (kp.K + kBlockK - 1) / kBlockK;
  int splits = a.splits < 1 ? 1 : a.splits;
  if (splits > kp.num_kb) splits = kp.num_kb;
  kp.kb_per_split = (kp.num_kb + splits - 1) / splits;
  if ((kp.num_kb + kp.kb_per_split - 1) / kp.kb_per_split != splits || splits != (a.splits < 1 ? 1 : a.splits))
    return "gemm_bf16: split count leaves an empty split";
  kp.cluster = 1;
  if (!global_split && splits > 1) {
    const long long ctas = static_cast<long long>((kp.N + kTileN - 1) / kTileN) * ((kp.T + tn - 1) / tn) * splits;
    const bool deep = use_deep(tn, ctas);  // (SwiGLU has more tiles: checked against the shallow limit)
    const int cap = (deep && a.epi != kEpiSwiglu) ? (tn == 64 ? 6 : 8) : gemm_max_cluster(tn);
    if (splits > cap) return "gemm_bf16: in-cluster split exceeds the tile's limit";
    kp.cluster = splits;
  }
  if (a.epi == kEpiPushPartial || a.epi == kEpiPushAll || a.epi == kEpiRsAg) {
    if (a.world < 1 || a.world > kMaxRanks || a.rank < 0 || a.rank >= a.world) return "gemm_bf16: bad rank/world";
    kp.rank = a.rank;
    kp.world = a.world;
    for (int r = 0; r < a.world; ++r) {
      if (a.peer_recv[r] == nullptr || (a.peer_flag[r] == nullptr && a.epi != kEpiRsAg))
        return "gemm_bf16: missing peer pointer";
      kp.peer_recv[r] = a.peer_recv[r];
      kp.peer_flag[r] = a.peer_flag[r];
    }
  }
  if (a.epi == kEpiPushPartial) {
    if (kp.N % a.world || (kp.N / a.world) % kTileN) return "gemm_bf16: N / world must be a multiple of 128";
    kp.slice_cols = kp.N / a.world;
  }
  if (a.epi == kEpiPushAll) {
    if (a.call_idx == nullptr || a.T_cap < kp.T) return "gemm_bf16: push-all needs the call counter and T <= T_cap";
    kp.call_idx = a.call_idx;
    kp.T_cap = a.T_cap;
  }
  if (a.epi == kEpiRsAg) {
    if (kp.N % a.world || (kp.N / a.world) % kTileN) return "gemm_bf16: N / world must be a multiple of 128";
    if (kp.N / kTileN > kRsMaxTiles || kp.N / kTileN > kRsSsStride)
      return "gemm_bf16: too many column tiles for the reduce-scatter bookkeeping";
    if ((kp.T + tn - 1) / tn > kRsMaxTokenTiles || a.T_cap < kp.T) return "gemm_bf16: too many rows for the receive buffer";
    if (a.rs_state == nullptr || a.rs_phase < 0 || a.rs_phase > 2 || (a.ld_resid % 8))
      return "gemm_bf16: reduce-scatter epilogue needs its state, a phase in 0..2 and a residual stride that is a multiple of 8";
    if (kp.T > 128) return "gemm_bf16: reduce-scatter epilogue is for decode sizes (T <= 128)";
    // the fp32 tile is staged behind the split-K landing zone inside the pipeline stages
    if (tn == 64 && splits > 5) return "gemm_bf16: reduce-scatter epilogue with a 64-token tile allows at most 5 splits";
    for (int r = 0; r < a.world; ++r)
      if (reinterpret_cast<uintptr_t>(a.peer_x[r]) & 15) return "gemm_bf16: residual buffers must be 16-byte aligned";
    // an owner CTA waits for peers while it holds its SM: every CTA of the grid has to be resident at once
    if (a.rs_phase == 0 && static_cast<long long>(kp.N / kTileN) * ((kp.T + tn - 1) / tn) * splits > device_sm_count())
      return "gemm_bf16: reduce-scatter epilogue needs a grid that is resident at once";
    kp.slice_cols = kp.N / a.world;
    kp.T_cap = a.T_cap;
    kp.ld_resid = a.ld_resid;
    kp.rs_state = a.rs_state;
    kp.rs_phase = a.rs_phase;
    for (int r = 0; r < a.world; ++r) {
      if (a.peer_x[r] == nullptr || a.peer_ss[r] == nullptr || a.peer_xflag[r] == nullptr)
        return "gemm_bf16: missing residual pointer of a rank";
      kp.peer_x[r] = static_cast<__nv_bfloat16*>(a.peer_x[r]);
      kp.peer_recv_ll[r] = reinterpret_cast<uint2*>(a.peer_recv[r]);
      kp.peer_ss[r] = a.peer_ss[r];
      kp.peer_xflag[r] = a.peer_xflag[r];
    }
  }
  if (a.gather.flag != nullptr) {
    if (a.epi != kEpiStore && a.epi != kEpiSwiglu) return "gemm_bf16: the gathered input needs the store or SwiGLU epilogue";
    if (a.gather.target == nullptr || a.gather.ss == nullptr || a.gather.ss_tiles < 1 ||
        a.gather.ss_tiles > kRsSsStride || a.gather.n_features < 1 || kp.T > 256)
      return "gemm_bf16: bad gathered-input description";
    kp.g_flag = a.gather.flag;
    kp.g_target = a.gather.target;
    kp.g_ss = a.gather.ss;
    kp.g_tiles = a.gather.ss_tiles;
    kp.g_inv_n = 1.f / static_cast<float>(a.gather.n_features);
    kp.g_eps = a.gather.eps;
  }
  if (a.conv.state != nullptr) {
    if (a.epi != kEpiStore || a.bias != nullptr || a.act != kActNone)
      return "gemm_bf16: the conv epilogue needs the plain store epilogue";
    if (a.conv.w == nullptr || a.conv.slot == nullptr || a.conv.out == nullptr || a.conv.C <= 0 ||
        a.conv.C % kTileN || a.conv.C > kp.N || kp.T > 256)
      return "gemm_bf16: bad conv description (C must be a multiple of 128 within N, decode sizes only)";
    if (reinterpret_cast<uintptr_t>(a.conv.w) & 7) return "gemm_bf16: conv weights must be 8-byte aligned";
    kp.conv_w = static_cast<const __nv_bfloat16*>(a.conv.w);
    kp.conv_state = static_cast<__nv_bfloat16*>(a.conv.state);
    kp.conv_slot = a.conv.slot;
    kp.conv_out = static_cast<__nv_bfloat16*>(a.conv.out);
    kp.conv_C = a.conv.C;
  }
  kp.swiglu_half = a.epi == kEpiSwiglu ? kp.N / 2 : 0;
  if (a.epi == kEpiSwiglu && (kp.N % 4)) return "gemm_bf16: SwiGLU needs N % 4 == 0";
  kp.out = static_cast<__nv_bfloat16*>(a.out); kp.ldo = a.ldo;
  kp.resid = static_cast<const __nv_bfloat16*>(a.resid); kp.ldr = a.ldr;
  kp.bias = a.bias; kp.act = a.epi == kEpiStore ? a.act : kActNone; kp.partial = a.partial; kp.status = a.status;
  if (a.epi == kEpiResidual && a.resid == nullptr) return "gemm_bf16: residual epilogue without residual";
  if (a.epi == kEpiPartial && a.partial == nullptr) return "gemm_bf16: split-K without workspace";
  const bool needs_out = a.epi == kEpiStore || a.epi == kEpiResidual || a.epi == kEpiSwiglu;
  if (needs_out && a.out == nullptr) return "gemm_bf16: no output";

  CUtensorMap tw, tx;
  if (!cached_tmap(&tw, a.w, a.N, a.K, a.ldw, 64)) return "gemm_bf16: weight tensor map rejected";
  if (!cached_tmap(&tx, a.x, a.T, a.K, a.ldx, tn)) return "gemm_bf16: activation tensor map rejected";

  dim3 grid;
  grid.x = a.epi == kEpiSwiglu ? (kp.swiglu_half + 63) / 64 : (kp.N + kTileN - 1) / kTileN;
  grid.y = (kp.T + tn - 1) / tn;
  grid.z = splits;
  if (a.prefetch != nullptr && a.prefetch_bytes > 0 && (reinterpret_cast<uintptr_t>(a.prefetch) & 15) == 0) {
    const long long ctas = static_cast<long long>(grid.x) * grid.y * grid.z;
    long long per = (a.prefetch_bytes + ctas - 1) / ctas;
    per = (per + 4095) & ~4095LL;                 // whole 4 KB pieces per CTA
    if (per > (1 << 20)) per = 1 << 20;           // at most 1 MB per CTA
    kp.pf_ptr = static_cast<const uint8_t*>(a.prefetch);
    kp.pf_bytes = a.prefetch_bytes;
    kp.pf_per_cta = static_cast<int>(per);
  }
  cudaError_t e;
  // prefill-sized problems with more tiles than SMs: persistent kernel, epilogue overlapped with the next main loop
  // (NFB_GEMM_PERSISTENT=0 keeps the one-tile-per-CTA kernel for every size)
  static const bool persistent_enabled = [] {
    const char* e = getenv("NFB_GEMM_PERSISTENT");
    return !(e != nullptr && e[0] == '0');
  }();
  if (tn == kPersistTN && splits == 1 && persistent_enabled && !g_trace_enabled && a.gather.flag == nullptr &&
      a.conv.state == nullptr &&
      (a.epi == kEpiStore || a.epi == kEpiResidual || a.epi == kEpiSwiglu) &&
      static_cast<long long>(grid.x) * grid.y > device_sm_count()) {
    const int n_tiles = static_cast<int>(grid.x * grid.y);
    switch (a.epi) {
      case kEpiStore: e = launch_persist<kEpiStore>(tw, tx, kp, n_tiles, a.stream, a.pdl); break;
      case kEpiResidual: e = launch_persist<kEpiResidual>(tw, tx, kp, n_tiles, a.stream, a.pdl); break;
      default: e = launch_persist<kEpiSwiglu>(tw, tx, kp, n_tiles, a.stream, a.pdl); break;
    }
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  }
  switch (a.epi) {
    case kEpiStore: e = launch_tn<kEpiStore>(tn, tw, tx, kp, grid, a.stream, a.pdl); break;
    case kEpiResidual: e = launch_tn<kEpiResidual>(tn, tw, tx, kp, grid, a.stream, a.pdl); break;
    case kEpiSwiglu: e = launch_tn<kEpiSwiglu>(tn, tw, tx, kp, grid, a.stream, a.pdl); break;
    case kEpiPartial: e = launch_tn<kEpiPartial>(tn, tw, tx, kp, grid, a.stream, a.pdl); break;
    case kEpiPushPartial: e = launch_tn<kEpiPushPartial>(tn, tw, tx, kp, grid, a.stream, a.pdl); break;
    case kEpiPushAll: e = launch_tn<kEpiPushAll>(tn, tw, tx, kp, grid, a.stream, a.pdl); break;
    case kEpiRsAg: e = launch_tn<kEpiRsAg>(tn, tw, tx, kp, grid, a.stream, a.pdl); break;
    default: return "gemm_bf16: unknown epilogue";
  }
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
