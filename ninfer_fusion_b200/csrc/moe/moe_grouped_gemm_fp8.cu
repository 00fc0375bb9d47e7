// Grouped expert GEMM over fp8 (e4m3) weights with one fp32 scale per 128 x 128 weight block and one fp32 scale per
// (activation row, 128-wide k-block):  out[row, n] = sum_kb  sx[row, kb] * sw[e, n/128, kb] * dot_kb(x_q[row], W_q[e, n]).
//
// The scales change every 128 values of K, so the tensor core cannot accumulate across k-blocks in one TMEM
// accumulator.  Two-level accumulation instead: tcgen05.mma (kind::f8f6f4) produces the 128-deep partial products of
// one k-block into one of TWO TMEM buffers; four epilogue warps read that buffer with tcgen05.ld, apply
// sx * sw and add into fp32 registers while the tensor core already works on the next k-block in the other
// buffer.  Warp roles: 0 = TMA producer, 1 = MMA issuer, 2..5 = scale-and-accumulate + final epilogue
// (SwiGLU or "return" exactly as in the bf16 kernel, moe_grouped_gemm.cu).
//
// WIDE variant (decode-sized tiles, num_kb * TN <= 512): every k-block gets TMEM columns of its own, so the MMA issuer
// never waits for the accumulate warps and the weight stream runs at the pace of TMA alone; the accumulate warps follow
// one mbarrier per k-block and read the tile's activation scales from shared memory.  With two buffers the issuer is at
// most one k-block ahead, and a 128-deep MMA is far shorter than the read-scale-add of one k-block: the hand-shake,
// not the bytes, set the pace of the kernel at a few tokens per expert.
//
// The reference has no fp8 block-scaled expert format (its routed banks are Q4+Q5 / Q4+Q6 / W8 row-split,
// src/ops/sparse_moe); the container registers it as FP8_E4M3FN_BLOCK128_F32S / blockscale-128x128-f32-v1.
#include "moe.h"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "../comm/peer_sync.cuh"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "../kv/codec.cuh"

namespace nfb {

namespace {

constexpr int kKBytes = 128;           // one k-block: 128 fp8 values = one swizzle row
constexpr int kTileN = 128;
constexpr int kWTileBytes = kTileN * kKBytes;
constexpr int kThreads = 192;

constexpr int kWideMaxKb = 32;         // WIDE: one accumulator and one mbarrier per k-block
constexpr int kWideCols = 512;

template <int TN>
struct Fp8Cfg {
  static constexpr int kStages = TN <= 32 ? 6 : 4;
  static constexpr int kStageBytes = kWTileBytes + TN * kKBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kTmemCols = 2 * TN < 32 ? 32 : 2 * TN;
};

struct Fp8Params {
  int num_kb;
  int rows_per_expert;
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const MoeState* state;
  const float* w_scale;   // [experts, rows_per_expert / 128, num_kb]
  const float* x_scale;   // [cap, num_kb]
  __nv_bfloat16* out;
  long long ldo;
  int world;
  const int* recv_meta;
  __nv_bfloat16* peer_ret[kMoeMaxRanks];
  unsigned int* peer_ret_flag[kMoeMaxRanks];
  int* status;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int TN, int EPI, bool WIDE>
__global__ void __launch_bounds__(kThreads) moe_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                                                 const __grid_constant__ CUtensorMap tmap_x,
                                                                 const Fp8Params p) {
  using Cfg = Fp8Cfg<TN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  constexpr int kAccBars = WIDE ? kWideMaxKb : 2;
  __shared__ __align__(8) uint64_t bar_acc_full[kAccBars];
  __shared__ __align__(8) uint64_t bar_acc_free[2];
  __shared__ float sx_s[WIDE ? kWideCols : 1];   // WIDE: activation scales of the tile, [token][k-block]
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int meta_s[TN];
  __shared__ int src_cnt[kMoeMaxRanks];
  __shared__ float up_s[TN * 64];          // SwiGLU exchange between the up-row and gate-row warps
  __shared__ int epi_ok;                   // common verdict of the four epilogue warps

  if (static_cast<int>(blockIdx.y) >= p.state->n_tiles) return;
  const int expert = p.tile_expert[blockIdx.y];
  const int row0 = p.tile_row0[blockIdx.y];
  const int rows = p.tile_rows[blockIdx.y];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int half = p.rows_per_expert / 2;
  const int n0 = (EPI == kMoeEpiSwiglu) ? blockIdx.x * 64 : blockIdx.x * kTileN;
  const int num_kb = p.num_kb;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < kAccBars; ++b) mbar_init(smem_u32(&bar_acc_full[b]), 1);
    for (int b = 0; b < 2; ++b) mbar_init(smem_u32(&bar_acc_free[b]), 4);   // one arrival per epilogue warp
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (threadIdx.x < kMoeMaxRanks) src_cnt[threadIdx.x] = 0;
  if (threadIdx.x == 0) epi_ok = 1;
  if (EPI == kMoeEpiReturn) {
    for (int j = threadIdx.x; j < TN; j += kThreads) meta_s[j] = j < rows ? p.recv_meta[row0 + j] : -1;
  }
  // WIDE: num_kb * TN columns, rounded up to a power of two (the host admits the variant only up to 512)
  uint32_t tmem_cols = Cfg::kTmemCols;
  if (WIDE) {
    tmem_cols = 32;
    while (tmem_cols < static_cast<uint32_t>(num_kb * TN)) tmem_cols <<= 1;
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_base_slot), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (elect_one()) {
      // ---------------- TMA producer ----------------
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const int wrow = expert * p.rows_per_expert;
      const int row_a = wrow + n0;
      const int row_b = (EPI == kMoeEpiSwiglu) ? wrow + half + n0 : wrow + n0 + 64;
      int it = 0;
      for (; it < num_kb; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (it >= kStages &&
            !mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, kStatusEmptyWaitTimeout))
          break;
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t dst = smem_base + s * Cfg::kStageBytes;
        const int kx = it * kKBytes;
        mbar_expect_tx(full, Cfg::kStageBytes);
        tma_load_2d(dst, &tmap_w, full, kx, row_a, pol_w);
        tma_load_2d(dst + 64 * 128, &tmap_w, full, kx, row_b, pol_w);
        tma_load_2d(dst + kWTileBytes, &tmap_x, full, kx, row0, pol_x);
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
      // ---------------- MMA issuer: one TMEM buffer per k-block, alternating ----------------
      constexpr uint32_t idesc = umma_idesc(kTileN, TN, 0, 0);
      for (int it = 0; it < num_kb; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        const int b = WIDE ? it : (it & 1);
        const int use = it >> 1;   // how often buffer b has been filled before
        if (!WIDE && use > 0 &&
            !mbar_wait(smem_u32(&bar_acc_free[b]), (use - 1) & 1, &abort_flag, p.status, kStatusAccumWaitTimeout))
          break;
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag, p.status, kStatusTmaWaitTimeout)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
        const uint64_t a_desc = umma_desc_k_sw128(a_addr);
        const uint64_t b_desc = umma_desc_k_sw128(a_addr + kWTileBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f8f6f4(tmem_base + b * TN, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_empty[s]));
        tc_commit(smem_u32(&bar_acc_full[b]));
      }
    }
    __syncwarp();
  } else {
    // ---------------- scale-and-accumulate warps (TMEM lane quadrant = warp % 4) ----------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // TMEM lane = row of the 128-row tile
    const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    // weight-scale block of this row: SwiGLU tiles hold 64 gate rows (lanes 0..63) and 64 up rows (lanes 64..127)
    int wrow_in_expert;
    if (EPI == kMoeEpiSwiglu) wrow_in_expert = r < 64 ? n0 + r : half + n0 + (r - 64);
    else wrow_in_expert = n0 + r;
    const float* sw = p.w_scale + (static_cast<long long>(expert) * (p.rows_per_expert / 128) + wrow_in_expert / 128) * num_kb;
    const float* sx = p.x_scale + static_cast<long long>(row0) * num_kb;
    float acc[TN];
#pragma unroll
    for (int c = 0; c < TN; ++c) acc[c] = 0.f;
    bool ok = true;
    if (WIDE) {
      // the tile's rows are consecutive in x_scale: rows * num_kb floats, zero beyond the tile's live rows
      for (int i = threadIdx.x - 64; i < TN * num_kb; i += 128) sx_s[i] = i < rows * num_kb ? sx[i] : 0.f;
      epi_bar_sync();
    }
    for (int it = 0; it < num_kb; ++it) {
      const int b = WIDE ? it : (it & 1);
      const int use = WIDE ? 0 : (it >> 1);
      if (!mbar_wait(smem_u32(&bar_acc_full[b]), use & 1, &abort_flag, p.status, kStatusAccumWaitTimeout)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const float swk = sw[it];
#pragma unroll
      for (int c = 0; c < TN; c += 16) {
        if (c < rows) {
          uint32_t v[16];
          tmem_ld_x16(lane_taddr + b * TN + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float s;
            if (WIDE) s = swk * sx_s[(c + j) * num_kb + it];
            else s = (c + j < rows) ? swk * sx[(c + j) * num_kb + it] : 0.f;
            acc[c + j] += __uint_as_float(v[j]) * s;
          }
        }
      }
      if (!WIDE) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_acc_free[b]));
      }
    }

    // ---------------- final epilogue from the register accumulators ----------------
    // one verdict for all four warps, so that the named barriers below are never divergent
    if (!ok || abort_flag) atomicAnd(&epi_ok, 0);
    epi_bar_sync();
    if (epi_ok) {
      if constexpr (EPI == kMoeEpiSwiglu) {
        if (r >= 64) {
#pragma unroll
          for (int c = 0; c < TN; ++c) up_s[c * 64 + (r - 64)] = acc[c];
        }
        epi_bar_sync();
        if (r < 64) {
          const int n = n0 + r;
#pragma unroll
          for (int m = 0; m < TN / 2; ++m) {
            float a[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const float g = acc[2 * m + h];
              a[h] = g / (1.f + __expf(-g)) * up_s[(2 * m + h) * 64 + r];
            }
            const float send = (lane & 1) ? a[0] : a[1];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
            const int tl = 2 * m + (lane & 1);
            const int ne = n & ~1;
            if (tl < rows && ne < half) {
              const uint32_t packed = (lane & 1) ? pack_bf16x2(recv, a[1]) : pack_bf16x2(a[0], recv);
              *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(row0 + tl) * p.ldo + ne) = packed;
            }
          }
        }
      } else {
        const int n = n0 + r;
        const int N = p.rows_per_expert;
#pragma unroll
        for (int m = 0; m < TN / 2; ++m) {
          const float a0 = acc[2 * m], a1 = acc[2 * m + 1];
          const float send = (lane & 1) ? a0 : a1;
          const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
          const int tl = 2 * m + (lane & 1);
          const int ne = n & ~1;
          if (tl < rows && ne < N) {
            const int meta = meta_s[tl];
            const int src = meta >> 24;
            const long long a = meta & 0xffffff;
            const float lo = (lane & 1) ? recv : a0;
            const float hi = (lane & 1) ? a1 : recv;
            *reinterpret_cast<uint32_t*>(p.peer_ret[src] + a * N + ne) = pack_bf16x2(lo, hi);
          }
        }
        const int t = threadIdx.x - 64;   // 0..127 over the four epilogue warps
        if (t < rows) atomicAdd(&src_cnt[meta_s[t] >> 24], 1);
        if (p.world == 1) __threadfence(); else __threadfence_system();
        epi_bar_sync();
        if (t < p.world && src_cnt[t] > 0) {
          if (p.world == 1) red_release_gpu_add(p.peer_ret_flag[t], static_cast<uint32_t>(src_cnt[t]));
          else red_release_sys_add(p.peer_ret_flag[t], static_cast<uint32_t>(src_cnt[t]));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, tmem_cols);
}

// ---- activation quantiser: per row and 128-wide k-block, scale = amax / 448 ----
__global__ void __launch_bounds__(128) quant_rows_block128_kernel(const __nv_bfloat16* x, long long ldx, int K,
                                                                  const MoeState* state, int max_rows, uint8_t* codes,
                                                                  float* scales) {
  const int row = blockIdx.x;
  const int live = state != nullptr ? min(max_rows, state->total_rows) : max_rows;
  if (row >= live) return;
  const int num_kb = K / 128;
  // one warp per k-block: lane holds 4 consecutive values
  for (int kb = threadIdx.x >> 5; kb < num_kb; kb += 4) {
    const int lane = threadIdx.x & 31;
    const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<long long>(row) * ldx + kb * 128 + lane * 4);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float v[4] = {__bfloat162float(p2[0].x), __bfloat162float(p2[0].y), __bfloat162float(p2[1].x), __bfloat162float(p2[1].y)};
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float sc = fmaxf(amax / 448.f, 1e-12f);
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) packed |= static_cast<uint32_t>(float_to_e4m3(__fdiv_rn(v[i], sc))) << (8 * i);
    *reinterpret_cast<uint32_t*>(codes + static_cast<long long>(row) * K + kb * 128 + lane * 4) = packed;
    if (lane == 0) scales[static_cast<long long>(row) * num_kb + kb] = sc;
  }
}

template <int TN, int EPI, bool WIDE>
cudaError_t launch_one(const CUtensorMap& tw, const CUtensorMap& tx, const Fp8Params& kp, dim3 grid, cudaStream_t stream) {
  using Cfg = Fp8Cfg<TN>;
  auto kern = moe_gemm_fp8_kernel<TN, EPI, WIDE>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(tw, tx, kp);
  return cudaGetLastError();
}

template <int EPI>
cudaError_t launch_tn(int tn, const CUtensorMap& tw, const CUtensorMap& tx, const Fp8Params& kp, dim3 grid,
                      cudaStream_t stream) {
  static const bool wide_on = [] {
    const char* e = std::getenv("NFB_MOE_FP8_WIDE");
    return e == nullptr || e[0] != '0';
  }();
  const bool wide = wide_on && kp.num_kb <= kWideMaxKb && kp.num_kb * tn <= kWideCols;
  switch (tn) {
    case 16: return wide ? launch_one<16, EPI, true>(tw, tx, kp, grid, stream) : launch_one<16, EPI, false>(tw, tx, kp, grid, stream);
    case 32: return wide ? launch_one<32, EPI, true>(tw, tx, kp, grid, stream) : launch_one<32, EPI, false>(tw, tx, kp, grid, stream);
    case 64: return wide ? launch_one<64, EPI, true>(tw, tx, kp, grid, stream) : launch_one<64, EPI, false>(tw, tx, kp, grid, stream);
    default: return launch_one<128, EPI, false>(tw, tx, kp, grid, stream);
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

}  // namespace

const char* moe_quant_rows_block128(const __nv_bfloat16* x, long long ldx, int max_rows, int K, const MoeState* state,
                                    uint8_t* codes, float* scales, cudaStream_t stream) {
  if (max_rows <= 0) return nullptr;
  if (K % 128 || ldx % 4 || (reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(codes) & 3))
    return "moe_quant_rows_block128: K must be a multiple of 128, rows 8-byte aligned";
  quant_rows_block128_kernel<<<max_rows, 128, 0, stream>>>(x, ldx, K, state, max_rows, codes, scales);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* moe_gemm_fp8(const MoeGemmArgs& a) {
  if (a.n_local_experts <= 0 || a.rows_per_expert <= 0 || a.K <= 0 || a.cap <= 0) return "moe_gemm_fp8: empty problem";
  if ((a.K % 128) || (a.ldw % 16) || (a.ldx % 16)) return "moe_gemm_fp8: K must be a multiple of 128, leading dims of 16 bytes";
  if ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.x)) & 15) return "moe_gemm_fp8: operands must be 16-byte aligned";
  int tn = a.tile_tokens;
  if (tn != 16 && tn != 32 && tn != 64 && tn != 128) return "moe_gemm_fp8: token tile must be 16, 32, 64 or 128";
  if (a.max_tiles < 1 || a.max_tiles > 65535) return "moe_gemm_fp8: tile bound out of range";
  if (a.tile_expert == nullptr || a.state == nullptr || a.w_scale == nullptr || a.x_scale == nullptr)
    return "moe_gemm_fp8: missing tile table or scales";
  if (a.rows_per_expert % 128) return "moe_gemm_fp8: expert rows must be a multiple of 128";
  Fp8Params kp = {};
  kp.num_kb = static_cast<int>(a.K / 128);
  kp.rows_per_expert = static_cast<int>(a.rows_per_expert);
  kp.tile_expert = a.tile_expert; kp.tile_row0 = a.tile_row0; kp.tile_rows = a.tile_rows; kp.state = a.state;
  kp.w_scale = a.w_scale; kp.x_scale = a.x_scale; kp.status = a.status;
  dim3 grid;
  grid.y = a.max_tiles;
  if (a.epi == kMoeEpiSwiglu) {
    if ((a.rows_per_expert / 2) % 128) return "moe_gemm_fp8: SwiGLU needs the intermediate size in multiples of 128";
    if (a.out == nullptr || (a.ldo & 1)) return "moe_gemm_fp8: no output";
    kp.out = static_cast<__nv_bfloat16*>(a.out); kp.ldo = a.ldo;
    grid.x = static_cast<unsigned>(a.rows_per_expert / 2 / 64);
  } else if (a.epi == kMoeEpiReturn) {
    if (a.world < 1 || a.world > kMoeMaxRanks || a.recv_meta == nullptr) return "moe_gemm_fp8: bad return set-up";
    kp.world = a.world; kp.recv_meta = a.recv_meta;
    for (int r = 0; r < a.world; ++r) {
      if (a.peer_ret[r] == nullptr || a.peer_ret_flag[r] == nullptr) return "moe_gemm_fp8: missing peer pointer";
      kp.peer_ret[r] = a.peer_ret[r]; kp.peer_ret_flag[r] = a.peer_ret_flag[r];
    }
    grid.x = static_cast<unsigned>(a.rows_per_expert / 128);
  } else {
    return "moe_gemm_fp8: unknown epilogue";
  }
  CUtensorMap tw, tx;
  if (!cached_tmap(&tw, a.w, static_cast<uint64_t>(a.n_local_experts) * a.rows_per_expert, a.K, a.ldw, 64))
    return "moe_gemm_fp8: weight tensor map rejected";
  if (!cached_tmap(&tx, a.x, a.cap, a.K, a.ldx, tn)) return "moe_gemm_fp8: activation tensor map rejected";
  cudaError_t e = a.epi == kMoeEpiSwiglu ? launch_tn<kMoeEpiSwiglu>(tn, tw, tx, kp, grid, a.stream)
                                         : launch_tn<kMoeEpiReturn>(tn, tw, tx, kp, grid, a.stream);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
