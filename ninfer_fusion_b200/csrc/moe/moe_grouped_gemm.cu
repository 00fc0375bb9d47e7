// Grouped expert GEMM for sm_100a: for every token tile of the expert-sorted receive buffer,
// out[rows, N_e] = x[rows, K] * W_e[N_e, K]^T with the expert taken from a device-side tile table.
//
// Same weight-stationary shape as the dense kernel (gemm_bf16.cu): 128 rows of W_e are the UMMA A
// operand, the tile's tokens the N operand (16..256), TMA -> 128B-swizzled shared memory ->
// tcgen05.mma -> TMEM -> tcgen05.ld epilogue.  blockIdx.y walks a fixed upper bound of token tiles
// and CTAs beyond the device-side tile count leave at once, so the launch is graph-capturable although
// the routing is data dependent.  Epilogues:
//   SwiGLU : W_e = [gate; up]; 64 gate rows + the matching 64 up rows form one 128-row tile;
//   return : each output row is stored into the return buffer of the rank that owns the token
//            (peer stores over NVLink), then that rank's arrival counter is advanced by the number
//            of rows it got from this CTA -- the combine all-to-all happens inside the GEMM.
//
// Reference: src/ops/sparse_moe/prefill/sparse_moe_prefill_kernels.cu (grouped mma.sync 64x64x64
// gate_up/down kernels after a select/scan/permute chain) and decode/sparse_moe_decode_kernels.cu.
#include "moe.h"

#include <mutex>
#include <unordered_map>

#include "../comm/peer_sync.cuh"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"

namespace nfb {

namespace {

constexpr int kBlockK = 64;
constexpr int kTileN = 128;
constexpr int kWTileBytes = kTileN * 128;

template <int TN>
struct MoeCfg {
  static constexpr int kStages = TN <= 32 ? 6 : 4;
  static constexpr int kXTileBytes = TN * 128;
  static constexpr int kStageBytes = kWTileBytes + kXTileBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kTmemCols = TN < 32 ? 32 : TN;
};

struct MoeKernelParams {
  int num_kb;
  int rows_per_expert;  // N_e
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const MoeState* state;
  __nv_bfloat16* out;
  long long ldo;
  int world;
  const int* recv_meta;
  __nv_bfloat16* peer_ret[kMoeMaxRanks];
  unsigned int* peer_ret_flag[kMoeMaxRanks];
  int* status;
};

template <int TN, int EPI>
__global__ void __launch_bounds__(128) moe_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                                        const __grid_constant__ CUtensorMap tmap_x,
                                                        const MoeKernelParams p) {
  using Cfg = MoeCfg<TN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_accum;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int meta_s[TN];
  __shared__ int src_cnt[kMoeMaxRanks];

  if (static_cast<int>(blockIdx.y) >= p.state->n_tiles) return;  // uniform: nothing allocated yet
  const int expert = p.tile_expert[blockIdx.y];
  const int row0 = p.tile_row0[blockIdx.y];
  const int rows = p.tile_rows[blockIdx.y];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int half = p.rows_per_expert / 2;
  const int n0 = (EPI == kMoeEpiSwiglu) ? blockIdx.x * 64 : blockIdx.x * kTileN;  // row inside the expert
  const int num_it = p.num_kb;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_accum), 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (threadIdx.x < kMoeMaxRanks) src_cnt[threadIdx.x] = 0;
  if (EPI == kMoeEpiReturn) {
    for (int j = threadIdx.x; j < TN; j += 128) meta_s[j] = j < rows ? p.recv_meta[row0 + j] : -1;
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_base_slot), Cfg::kTmemCols);
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
      for (; it < num_it; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (it >= kStages &&
            !mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, &abort_flag, p.status, kStatusEmptyWaitTimeout))
          break;
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t dst = smem_base + s * Cfg::kStageBytes;
        const int kx = it * kBlockK;
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
        for (int k = 0; k < kBlockK / 16; ++k)
          tc_mma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
        tc_commit(smem_u32(&bar_empty[s]));
      }
      if (ok) tc_commit(smem_u32(&bar_accum));
    }
    __syncwarp();
  }

  // ---------------- epilogue ----------------
  const bool have_acc = mbar_wait(smem_u32(&bar_accum), 0, &abort_flag, p.status, kStatusAccumWaitTimeout);
  tc_fence_after();
  const int epilogue_ok = __syncthreads_and(have_acc && !abort_flag);
  const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  constexpr int kChunk = 16;
  auto load_acc = [&](int c, float* acc) {
    uint32_t v[kChunk];
    tmem_ld_x16(lane_taddr + c, v);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < kChunk; ++j) acc[j] = __uint_as_float(v[j]);
  };

  if (epilogue_ok) {
    if constexpr (EPI == kMoeEpiSwiglu) {
      // lanes 0..63 hold gate rows, lanes 64..127 the matching up rows; exchange through the idle stages
      float* up_s = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));  // [TN][64]
      if (warp >= 2) {
        const int r = (warp - 2) * 32 + lane;
        for (int c = 0; c < TN; c += kChunk) {
          if (c >= rows) break;
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
          if (c >= rows) break;
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
            const int tl = c + 2 * m + (lane & 1);
            const int ne = n & ~1;
            if (tl < rows && ne < half) {
              const uint32_t packed = (lane & 1) ? pack_bf16x2(recv, a[1]) : pack_bf16x2(a[0], recv);
              *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(row0 + tl) * p.ldo + ne) = packed;
            }
          }
        }
      }
    } else {
      const int n = n0 + warp * 32 + lane;
      const int N = p.rows_per_expert;
      for (int c = 0; c < TN; c += kChunk) {
        if (c >= rows) break;
        float v[kChunk];
        load_acc(c, v);
#pragma unroll
        for (int m = 0; m < kChunk / 2; ++m) {
          const float a0 = v[2 * m], a1 = v[2 * m + 1];
          const float send = (lane & 1) ? a0 : a1;
          const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
          const int tl = c + 2 * m + (lane & 1);
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
      }
      // one arrival unit per returned row of this 128-column tile
      if (threadIdx.x < rows) atomicAdd(&src_cnt[meta_s[threadIdx.x] >> 24], 1);
      if (TN > 128 && threadIdx.x + 128 < rows) atomicAdd(&src_cnt[meta_s[threadIdx.x + 128] >> 24], 1);
      // one GPU: device-scope fence and counter (a prefill chunk has thousands of tiles signalling one word)
      // (several ranks: the block barrier orders all stores before the signalling threads, whose system-scope fence +
      // release is cumulative over them)
      if (p.world == 1) __threadfence();
      __syncthreads();
      if (threadIdx.x < p.world && src_cnt[threadIdx.x] > 0) {
        if (p.world == 1) {
          red_release_gpu_add(p.peer_ret_flag[threadIdx.x], static_cast<uint32_t>(src_cnt[threadIdx.x]));
        } else {
          __threadfence_system();
          red_release_sys_add(p.peer_ret_flag[threadIdx.x], static_cast<uint32_t>(src_cnt[threadIdx.x]));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int TN, int EPI>
cudaError_t launch_one(const CUtensorMap& tw, const CUtensorMap& tx, const MoeKernelParams& kp, dim3 grid,
                       cudaStream_t stream) {
  using Cfg = MoeCfg<TN>;
  auto kern = moe_gemm_kernel<TN, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  kern<<<grid, 128, Cfg::kSmemBytes, stream>>>(tw, tx, kp);
  return cudaGetLastError();
}

template <int EPI>
cudaError_t launch_tn(int tn, const CUtensorMap& tw, const CUtensorMap& tx, const MoeKernelParams& kp, dim3 grid,
                      cudaStream_t stream) {
  switch (tn) {
    case 16: return launch_one<16, EPI>(tw, tx, kp, grid, stream);
    case 32: return launch_one<32, EPI>(tw, tx, kp, grid, stream);
    case 64: return launch_one<64, EPI>(tw, tx, kp, grid, stream);
    case 128: return launch_one<128, EPI>(tw, tx, kp, grid, stream);
    default: return launch_one<256, EPI>(tw, tx, kp, grid, stream);
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
  if (!make_tmap_2d(&m, TmapDtype::BF16, base, rows, cols, ld, box, kBlockK, true)) return false;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

}  // namespace

int moe_tile_tokens(double rows_per_expert) {
  if (rows_per_expert <= 16) return 16;
  if (rows_per_expert <= 32) return 32;
  if (rows_per_expert <= 64) return 64;
  if (rows_per_expert <= 160) return 128;
  return 256;
}

const char* moe_gemm(const MoeGemmArgs& a) {
  if (a.n_local_experts <= 0 || a.rows_per_expert <= 0 || a.K <= 0 || a.cap <= 0) return "moe_gemm: empty problem";
  if ((a.K % 8) || (a.ldw % 8) || (a.ldx % 8)) return "moe_gemm: K and leading dims must be multiples of 8";
  if ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.x)) & 15) return "moe_gemm: operands must be 16-byte aligned";
  const int tn = a.tile_tokens;
  if (tn != 16 && tn != 32 && tn != 64 && tn != 128 && tn != 256) return "moe_gemm: bad token tile";
  if (a.max_tiles < 1 || a.max_tiles > 65535) return "moe_gemm: tile bound out of range";
  if (a.tile_expert == nullptr || a.tile_row0 == nullptr || a.tile_rows == nullptr || a.state == nullptr)
    return "moe_gemm: missing tile table";
  MoeKernelParams kp = {};
  kp.num_kb = static_cast<int>((a.K + kBlockK - 1) / kBlockK);
  kp.rows_per_expert = static_cast<int>(a.rows_per_expert);
  kp.tile_expert = a.tile_expert; kp.tile_row0 = a.tile_row0; kp.tile_rows = a.tile_rows; kp.state = a.state;
  kp.status = a.status;
  dim3 grid;
  grid.y = a.max_tiles;
  if (a.epi == kMoeEpiSwiglu) {
    if (a.rows_per_expert % 128) return "moe_gemm: SwiGLU needs expert rows in multiples of 128 (64 gate + 64 up per tile)";
    if (a.out == nullptr || (a.ldo & 1)) return "moe_gemm: no output";
    kp.out = static_cast<__nv_bfloat16*>(a.out); kp.ldo = a.ldo;
    grid.x = static_cast<unsigned>(a.rows_per_expert / 2 / 64);
  } else if (a.epi == kMoeEpiReturn) {
    if (a.rows_per_expert % 128) return "moe_gemm: expert rows must be a multiple of 128";
    if (a.world < 1 || a.world > kMoeMaxRanks || a.recv_meta == nullptr) return "moe_gemm: bad return set-up";
    kp.world = a.world; kp.recv_meta = a.recv_meta;
    for (int r = 0; r < a.world; ++r) {
      if (a.peer_ret[r] == nullptr || a.peer_ret_flag[r] == nullptr) return "moe_gemm: missing peer pointer";
      kp.peer_ret[r] = a.peer_ret[r]; kp.peer_ret_flag[r] = a.peer_ret_flag[r];
    }
    grid.x = static_cast<unsigned>(a.rows_per_expert / 128);
  } else {
    return "moe_gemm: unknown epilogue";
  }
  CUtensorMap tw, tx;
  if (!cached_tmap(&tw, a.w, static_cast<uint64_t>(a.n_local_experts) * a.rows_per_expert, a.K, a.ldw, 64))
    return "moe_gemm: weight tensor map rejected";
  if (!cached_tmap(&tx, a.x, a.cap, a.K, a.ldx, tn)) return "moe_gemm: activation tensor map rejected";
  cudaError_t e = a.epi == kMoeEpiSwiglu ? launch_tn<kMoeEpiSwiglu>(tn, tw, tx, kp, grid, a.stream)
                                         : launch_tn<kMoeEpiReturn>(tn, tw, tx, kp, grid, a.stream);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
