// Host entry points of the sparse mixture-of-experts family (plain C++ ABI).
//
// One code path serves a single GPU (world = 1) and expert parallelism over
// NVLink (world = 2..8, experts split in contiguous ranges of E / world):
//
//   moe_route    softmax -> top-k (ties: lower id) -> renormalise, per-expert histogram
//   moe_plan     all ranks exchange their histograms by push, then every rank knows where each
//                (source, expert) group starts in every destination's receive buffer and builds
//                the tile table of its own grouped GEMMs
//   moe_push     dispatch: token rows are stored straight into their final, expert-sorted slot of
//                the destination rank's receive buffer (all-to-all by peer stores)
//   moe_gemm     grouped tcgen05 GEMM over the expert-sorted rows; epilogue SwiGLU, or
//                "return": the down projection's bf16 rows are stored straight into the SOURCE
//                rank's return buffer (the combine all-to-all fused into the GEMM)
//   moe_combine  waits for the returned rows, weighted sum in fixed order + shared expert +
//                residual add + next RMSNorm
//
// Counters only grow, every wait is bounded and reports through the status word.
//
// Reference: include/ninfer/ops/sparse_moe.h:13-63 and src/ops/sparse_moe/{decode,small_t,prefill}
// (a closed single-GPU op; it has no expert parallelism).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfb {

constexpr int kMoeMaxRanks = 8;
constexpr int kMoePushCtas = 128;   // fixed dispatch grid, so every source signals a destination 128 times per call
constexpr int kMoeMaxExperts = 512;
constexpr int kMoeMaxTopK = 16;

// Rank-local bookkeeping (ordinary device memory, zero-initialised).
struct MoeState {
  unsigned int call_idx;      // finished moe_plan calls
  unsigned int ret_expected;  // cumulative returned-row arrivals consumed by finished combines
  unsigned int ctas_done;
  int n_tiles;                // token tiles of this call's grouped GEMMs
  int total_rows;             // rows this rank received in this call
  int overflow;               // 1 if some rank's receive buffer was too small in this call
};

struct MoeRouteParams {
  int T, E, k, norm_topk;
  const __nv_bfloat16* logits;  // [T, ld]; column E (if has_shared_gate) is the shared expert's gate logit
  long long ld;
  int has_shared_gate;
  int* hist;        // [E], zero on entry (moe_plan clears it again)
  int* ids;         // [T, k]
  float* weights;   // [T, k]
  int* pos;         // [T, k] rank of the assignment among this rank's assignments of the same expert
  float* shared_gate;  // [T] sigmoid of the shared gate logit
};
const char* moe_route(const MoeRouteParams& p, cudaStream_t stream);

struct MoePlanParams {
  int world, rank, E, tile_tokens, cap, max_tiles;
  int* hist;                              // [E] local histogram (cleared at the end)
  int* my_counts;                         // [world, E] (symmetric)
  int* peer_counts[kMoeMaxRanks];
  unsigned int* my_count_flag;
  unsigned int* peer_count_flag[kMoeMaxRanks];
  int* send_base;                         // [E] first slot of this rank's group in the destination's buffer
  int* tile_expert;                       // [max_tiles] local expert of each token tile
  int* tile_row0;                         // [max_tiles] first receive-buffer row
  int* tile_rows;                         // [max_tiles] valid rows
  MoeState* state;
  int* status;
};
const char* moe_plan(const MoePlanParams& p, cudaStream_t stream);

struct MoePushParams {
  int world, rank, T, k, H, E, cap;
  const __nv_bfloat16* x;   // [T, ldx] normalised hidden rows
  long long ldx;
  const int* ids;
  const int* pos;
  const int* send_base;
  __nv_bfloat16* peer_recv_x[kMoeMaxRanks];  // [cap, H]
  int* peer_recv_meta[kMoeMaxRanks];         // [cap]: source rank << 24 | (token * k + j)
  unsigned int* peer_arrive_flag[kMoeMaxRanks];
  const unsigned int* my_arrive_flag;
  const MoeState* state;
  int* status;
};
const char* moe_push(const MoePushParams& p, cudaStream_t stream);

enum MoeGemmEpilogue : int {
  kMoeEpiSwiglu = 0,  // W_e = [gate; up], out[row, n] = silu(gate) * up
  kMoeEpiReturn = 1,  // out row goes to the source rank's return buffer [token * k + j, N]
};

struct MoeGemmArgs {
  const void* w = nullptr;  // [n_local_experts * rows_per_expert, K] bf16, leading dimension ldw
  int64_t rows_per_expert = 0, K = 0, ldw = 0;
  int n_local_experts = 0;
  const void* x = nullptr;  // [cap, K] expert-sorted rows
  int64_t cap = 0, ldx = 0;
  int tile_tokens = 16, max_tiles = 0;
  const int* tile_expert = nullptr;
  const int* tile_row0 = nullptr;
  const int* tile_rows = nullptr;
  const MoeState* state = nullptr;
  int epi = kMoeEpiSwiglu;
  void* out = nullptr;      // kMoeEpiSwiglu: [cap, rows_per_expert / 2] bf16
  int64_t ldo = 0;
  // kMoeEpiReturn
  int world = 1;
  const int* recv_meta = nullptr;
  __nv_bfloat16* peer_ret[kMoeMaxRanks] = {};   // [T_cap * k, rows_per_expert]
  unsigned int* peer_ret_flag[kMoeMaxRanks] = {};
  int* status = nullptr;
  cudaStream_t stream = nullptr;
  // fp8 block-scaled experts (moe_gemm_fp8): w / x are e4m3 codes, scales are fp32
  const float* w_scale = nullptr;   // [experts, rows_per_expert / 128, K / 128]
  const float* x_scale = nullptr;   // [cap, K / 128]
};
const char* moe_gemm(const MoeGemmArgs& a);
// Same tile walk over e4m3 weights with 128 x 128 block scales and activations quantised per row and 128-wide k-block.
const char* moe_gemm_fp8(const MoeGemmArgs& a);
// Quantises the first min(max_rows, state->total_rows) rows of x [max_rows, K] (state may be null: all rows).
const char* moe_quant_rows_block128(const __nv_bfloat16* x, long long ldx, int max_rows, int K, const MoeState* state,
                                    uint8_t* codes, float* scales, cudaStream_t stream);
// Token-tile width for an expected number of rows per expert.
int moe_tile_tokens(double rows_per_expert);

struct MoeCombineParams {
  int T, k, H;
  unsigned int arrivals_this_call;  // T * k * (H / 128): one unit per returned row per 128-column tile
  __nv_bfloat16* x;                 // [T, H] residual stream, updated in place
  const float* weights;             // [T, k]
  const __nv_bfloat16* ret;         // [T * k, H] returned expert rows (symmetric)
  const unsigned int* ret_flag;
  const __nv_bfloat16* shared;      // [T, H] shared-expert output, may be null
  const float* shared_gate;         // [T]
  const __nv_bfloat16* norm_w;      // [H] next RMSNorm (unit offset), may be null
  __nv_bfloat16* normed;            // [T, H]
  float eps;
  MoeState* state;
  int* status;
};
const char* moe_combine(const MoeCombineParams& p, cudaStream_t stream);

}  // namespace nfb
