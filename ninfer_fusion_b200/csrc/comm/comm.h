// Host entry points of the tensor-/expert-parallel peer-memory kernels and of the
// symmetric-buffer plumbing (plain C++ ABI).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfb {

constexpr int kMaxTpRanks = 8;
constexpr int kTpMaxRows = 4096;

// Rank-local bookkeeping of the counter protocol (ordinary device memory, zero-initialised).
struct TpState {
  unsigned int expected_arrivals;  // cumulative arrivals consumed by finished reduce calls
  unsigned int ctas_done;
  unsigned int row_calls[kTpMaxRows];     // finished reduce calls per token row
  unsigned int argmax_calls[kTpMaxRows];  // finished arg-max exchanges per token row
  unsigned int call_idx;                  // finished one-shot (push-all) reductions; parity = receive buffer
  unsigned int expected_all;              // cumulative push-all arrivals consumed so far
  unsigned int ctas_done_all;
};

// Decode-sized all-reduce finish: the GEMMs of all ranks pushed fp32 tiles into this rank's buffer
// [parity][src_rank][T_cap][N] (gemm kEpiPushAll); sum the `world` sources in rank order, add the residual,
// round to bf16 and RMS-normalise.  Every rank computes the identical full row, so nothing is gathered.
struct TpSumNormParams {
  int world, T, T_cap, N;
  unsigned int arrivals_this_call;   // world * (column tiles) * (token tiles)
  const float* my_recv;
  const unsigned int* my_flag;
  __nv_bfloat16* x;                  // [T, N] residual stream, updated in place (local memory)
  const __nv_bfloat16* norm_w;
  __nv_bfloat16* normed;             // [T, N], may be null
  float eps;
  int unit_offset;
  TpState* state;
  int* status;
};
const char* tp_sum_norm(const TpSumNormParams& p, cudaStream_t stream, bool pdl);

struct TpReduceParams {
  int world, rank, T, T_cap, N, splits;
  unsigned int arrivals_this_call;   // world * (tiles in my slice) * (token tiles) * splits
  const float* my_recv;              // [world * splits, T, N / world] fp32 partials pushed by the GEMMs
  const unsigned int* my_arrival_flag;
  __nv_bfloat16* my_x;               // [T_cap, N] residual stream (symmetric)
  __nv_bfloat16* peer_x[kMaxTpRanks];
  float* my_ss;                      // [2, T_cap, world] sums of squares per slice (symmetric)
  float* peer_ss[kMaxTpRanks];
  unsigned int* my_row_flag;         // [T_cap]
  unsigned int* peer_row_flag[kMaxTpRanks];
  const __nv_bfloat16* norm_w;       // [N]
  __nv_bfloat16* normed;             // [T, N] local output, may be null
  float eps;
  int unit_offset;
  TpState* state;
  int* status;
};
const char* tp_reduce_ag_norm(const TpReduceParams& p, cudaStream_t stream, bool pdl);

struct TpArgmaxParams {
  int world, rank, T, T_cap, V_local;
  const __nv_bfloat16* logits;       // [T, ld] this rank's vocabulary slice
  long long ld;
  float2* my_cand;                   // [2, T_cap, world] (value, id bits) (symmetric)
  float2* peer_cand[kMaxTpRanks];
  unsigned int* my_flag;             // [T_cap]
  unsigned int* peer_flag[kMaxTpRanks];
  int* out;                          // [T] global token ids
  TpState* state;
  int* status;
};
const char* tp_argmax(const TpArgmaxParams& p, cudaStream_t stream, bool pdl);

// ---- symmetric buffers over CUDA IPC (one process per GPU, one node) ----
// Allocates `bytes` with cudaMalloc (zero-filled) and exports a 64-byte IPC handle.
const char* symm_alloc(size_t bytes, void** ptr, unsigned char handle_out[64]);
// Maps a peer's allocation into this process (peer access is enabled lazily by the driver).
const char* symm_open(const unsigned char handle[64], void** ptr);
const char* symm_close(void* ptr);
const char* symm_free(void* ptr);

}  // namespace nfb
