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
  // bit 0: phase A (reduce my slice, push it to every rank), bit 1: phase B (wait for all slices, normalise).
  // 3 = both in one launch (production); the halves are launched separately only to walk several ranks through on
  // one GPU, where a kernel must never wait for a later launch
  int phases = 3;
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
  int phases = 3;                    // bit 0: scan + push the candidate, bit 1: wait for all candidates + pick
};
const char* tp_argmax(const TpArgmaxParams& p, cudaStream_t stream, bool pdl);

// Materialises the RMS-normalised residual stream after a GEMM whose epilogue reduce-scattered and all-gathered
// it (gemm kEpiRsAg): waits (bounded) until `*flag - *target >= 0`, i.e. every residual tile of every owner has
// landed in this rank's buffer, then writes normed[t] = x[t] * rsqrt(mean(x[t]^2) + eps) * (unit_offset + w).
// Used where the consumer is not a column-parallel GEMM that can wait and scale by itself (the final norm before
// the vocabulary head, a draft module, a router).
struct TpGatherNormParams {
  int T, N;
  const unsigned int* flag;      // this rank's residual arrival counter
  const unsigned int* target;    // cumulative arrivals to wait for (device word written by the producing GEMM)
  const __nv_bfloat16* x;        // [T, ldx]
  long long ldx;
  const __nv_bfloat16* norm_w;   // [N]
  __nv_bfloat16* normed;         // [T, N] contiguous
  float eps;
  int unit_offset;
  int* status;
};
const char* tp_gather_norm(const TpGatherNormParams& p, cudaStream_t stream, bool pdl);

// ---- symmetric buffers over CUDA IPC (one process per GPU, one node) ----
// Allocates `bytes` with cudaMalloc (zero-filled) and exports a 64-byte IPC handle.
const char* symm_alloc(size_t bytes, void** ptr, unsigned char handle_out[64]);
// Maps a peer's allocation into this process (peer access is enabled lazily by the driver).
const char* symm_open(const unsigned char handle[64], void** ptr);
const char* symm_close(void* ptr);
const char* symm_free(void* ptr);

}  // namespace nfb
