// Relocation of KV rows inside one sequence's pages: after a tree verification the accepted nodes' K/V (written
// at frontier + node index) move to their final positions frontier + depth.  One CTA per (sequence, kv head)
// performs the moves of that sequence in order, with a barrier between two moves, because the destination of a
// later move may be the source of an earlier one.
//
// Reference: mtp_tree_commit_history (include/ninfer/ops/mtp_round.h): "relocates accepted tree K/V to
// frontier+1..frontier+A".
#include "kv_layout.h"

#include <cuda_runtime.h>

namespace nfb {

namespace {

__global__ void __launch_bounds__(128) kv_move_rows_kernel(KvLayer L, const int* __restrict__ table, int table_cols,
                                                           const int* __restrict__ table_row, const int* __restrict__ src_pos,
                                                           const int* __restrict__ dst_pos, int max_moves) {
  const int b = blockIdx.x, h = blockIdx.y;
  const int rb = kv_row_bytes(L.format, L.head_dim);
  const int sb = kv_scale_bytes(L.format, L.head_dim, L.group);
  const int* pages = table + static_cast<long long>(table_row[b]) * table_cols;
  for (int m = 0; m < max_moves; ++m) {
    const int s = src_pos[b * max_moves + m], d = dst_pos[b * max_moves + m];
    if (s >= 0 && d >= 0 && s != d) {
      const long long so = ((static_cast<long long>(pages[s / L.page_size]) * L.n_kv_heads + h) * L.page_size + s % L.page_size);
      const long long dof = ((static_cast<long long>(pages[d / L.page_size]) * L.n_kv_heads + h) * L.page_size + d % L.page_size);
      for (int i = threadIdx.x; i < rb / 4; i += blockDim.x) {
        reinterpret_cast<uint32_t*>(L.k_codes + dof * rb)[i] = reinterpret_cast<const uint32_t*>(L.k_codes + so * rb)[i];
        reinterpret_cast<uint32_t*>(L.v_codes + dof * rb)[i] = reinterpret_cast<const uint32_t*>(L.v_codes + so * rb)[i];
      }
      if (sb > 0) {
        for (int i = threadIdx.x; i < sb; i += blockDim.x) {
          L.k_scales[dof * sb + i] = L.k_scales[so * sb + i];
          L.v_scales[dof * sb + i] = L.v_scales[so * sb + i];
        }
      }
    }
    __syncthreads();
  }
}

}  // namespace

const char* kv_move_rows(const KvLayer& L, const int* table, int table_cols, const int* table_row, const int* src_pos,
                         const int* dst_pos, int n_seq, int max_moves, cudaStream_t stream) {
  if (n_seq <= 0 || max_moves <= 0) return nullptr;
  kv_move_rows_kernel<<<dim3(n_seq, L.n_kv_heads), 128, 0, stream>>>(L, table, table_cols, table_row, src_pos, dst_pos,
                                                                       max_moves);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
