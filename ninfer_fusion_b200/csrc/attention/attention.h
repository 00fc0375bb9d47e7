// Host entry points of the attention family (plain C++ ABI).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../kv/kv_layout.h"

namespace nfb {

struct AttnPrepParams {
  const __nv_bfloat16* proj;  // [T, ld_proj] fused projection output
  long long ld_proj;
  int q_off, k_off, v_off;    // column offsets of the Q / K / V blocks inside a row
  int T, n_q_heads, n_kv_heads, head_dim;
  const __nv_bfloat16* q_norm_w;  // [head_dim] or nullptr
  const __nv_bfloat16* k_norm_w;
  float eps;
  int unit_offset;
  int rot_dim;                // rotary dims (first rot_dim of each head), 0 = no RoPE
  const float* inv_freq;      // [rot_dim / 2] device
  float rope_attn_factor;     // YaRN attention factor folded into sin/cos (1 when unused)
  const int* rope_pos;        // [T, pos_axes]
  int pos_axes;               // 1 (text) or 3 (MRoPE t/h/w)
  const int* token_seq;       // [T] row of the block table (-1 = padding)
  const int* cache_pos;       // [T] position inside the sequence's KV cache
  const int* block_table;     // [n_seq, table_stride] page ids (-1 = unmapped)
  int table_stride;
  __nv_bfloat16* q_out;       // [T, n_q_heads, head_dim]
  KvLayer kv;
  // K frame: 1 = q and k are rotated by the normalised Hadamard matrix of the head dimension before q is written
  // and k is quantised (q . k is unchanged; outlier channels of k are spread over the row, which is what a per-row
  // fp8 scale needs).  V is stored from its source values.
  int k_hadamard = 0;
  // Per-channel row scale of the stored K frame, [n_kv_heads, head_dim] bf16 for this layer or nullptr: k is
  // multiplied by s_d before it is quantised and q (of the heads that read that kv head) by 1 / s_d, so q . k is
  // unchanged while the channel magnitudes of k are balanced for the group / row scales of the codec
  // (the reference's Sinkhorn row scale, s_d in [0.5, 2]: src/ops/kernel/gqa_isoquant_row_scale.cuh).
  const __nv_bfloat16* k_row_scale = nullptr;
};
const char* attn_prep(const AttnPrepParams& p, cudaStream_t stream, bool pdl);

struct PagedAttnParams {
  const __nv_bfloat16* q;     // [Tq, n_q_heads, head_dim]
  int Tq, n_q_heads, n_kv_heads, head_dim;
  const int* q_seq;           // [Tq] block-table row of each query token
  const int* q_kv_len;        // [Tq] number of visible keys (cache_pos + 1)
  const int* block_table;
  int table_stride;
  KvLayer kv;
  float sm_scale;
  int split_keys;             // keys per split (multiple of 128); splits cover absolute ranges
  int n_splits;               // grid.z = ceil(max_kv_len / split_keys)
  float* part_o;              // [Tq, n_q_heads, n_splits, head_dim] fp32 un-normalised
  float* part_ml;             // [Tq, n_q_heads, n_splits, 2] (max, sum)
  // merge epilogue
  const __nv_bfloat16* gate;  // optional [Tq, ld_gate] sigmoid gate, column h*head_dim + d
  long long ld_gate;
  __nv_bfloat16* out;         // [Tq, n_q_heads * head_dim]
  // optional tree-verify mask: bit j of tree_mask[t] set = query t may see the key at
  // position (tree_base[t] + j); keys below tree_base[t] are always visible.
  const unsigned long long* tree_mask;
  const int* tree_base;
  int impl;  // 0 = pick, 1 = SIMT kernel, 2 = mma.sync tensor-core kernel, 3 = tcgen05 kernel (fp8-row pages)
  long long kv_plane_rows = 0;  // rows (page x head x token) of the K / V code planes; 0 = unknown (no TMA path)
  int* status = nullptr;        // optional device status word for the bounded waits of the tcgen05 kernel
  // optional: the merged output also as the next GEMM's nvfp4 operand (gemm/nvfp4_act.cuh): codes [Tq][Hq * D / 2]
  // bytes and the scale plane of Tq x (Hq * D) values
  uint8_t* q_codes = nullptr;
  uint8_t* q_sf = nullptr;
  int window = 0;  // sliding window: a query sees only its last `window` keys (0 = all of them)
  // Selected-block attention (optional, decode only): query t attends to sel_count[t] blocks of four consecutive
  // tokens, block ids in sel_blocks[t * sel_stride ..] (each below the number of complete blocks, kv_len / 4), plus
  // the tokens of the last incomplete block [4 * (kv_len / 4), kv_len).  The splits then cover ordinals of that
  // gathered key list instead of absolute positions.  Not combined with a window or a tree mask.
  // (Reference: include/ninfer/ops/selected_block_attention.h, query-selected sparse attention of the FlashNext target.)
  const int* sel_blocks = nullptr;
  const int* sel_count = nullptr;
  int sel_stride = 0;
};
// Split-KV paged attention over quantised pages with in-register dequantisation,
// followed by the (m, l, o) merge fused with the output sigmoid gate.
const char* paged_attention(const PagedAttnParams& p, cudaStream_t stream, bool pdl);
// Tensor-core split kernels; cudaErrorNotSupported when the problem is outside a kernel's envelope.
cudaError_t paged_attention_mma_split(const PagedAttnParams& p, cudaStream_t stream, bool pdl);
cudaError_t paged_attention_tc_split(const PagedAttnParams& p, cudaStream_t stream, bool pdl);   // tcgen05, fp8-row pages
void paged_attention_tc_trace(bool enable, unsigned long long* host_out);   // event trace of CTA 0: [5][1024] words

// Causal prefill / wide-verify attention over blocks of consecutive query tokens of one sequence.
struct PrefillAttnParams {
  const __nv_bfloat16* q;     // [T, n_q_heads, head_dim]
  int n_q_heads, n_kv_heads, head_dim;
  const int* q_seq;           // [T] block-table row per token
  const int* q_kv_len;        // [T] visible keys per token (cache_pos + 1), increasing inside a block
  const int* blk_start;       // [n_blocks] first token of each query block
  const int* blk_count;       // [n_blocks] tokens in the block (<= prefill_attn_block_tokens)
  int n_blocks;
  const int* block_table;
  int table_stride;
  KvLayer kv;
  float sm_scale;
  const __nv_bfloat16* gate;  // optional sigmoid gate [T, ld_gate]
  long long ld_gate;
  __nv_bfloat16* out;         // [T, n_q_heads * head_dim]
  int window = 0;             // sliding window (0 = full causal attention)
};
const char* paged_attention_prefill(const PrefillAttnParams& p, cudaStream_t stream, bool pdl);
// Query tokens per block for a GQA geometry (128 MMA rows / group size).
int prefill_attn_block_tokens(int n_q_heads, int n_kv_heads);

// Moves K/V rows of each sequence from cache positions src_pos[b, m] to dst_pos[b, m], in order m = 0.. (a negative
// entry skips the move): accepted tree nodes go from frontier + node index to frontier + depth (kv/kv_move.cu).
// Re-encodes cells of a mixed-precision layer into another tier (see kv/kv_requant.cu).  `src_cell` / `dst_cell`:
// device arrays of n_cells entries, each tier << 28 | slot; the caller updates the layer's cell map afterwards.
struct KvRequantParams {
  KvLayer kv;             // format kKvMixed with all three tiers' planes
  const int* src_cell;
  const int* dst_cell;
  int n_cells;
};
const char* kv_requant(const KvRequantParams& p, cudaStream_t stream);

const char* kv_move_rows(const KvLayer& L, const int* table, int table_cols, const int* table_row, const int* src_pos,
                         const int* dst_pos, int n_seq, int max_moves, cudaStream_t stream);

}  // namespace nfb
