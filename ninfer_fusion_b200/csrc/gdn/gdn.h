// Host entry points of the Gated-DeltaNet family (plain C++ ABI).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace nfb {

// Depthwise causal conv (kernel 4) + SiLU over C channels of a fused projection
// row, for ragged batches.  Conv history lives per sequence slot as [slot, 3, C]
// bf16, oldest -> newest.  `update_state` also rolls the history forward.
struct ConvParams {
  const __nv_bfloat16* x;   // [T, ld_x], channels start at c_off
  long long ld_x;
  int c_off, C, T, n_seq;
  const __nv_bfloat16* w;   // [C, 4], tap 3 multiplies the newest input
  const int* cu_seqlens;    // [n_seq + 1]
  const int* token_seq;     // [T]
  const int* state_slot;    // [n_seq]
  __nv_bfloat16* conv_state;  // [slots, 3, C]
  __nv_bfloat16* out;       // [T, C]
  int update_state;
  int one_token_per_seq;     // decode: token i belongs to sequence i; conv + history roll in one launch
  const int* seq_end = nullptr;  // optional [n_seq]: sequence s covers [cu_seqlens[s], seq_end[s]) (accepted prefix of a verify)
  int state_only = 0;        // only roll the history forward (replay of an accepted prefix), no output
  // Tree verification (optional): parent[t] = token index of t's parent in the draft tree, or -1 for the first
  // token of the window (its predecessors are the sequence's history).  The taps of a token follow its ancestors
  // instead of the preceding buffer rows.  With `last_token` (per sequence) the history roll ends at that token.
  const int* parent = nullptr;
  const int* last_token = nullptr;
};
const char* causal_conv1d_silu(const ConvParams& p, cudaStream_t stream, bool pdl);

// Gated delta rule over ragged sequences, state [slot, Hv, 128, 128] fp32 (dv-major):
//   alpha = exp(-exp(A_log) * softplus(a + dt_bias)), beta = sigmoid(b)
//   S = alpha * S;  u = beta * (v - S k);  S += u (x) k;  o = S q / sqrt(128)
// with q, k L2-normalised per head, then per-head gated RMSNorm:
//   y = o * rsqrt(mean(o^2) + eps) * norm_w * silu(z)
struct GdnParams {
  const __nv_bfloat16* qkv;  // [T, ld_qkv] conv output: q heads | k heads | v heads
  long long ld_qkv;
  int q_off, k_off, v_off;
  const __nv_bfloat16* proj; // [T, ld_proj] raw projection (z, a, b columns)
  long long ld_proj;
  int z_off, a_off, b_off;
  int T, n_seq, n_qk_heads, n_v_heads;
  const float* A_log;        // [Hv]
  const float* dt_bias;      // [Hv]
  const __nv_bfloat16* norm_w;  // [128]
  float eps;
  const int* cu_seqlens;     // [n_seq + 1]
  const int* state_slot;     // [n_seq]
  float* state;              // [slots, Hv, 128, 128]
  int write_state;           // 0: verify pass, state untouched
  __nv_bfloat16* out;        // [T, Hv * 128]
  const int* seq_end = nullptr;  // optional [n_seq]: sequence s covers [cu_seqlens[s], seq_end[s])
  // Tree verification / selective replay (optional, per token): commit[t] = 0 means "side branch": the token sees
  // the current state, produces its output, and leaves the state as it was.  Tokens are visited in buffer order, so
  // a side branch must directly follow the state it hangs off.
  const unsigned char* commit = nullptr;
  // Decode with the causal convolution fused in (exactly one token per sequence, state written, no seq_end / commit):
  // `qkv` is then the RAW input projection (conv channel c at column c), conv_w is [C, 4], conv_state [slots, 3, C]
  // holds the last three inputs of every channel; q_off / k_off / v_off index conv channels.  The kernel applies the
  // four taps and SiLU, rounds to bf16 like the separate conv kernel does, and rolls the history; the CTAs of the
  // value heads that share a key head form a cluster, so that all of them have read the shared q / k history before
  // one of them rewrites it.
  const __nv_bfloat16* conv_w = nullptr;
  __nv_bfloat16* conv_state = nullptr;
  int conv_C = 0;
  // Optional (recurrent kernel only): the output rows also as the next GEMM's nvfp4 operand (see gemm/nvfp4_act.cuh):
  // codes [T][Hv * 64] bytes and the scale plane of T x (Hv * 128) values.
  uint8_t* q_codes = nullptr;
  uint8_t* q_sf = nullptr;
};
const char* gdn_recurrent(const GdnParams& p, cudaStream_t stream, bool pdl);
// Multi-token variant (token groups staged in shared memory); gdn_recurrent dispatches to it when T > n_seq.
const char* gdn_prefill(const GdnParams& p, cudaStream_t stream, bool pdl);
// Chunked (WY) tensor-core formulation for long prefill chunks: 64-token chunks, all chunks prepared in parallel,
// then one pass per (sequence, head) over the chunks.  Needs a workspace of gdn_chunked_workspace_bytes(
// gdn_chunked_max_chunks(T, n_seq), n_v_heads) bytes; seq_end / commit passes are not supported (they are short).
size_t gdn_chunked_workspace_bytes(int max_chunks, int n_v_heads);
int gdn_chunked_max_chunks(int T, int n_seq);
const char* gdn_chunked(const GdnParams& p, void* workspace, size_t workspace_bytes, cudaStream_t stream);
// Performance debugging of the row-split variant: switches the phase profile on/off and reads the last profile
// (cycles of CTA (0,0): operand wait, prologue, serial steps, partial sums + cluster barrier, epilogue).
void gdn_prefill_trace(bool enable, long long* host5);

}  // namespace nfb
