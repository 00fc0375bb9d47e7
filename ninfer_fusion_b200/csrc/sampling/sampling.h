// Host entry points of the token-selection kernels (plain C++ ABI).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfb {

constexpr int kMaxTopK = 32;

const char* argmax_rows(const void* logits, long long ld, int T, int V, int* out, cudaStream_t stream, bool pdl);

struct SampleParams {
  const __nv_bfloat16* logits;  // [T, ld]
  long long ld;
  int T, V;
  const float* temperature;     // per row; <= 0 means greedy.  Null = 1
  const int* top_k;             // per row; <= 0 or > 32 means 32.  Null = 32
  const float* top_p;           // null = 1
  const float* min_p;           // null = 0
  const float* presence;        // null = 0
  const float* frequency;       // null = 0
  const int* token_counts;      // [T, V] occurrences so far, or null
  const unsigned long long* seeds;  // per row
  const int* positions;         // logical position of the token being drawn, per row
  unsigned int purpose;         // stream id: 0 = sample, 1 = spec accept, 2 = residual resample, ...
  int* out;                     // [T]
  float* out_prob;              // optional: probability of the drawn token under the final distribution
  // Speculative verification of deterministic drafts (optional): row r checks draft_ids[r] (< 0: no draft, plain
  // sampling).  The draft is accepted with probability p(draft) under the row's final distribution (random stream
  // `purpose` = 1); on rejection the token is drawn from that distribution with the draft removed and renormalised
  // (stream 2), so the emitted token is distributed exactly as p.  Greedy rows accept iff the draft is the arg-max.
  const int* draft_ids = nullptr;
  int* accepted = nullptr;      // [T] 1 = draft accepted (out = draft), 0 = rejected (out = replacement)
};
const char* sample_rows(const SampleParams& p, cudaStream_t stream);

const char* accept_greedy_chain(const int* target_ids, const int* draft_ids, int B, int K, int* n_accepted,
                                int* out_tokens, cudaStream_t stream);
const char* accept_greedy_tree(const int* target_ids, const int* node_tok, const int* parent, int B, int N,
                               int max_depth, int* n_accepted, int* out_tokens, int* out_nodes,
                               cudaStream_t stream);

}  // namespace nfb
