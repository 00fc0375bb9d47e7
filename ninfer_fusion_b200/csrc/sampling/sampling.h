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
  // Stochastic drafts (optional, with draft_ids): the drafter's own processed distribution q of each row as
  // dist_k (id, probability) pairs, probabilities summing to 1 over the ids with id >= 0.  The draft is then accepted
  // with probability min(1, p(d) / q(d)) and a rejection resamples from max(p - q, 0) renormalised -- speculative
  // sampling in its general form; without q the draft counts as deterministic (q = 1 at the draft).
  const int* draft_dist_ids = nullptr;     // [T, dist_k]
  const float* draft_dist_probs = nullptr; // [T, dist_k]
  int dist_k = 0;
  // Optional outputs: the row's final distribution (kept candidates, renormalised) as dist_out_k (id, prob) pairs,
  // padded with id = -1: what a drafter hands to the verifier as its q.
  int* out_dist_ids = nullptr;             // [T, dist_out_k]
  float* out_dist_probs = nullptr;         // [T, dist_out_k]
  int dist_out_k = 0;
};
const char* sample_rows(const SampleParams& p, cudaStream_t stream);

const char* accept_greedy_chain(const int* target_ids, const int* draft_ids, int B, int K, int* n_accepted,
                                int* out_tokens, cudaStream_t stream);
const char* accept_greedy_tree(const int* target_ids, const int* node_tok, const int* parent, int B, int N,
                               int max_depth, int* n_accepted, int* out_tokens, int* out_nodes,
                               cudaStream_t stream);

}  // namespace nfb
