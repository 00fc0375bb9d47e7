// Token selection kernels: greedy arg-max (lowest id wins ties) and the full
// sampler (presence / frequency penalties, temperature, top-k <= 32, min-p,
// top-p, renormalise, draw) with a counter-based Philox generator keyed by
// (seed, logical position, purpose) so that a draw is a pure function of its
// key and can be replayed by verify / rollback.  One CTA per logits row.
//
// Reference contract: include/ninfer/ops/sampling.h:25-84 (top-k <= 20 there),
// launcher/sampling.cu, kernel argmax.
#include "sampling.h"

#include <math_constants.h>

#include "../common/ptx.cuh"

namespace nfb {

namespace {

constexpr int kThreads = 1024;

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ Best warp_best(Best x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  return x;
}
__device__ __forceinline__ Best block_best(Best x, Best* red) {
  x = warp_best(x);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = x;
  __syncthreads();
  Best y = lane < (blockDim.x >> 5) ? red[lane] : Best{-CUDART_INF_F, 0x7fffffff};
  y = warp_best(y);
  return y;  // identical in every warp
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                                                          int V, int* __restrict__ out) {
  __shared__ Best red[32];
  pdl_launch_next();
  pdl_wait_prior();
  const __nv_bfloat16* row = logits + blockIdx.x * ld;
  Best b{-CUDART_INF_F, 0x7fffffff};
  const int nvec = V / 8;
  for (int c = threadIdx.x; c < nvec; c += kThreads) {
    const uint4 r = *reinterpret_cast<const uint4*>(row + c * 8);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = __bfloat162float(e[j]);
      if (f > b.v) { b.v = f; b.i = c * 8 + j; }  // ascending index: strict > keeps the lowest id
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kThreads) {
    const float f = __bfloat162float(row[i]);
    if (f > b.v || (f == b.v && i < b.i)) { b.v = f; b.i = i; }
  }
  b = block_best(b, red);
  if (threadIdx.x == 0) out[blockIdx.x] = b.i;
}

// Philox4x32-10
__device__ __forceinline__ uint4 philox(uint4 ctr, uint2 key) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const SampleParams p) {
  __shared__ Best red[32];
  __shared__ float top_v[kMaxTopK];
  __shared__ int top_i[kMaxTopK];
  pdl_launch_next();
  pdl_wait_prior();
  const int row_id = blockIdx.x;
  const __nv_bfloat16* row = p.logits + row_id * p.ld;
  const float temp = p.temperature ? p.temperature[row_id] : 1.f;
  const int top_k_req = p.top_k ? p.top_k[row_id] : kMaxTopK;
  const float top_p = p.top_p ? p.top_p[row_id] : 1.f;
  const float min_p = p.min_p ? p.min_p[row_id] : 0.f;
  const float pres = p.presence ? p.presence[row_id] : 0.f;
  const float freq = p.frequency ? p.frequency[row_id] : 0.f;
  const int* counts = p.token_counts ? p.token_counts + static_cast<long long>(row_id) * p.V : nullptr;
  const bool greedy = temp <= 0.f || top_k_req == 1;
  const int K = greedy ? 1 : (top_k_req <= 0 || top_k_req > kMaxTopK ? kMaxTopK : top_k_req);

  // K rounds of "best value strictly after the previous pick in (value desc, id asc) order".
  Best prev{CUDART_INF_F, -1};
  for (int k = 0; k < K; ++k) {
    Best b{-CUDART_INF_F, 0x7fffffff};
    for (int i = threadIdx.x; i < p.V; i += kThreads) {
      float f = __bfloat162float(row[i]);
      if (counts != nullptr) {
        const int c = counts[i];
        if (c > 0) f -= pres + freq * static_cast<float>(c);
      }
      const bool after = f < prev.v || (f == prev.v && i > prev.i);
      if (after && (f > b.v || (f == b.v && i < b.i))) { b.v = f; b.i = i; }
    }
    b = block_best(b, red);
    if (threadIdx.x == 0) { top_v[k] = b.v; top_i[k] = b.i; }
    prev = b;
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int draft = p.draft_ids != nullptr ? p.draft_ids[row_id] : -1;
  if (greedy) {
    p.out[row_id] = top_i[0];
    if (p.accepted != nullptr) p.accepted[row_id] = (draft >= 0 && draft == top_i[0]) ? 1 : 0;
    return;
  }

  // softmax over the K candidates at the given temperature, then min-p / top-p cuts
  const float inv_t = 1.f / temp;
  float prob[kMaxTopK];
  float sum = 0.f;
  int n = 0;
  for (int k = 0; k < K; ++k) {
    if (top_i[k] == 0x7fffffff) break;
    prob[k] = __expf((top_v[k] - top_v[0]) * inv_t);
    sum += prob[k];
    n = k + 1;
  }
  // min-p: keep p_i >= min_p * p_max (p_max is candidate 0, relative weights suffice)
  int keep = n;
  if (min_p > 0.f) {
    keep = 0;
    while (keep < n && prob[keep] >= min_p * prob[0]) ++keep;
    if (keep == 0) keep = 1;
  }
  float ksum = 0.f;
  for (int k = 0; k < keep; ++k) ksum += prob[k];
  // top-p over the renormalised kept set: smallest prefix whose mass reaches top_p
  if (top_p < 1.f) {
    float acc = 0.f;
    int m = 0;
    while (m < keep) {
      acc += prob[m] / ksum;
      ++m;
      if (acc >= top_p) break;
    }
    keep = m;
    ksum = 0.f;
    for (int k = 0; k < keep; ++k) ksum += prob[k];
  }
  const uint64_t seed = p.seeds ? p.seeds[row_id] : 0ull;
  const uint32_t pos = p.positions ? static_cast<uint32_t>(p.positions[row_id]) : 0u;
  const uint2 key = make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  auto uniform = [&](unsigned int purpose) {
    const uint4 r = philox(make_uint4(pos, purpose, 0u, 0u), key);
    return (static_cast<float>(r.x >> 8) + 0.5f) * (1.f / 16777216.f);
  };
  if (p.out_dist_ids != nullptr && p.out_dist_probs != nullptr) {
    for (int k = 0; k < p.dist_out_k; ++k) {
      p.out_dist_ids[static_cast<long long>(row_id) * p.dist_out_k + k] = k < keep ? top_i[k] : -1;
      p.out_dist_probs[static_cast<long long>(row_id) * p.dist_out_k + k] = k < keep ? prob[k] / ksum : 0.f;
    }
  }
  unsigned int purpose = p.purpose;
  if (draft >= 0) {
    int kd = -1;
    for (int k = 0; k < keep; ++k)
      if (top_i[k] == draft) kd = k;
    const float pd = kd >= 0 ? prob[kd] / ksum : 0.f;
    const bool have_q = p.draft_dist_ids != nullptr && p.draft_dist_probs != nullptr && p.dist_k > 0;
    const int* q_ids = have_q ? p.draft_dist_ids + static_cast<long long>(row_id) * p.dist_k : nullptr;
    const float* q_pr = have_q ? p.draft_dist_probs + static_cast<long long>(row_id) * p.dist_k : nullptr;
    auto q_of = [&](int token) {
      float q = 0.f;
      for (int j = 0; j < p.dist_k; ++j)
        if (q_ids[j] == token) q = q_pr[j];
      return q;
    };
    float accept_p = pd;                        // deterministic draft: q(d) = 1
    if (have_q) {
      const float qd = q_of(draft);
      accept_p = qd > 0.f ? fminf(1.f, pd / qd) : (pd > 0.f ? 1.f : 0.f);
    }
    const bool ok = kd >= 0 && ((!have_q && keep == 1) || uniform(1u) < accept_p);
    if (p.accepted != nullptr) p.accepted[row_id] = ok ? 1 : 0;
    if (ok) {
      p.out[row_id] = draft;
      if (p.out_prob != nullptr) p.out_prob[row_id] = pd;
      return;
    }
    if (have_q) {
      // residual max(p - q, 0), renormalised; if p <= q everywhere (p == q) the residual is empty and p itself is used
      float rsum = 0.f;
      float res[kMaxTopK];
      for (int k = 0; k < keep; ++k) {
        res[k] = fmaxf(prob[k] / ksum - q_of(top_i[k]), 0.f);
        rsum += res[k];
      }
      if (rsum > 1e-9f) {
        for (int k = 0; k < keep; ++k) prob[k] = res[k];
        ksum = rsum;
      }
    } else if (kd >= 0) {   // residual distribution: the draft's mass is removed, the rest renormalised
      ksum -= prob[kd];
      prob[kd] = 0.f;
    }
    purpose = 2u;
  } else if (p.accepted != nullptr) {
    p.accepted[row_id] = 0;
  }
  const float u = uniform(purpose);
  float acc = 0.f;
  int pick = -1;
  for (int k = 0; k < keep; ++k) {
    if (prob[k] <= 0.f) continue;
    pick = k;                      // the last candidate with mass absorbs the rounding tail
    acc += prob[k] / ksum;
    if (u < acc) break;
  }
  if (pick < 0) pick = 0;
  p.out[row_id] = top_i[pick];
  if (p.out_prob != nullptr) p.out_prob[row_id] = prob[pick] / ksum;
}

// Greedy chain acceptance: row b has W = K+1 verify columns; draft[b][j] (j < K)
// was fed at column j+1.  Accept the longest prefix with draft[j] == target[j],
// then emit target[n_acc] as the correction / bonus token.
__global__ void accept_greedy_chain_kernel(const int* __restrict__ target_ids, const int* __restrict__ draft_ids,
                                           int B, int K, int* __restrict__ n_accepted,
                                           int* __restrict__ out_tokens) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int* tg = target_ids + b * (K + 1);
  const int* dr = draft_ids + b * K;
  int n = 0;
  while (n < K && dr[n] == tg[n]) ++n;
  n_accepted[b] = n;
  for (int j = 0; j <= K; ++j) out_tokens[b * (K + 1) + j] = j < n ? dr[j] : (j == n ? tg[n] : -1);
}

// Greedy tree acceptance: node i (1..N-1) has parent[i] < i and token tok[i]; node 0 is the
// root (last committed token).  target[i] = arg-max of the target at node i's column.
// Node i is accepted iff its parent is accepted and tok[i] == target[parent[i]].
// The winning path is the deepest accepted node (lowest index on ties).
__global__ void accept_greedy_tree_kernel(const int* __restrict__ target_ids, const int* __restrict__ node_tok,
                                          const int* __restrict__ parent, int B, int N, int* __restrict__ n_accepted,
                                          int* __restrict__ out_tokens, int* __restrict__ out_nodes, int max_depth) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int* tg = target_ids + b * N;
  const int* tok = node_tok + b * N;
  const int* par = parent + b * N;
  int best = 0, best_depth = 0;
  // depth and acceptance via one forward sweep (parents precede children)
  int depth[64];
  bool acc[64];
  depth[0] = 0; acc[0] = true;
  for (int i = 1; i < N && i < 64; ++i) {
    const int pi = par[i];
    acc[i] = pi >= 0 && pi < i && acc[pi] && tok[i] == tg[pi];
    depth[i] = (pi >= 0 && pi < i) ? depth[pi] + 1 : 0;
    if (acc[i] && depth[i] > best_depth) { best = i; best_depth = depth[i]; }
  }
  n_accepted[b] = best_depth;
  int* ot = out_tokens + b * (max_depth + 1);
  int* on = out_nodes + b * (max_depth + 1);
  for (int j = 0; j <= max_depth; ++j) { ot[j] = -1; on[j] = -1; }
  int node = best;
  for (int d = best_depth; d >= 1; --d) { ot[d - 1] = tok[node]; on[d - 1] = node; node = par[node]; }
  ot[best_depth] = tg[best];  // correction / bonus token sampled at the deepest accepted node
  on[best_depth] = best;
}

}  // namespace

const char* argmax_rows(const void* logits, long long ld, int T, int V, int* out, cudaStream_t stream, bool pdl) {
  if (T <= 0) return nullptr;
  if (ld % 8) return "argmax_rows: leading dimension must be a multiple of 8";
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(T); cfg.blockDim = dim3(kThreads); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_kernel, static_cast<const __nv_bfloat16*>(logits), ld, V, out);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* sample_rows(const SampleParams& p, cudaStream_t stream) {
  if (p.T <= 0) return nullptr;
  sample_kernel<<<p.T, kThreads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* accept_greedy_chain(const int* target_ids, const int* draft_ids, int B, int K, int* n_accepted,
                                int* out_tokens, cudaStream_t stream) {
  if (B <= 0) return nullptr;
  accept_greedy_chain_kernel<<<(B + 63) / 64, 64, 0, stream>>>(target_ids, draft_ids, B, K, n_accepted, out_tokens);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* accept_greedy_tree(const int* target_ids, const int* node_tok, const int* parent, int B, int N,
                               int max_depth, int* n_accepted, int* out_tokens, int* out_nodes,
                               cudaStream_t stream) {
  if (B <= 0) return nullptr;
  if (N > 64) return "accept_greedy_tree: at most 64 tree nodes";
  accept_greedy_tree_kernel<<<(B + 31) / 32, 32, 0, stream>>>(target_ids, node_tok, parent, B, N, n_accepted,
                                                              out_tokens, out_nodes, max_depth);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
