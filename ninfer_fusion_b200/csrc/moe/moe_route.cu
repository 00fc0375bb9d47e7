// Routing, dispatch and combine of the sparse mixture-of-experts block (see moe.h for the
// protocol).  All cross-rank traffic is ordinary stores into peer memory plus release/acquire
// counters; with world = 1 the same kernels run on local pointers.
//
// Routing math (include/ninfer/ops/sparse_moe.h:36-48): p = softmax(router logits) over the
// routed experts, top-k by probability with the lower id winning ties, weights renormalised to
// sum 1, shared expert scaled by sigmoid(shared gate logit).
#include "moe.h"

#include "../comm/peer_sync.cuh"
#include "../common/ptx.cuh"

namespace nfb {

namespace {

// ---------------------------------------------------------------------------------------------
// moe_route: one warp per token
// ---------------------------------------------------------------------------------------------
constexpr int kRouteWarps = 4;
constexpr int kPerLane = kMoeMaxExperts / 32;

__global__ void __launch_bounds__(kRouteWarps * 32) moe_route_kernel(const MoeRouteParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= p.T) return;
  const __nv_bfloat16* row = p.logits + static_cast<long long>(t) * p.ld;
  float v[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < p.E ? __bfloat162float(row[e]) : -INFINITY;
  }
  uint32_t taken = 0;
  float sel_v = 0.f, vmax = 0.f;
  int sel_id = 0;
  for (int r = 0; r < p.k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = lane + 32 * i;
      if (!((taken >> i) & 1u) && e < p.E && (v[i] > bv || (v[i] == bv && e < bi))) { bv = v[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (r == 0) vmax = bv;
    if (lane == r) { sel_v = bv; sel_id = bi; }
  }
  const float ex = lane < p.k ? __expf(sel_v - vmax) : 0.f;
  float denom;
  if (p.norm_topk) {
    denom = warp_sum(ex);
  } else {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) s += (lane + 32 * i) < p.E ? __expf(v[i] - vmax) : 0.f;
    denom = warp_sum(s);
  }
  if (lane < p.k) {
    const int a = t * p.k + lane;
    p.ids[a] = sel_id;
    p.weights[a] = ex / denom;
    p.pos[a] = atomicAdd(p.hist + sel_id, 1);
  }
  if (lane == 0 && p.shared_gate != nullptr)
    p.shared_gate[t] = p.has_shared_gate ? 1.f / (1.f + __expf(-__bfloat162float(row[p.E]))) : 1.f;
}

// ---------------------------------------------------------------------------------------------
// moe_plan: one CTA
// ---------------------------------------------------------------------------------------------
constexpr int kPlanThreads = 512;

__global__ void __launch_bounds__(kPlanThreads) moe_plan_kernel(const MoePlanParams p) {
  __shared__ int total_s[kMoeMaxExperts];
  __shared__ int before_s[kMoeMaxExperts];
  __shared__ int ntile_s[kMoeMaxExperts];
  __shared__ int tstart_s[kMoeMaxExperts];
  __shared__ int ok_s, overflow_s, ntiles_s;
  const int tid = threadIdx.x;
  const int W = p.world, E = p.E, El = p.E / p.world;
  const unsigned int c = p.state->call_idx;
  if (tid == 0) { overflow_s = 0; ntiles_s = 0; }

  // 1. my histogram goes to every rank (own copy included)
  for (int e = tid; e < E; e += kPlanThreads) {
    const int h = p.hist[e];
    for (int r = 0; r < W; ++r) p.peer_counts[r][p.rank * E + e] = h;
  }
  if (W == 1) __threadfence(); else __threadfence_system();   // one GPU: device scope is enough (and much cheaper)
  __syncthreads();
  if (tid < W) {
    if (W == 1) red_release_gpu_add(p.peer_count_flag[tid], 1u);
    else red_release_sys_add(p.peer_count_flag[tid], 1u);
  }
  if (tid == 0) ok_s = wait_counter(p.my_count_flag, (c + 1u) * static_cast<uint32_t>(W), p.status) ? 1 : 0;
  __syncthreads();
  const bool ok = ok_s != 0;

  // 2. totals per expert and the number of rows of lower-ranked sources
  for (int e = tid; e < E; e += kPlanThreads) {
    int tot = 0, mine = 0;
    if (ok) {
      for (int s = 0; s < W; ++s) {
        const int v = __ldcg(p.my_counts + s * E + e);
        tot += v;
        if (s < p.rank) mine += v;
      }
    }
    total_s[e] = tot;
    before_s[e] = mine;
  }
  __syncthreads();

  // 3. slot of my group inside each destination's buffer; overflow verdict (identical on every rank)
  for (int e = tid; e < E; e += kPlanThreads) {
    const int seg0 = (e / El) * El;
    int base = 0;
    for (int i = seg0; i < e; ++i) base += total_s[i];
    p.send_base[e] = base + before_s[e];
    if (e == seg0 + El - 1 && base + total_s[e] > p.cap) atomicExch(&overflow_s, 1);
    if (e / El == p.rank) {
      const int i = e - seg0;
      ntile_s[i] = (total_s[e] + p.tile_tokens - 1) / p.tile_tokens;
      tstart_s[i] = base;  // row start, replaced by the tile start below
    }
  }
  __syncthreads();
  const bool overflow = overflow_s != 0;
  if (overflow) report_status(p.status, kStatusBadArgument);

  // 4. tile table of my experts
  if (tid == 0) {
    int run = 0, rows = 0;
    for (int i = 0; i < El; ++i) {
      const int n = ntile_s[i];
      ntile_s[i] = run;  // exclusive scan in place
      run += n;
      rows += total_s[p.rank * El + i];
    }
    ntiles_s = run;
    p.state->total_rows = rows;
  }
  __syncthreads();
  for (int i = tid; i < El; i += kPlanThreads) {
    const int cnt = total_s[p.rank * El + i];
    const int row0 = tstart_s[i];
    const int first = ntile_s[i];
    const int n = (cnt + p.tile_tokens - 1) / p.tile_tokens;
    for (int j = 0; j < n; ++j) {
      const int idx = first + j;
      if (idx < p.max_tiles) {
        p.tile_expert[idx] = i;
        p.tile_row0[idx] = row0 + j * p.tile_tokens;
        p.tile_rows[idx] = min(p.tile_tokens, cnt - j * p.tile_tokens);
      }
    }
  }
  for (int e = tid; e < E; e += kPlanThreads) p.hist[e] = 0;
  __syncthreads();
  if (tid == 0) {
    const bool usable = ok && !overflow && ntiles_s <= p.max_tiles;
    p.state->n_tiles = usable ? ntiles_s : 0;
    p.state->overflow = (ok && !overflow) ? 0 : 1;
    p.state->call_idx = c + 1u;
  }
}

// ---------------------------------------------------------------------------------------------
// moe_push: dispatch all-to-all by peer stores; CTA 0 finally waits until every source's rows
// have landed here, so the kernel boundary orders them before the grouped GEMM's TMA loads.
// ---------------------------------------------------------------------------------------------
constexpr int kPushThreads = 256;

__global__ void __launch_bounds__(kPushThreads) moe_push_kernel(const MoePushParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int El = p.E / p.world;
  const int n_assign = p.T * p.k;
  const int nvec = p.H / 8;
  if (!p.state->overflow) {
    for (int a = blockIdx.x * (kPushThreads / 32) + warp; a < n_assign; a += gridDim.x * (kPushThreads / 32)) {
      const int e = p.ids[a];
      const int dest = e / El;
      const int slot = p.send_base[e] + p.pos[a];
      if (slot >= p.cap) continue;
      const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(a / p.k) * p.ldx);
      uint4* dst = reinterpret_cast<uint4*>(p.peer_recv_x[dest] + static_cast<long long>(slot) * p.H);
      for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
      if (lane == 0) p.peer_recv_meta[dest][slot] = (p.rank << 24) | a;
    }
  }
  if (p.world == 1) __threadfence();
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (p.world == 1) {
      red_release_gpu_add(p.peer_arrive_flag[threadIdx.x], 1u);
    } else {
      __threadfence_system();   // cumulative over the stores the block barrier ordered before this thread
      red_release_sys_add(p.peer_arrive_flag[threadIdx.x], 1u);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const uint32_t target = p.state->call_idx * static_cast<uint32_t>(p.world) * gridDim.x;
    wait_counter(p.my_arrive_flag, target, p.status);
  }
}

// ---------------------------------------------------------------------------------------------
// moe_combine: one CTA per token
// ---------------------------------------------------------------------------------------------
constexpr int kCombineThreads = 256;

__global__ void __launch_bounds__(kCombineThreads) moe_combine_kernel(const MoeCombineParams p) {
  __shared__ float red[kCombineThreads / 32];
  __shared__ int ok_s;
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  MoeState* st = p.state;
  const bool skip = st->overflow != 0;
  const uint32_t target = st->ret_expected + (skip ? 0u : p.arrivals_this_call);
  if (threadIdx.x == 0) ok_s = skip ? 0 : (wait_counter(p.ret_flag, target, p.status) ? 1 : 0);
  __syncthreads();
  const bool ok = ok_s != 0;
  const int nvec = p.H / 8;
  __nv_bfloat16* xrow = p.x + static_cast<long long>(t) * p.H;
  const float gate = (p.shared != nullptr) ? p.shared_gate[t] : 0.f;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kCombineThreads) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (ok) {
      for (int j = 0; j < p.k; ++j) {
        const float w = p.weights[t * p.k + j];
        const uint4 rv = __ldcg(reinterpret_cast<const uint4*>(p.ret + (static_cast<long long>(t) * p.k + j) * p.H) + v);
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += w * __bfloat162float(rp[i].x);
          acc[2 * i + 1] += w * __bfloat162float(rp[i].y);
        }
      }
    }
    if (p.shared != nullptr) {
      const uint4 sv = *(reinterpret_cast<const uint4*>(p.shared + static_cast<long long>(t) * p.H) + v);
      const __nv_bfloat162* sp = reinterpret_cast<const __nv_bfloat162*>(&sv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += gate * __bfloat162float(sp[i].x);
        acc[2 * i + 1] += gate * __bfloat162float(sp[i].y);
      }
    }
    const uint4 xv = *(reinterpret_cast<const uint4*>(xrow) + v);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat16 lo = __float2bfloat16(__bfloat162float(xp[i].x) + acc[2 * i]);
      const __nv_bfloat16 hi = __float2bfloat16(__bfloat162float(xp[i].y) + acc[2 * i + 1]);
      const float fl = __bfloat162float(lo), fh = __bfloat162float(hi);
      ss += fl * fl + fh * fh;
      op[i] = pack_bf16x2(fl, fh);
    }
    *(reinterpret_cast<uint4*>(xrow) + v) = o;
  }
  if (p.normed != nullptr) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kCombineThreads / 32; ++w) tot += red[w];
    const float inv = rsqrtf(tot / static_cast<float>(p.H) + p.eps);
    for (int v = threadIdx.x; v < nvec; v += kCombineThreads) {
      const uint4 xv = *(reinterpret_cast<const uint4*>(xrow) + v);  // written by this thread above
      const uint4 wv = *(reinterpret_cast<const uint4*>(p.norm_w) + v);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        op[i] = pack_bf16x2(__bfloat162float(xp[i].x) * inv * (1.f + __bfloat162float(wp[i].x)),
                            __bfloat162float(xp[i].y) * inv * (1.f + __bfloat162float(wp[i].y)));
      *(reinterpret_cast<uint4*>(p.normed + static_cast<long long>(t) * p.H) + v) = o;
    }
  }
  // the last CTA to finish closes the call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&st->ctas_done, 1u) == gridDim.x - 1) {
      st->ret_expected = target;
      st->ctas_done = 0;
    }
  }
}

const char* launch_error(cudaError_t e) { return e == cudaSuccess ? nullptr : cudaGetErrorString(e); }

}  // namespace

const char* moe_route(const MoeRouteParams& p, cudaStream_t stream) {
  if (p.T <= 0) return nullptr;
  if (p.E < 1 || p.E > kMoeMaxExperts) return "moe_route: expert count out of range";
  if (p.k < 1 || p.k > kMoeMaxTopK || p.k > p.E) return "moe_route: top-k out of range";
  moe_route_kernel<<<(p.T + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, 0, stream>>>(p);
  return launch_error(cudaGetLastError());
}

const char* moe_plan(const MoePlanParams& p, cudaStream_t stream) {
  if (p.world < 1 || p.world > kMoeMaxRanks || p.rank < 0 || p.rank >= p.world) return "moe_plan: bad rank/world";
  if (p.E < 1 || p.E > kMoeMaxExperts || p.E % p.world) return "moe_plan: experts must divide evenly over ranks";
  if (p.tile_tokens < 16 || p.cap < 1 || p.max_tiles < 1) return "moe_plan: bad tile geometry";
  moe_plan_kernel<<<1, kPlanThreads, 0, stream>>>(p);
  return launch_error(cudaGetLastError());
}

const char* moe_push(const MoePushParams& p, cudaStream_t stream) {
  if (p.H % 8 || p.ldx % 8) return "moe_push: hidden size and row stride must be multiples of 8";
  if (p.T * static_cast<long long>(p.k) >= (1 << 24)) return "moe_push: too many assignments per call";
  moe_push_kernel<<<kMoePushCtas, kPushThreads, 0, stream>>>(p);
  return launch_error(cudaGetLastError());
}

const char* moe_combine(const MoeCombineParams& p, cudaStream_t stream) {
  if (p.T <= 0) return nullptr;
  if (p.H % 8) return "moe_combine: hidden size must be a multiple of 8";
  moe_combine_kernel<<<p.T, kCombineThreads, 0, stream>>>(p);
  return launch_error(cudaGetLastError());
}

}  // namespace nfb
