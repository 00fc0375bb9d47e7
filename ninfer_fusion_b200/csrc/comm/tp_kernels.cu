// Tensor-parallel collectives written as peer-memory kernels (NVLink P2P
// loads/stores + release/acquire counters in symmetric buffers).
//
// tp_reduce_ag_norm finishes a row-parallel GEMM whose epilogue already pushed
// fp32 partial tiles into the owner ranks (gemm kEpiPushPartial):
//   phase A (owner of a column slice): wait for all arrivals, sum partials over
//           ranks and K-splits, add the residual, round to bf16, store the new
//           residual slice into EVERY rank's residual buffer (all-gather by
//           push) together with the slice's sum of squares, bump each rank's
//           per-row counter;
//   phase B (every rank): wait until the row has all W slices, combine the W
//           sums of squares and write the RMS-normalised row that feeds the
//           next column-parallel GEMM.
// One CTA per token row; CTAs never wait on other CTAs of the same GPU, only on
// counters that remote GPUs advance, so no co-residency is required.  Every
// wait is bounded and reports kStatusPeerWaitTimeout instead of hanging.
//
// The reference has no counterpart: its multi-device code is host-only shard
// arithmetic plus a 2-rank pull all-reduce seam (src/core/tp_transport.h:1045-1366,
// include/ninfer/ops/allreduce.h).  The counter protocol keeps that seam's rules:
// counters only grow, waits are ">=", a buffer is reused only after the
// consumer's completion is implied by a later arrival.
#include "comm.h"

#include <math_constants.h>

#include "../common/ptx.cuh"
#include "peer_sync.cuh"

namespace nfb {

namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads) tp_reduce_ag_norm_kernel(const TpReduceParams p) {
  __shared__ float red[kThreads / 32];
  __shared__ int ok_s;
  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  const int W = p.world, me = p.rank;
  const int slice = p.N / W;
  const int c0 = me * slice;
  TpState* st = p.state;

  // ---- phase A: reduce my column slice of row t ----
  const bool do_a = (p.phases & 1) != 0, do_b = (p.phases & 2) != 0;
  const uint32_t target1 = st->expected_arrivals + p.arrivals_this_call;
  if (threadIdx.x == 0) ok_s = (!do_a || wait_counter(p.my_arrival_flag, target1, p.status)) ? 1 : 0;
  __syncthreads();
  const bool ok = ok_s != 0;
  float ss = 0.f;
  const int nvec = slice / 4;
  if (ok && do_a) {
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int src = 0; src < W * p.splits; ++src) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(
            p.my_recv + (static_cast<long long>(src) * p.T + t) * slice + v * 4));
        acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
      }
      const uint2 rv = *reinterpret_cast<const uint2*>(p.my_x + static_cast<long long>(t) * p.N + c0 + v * 4);
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
      uint2 o;
      o.x = pack_bf16x2(acc.x + __bfloat162float(rp[0].x), acc.y + __bfloat162float(rp[0].y));
      o.y = pack_bf16x2(acc.z + __bfloat162float(rp[1].x), acc.w + __bfloat162float(rp[1].y));
      const __nv_bfloat162* op = reinterpret_cast<const __nv_bfloat162*>(&o);
      const float f0 = __bfloat162float(op[0].x), f1 = __bfloat162float(op[0].y);
      const float f2 = __bfloat162float(op[1].x), f3 = __bfloat162float(op[1].y);
      ss += f0 * f0 + f1 * f1 + f2 * f2 + f3 * f3;
      for (int r = 0; r < W; ++r)  // all-gather by push (own copy included)
        *reinterpret_cast<uint2*>(p.peer_x[r] + static_cast<long long>(t) * p.N + c0 + v * 4) = o;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();   // orders every thread's peer stores before the signalling threads below
  const uint32_t row_epoch = st->row_calls[t];
  if (threadIdx.x < W && ok && do_a) {
    // thread r signals rank r: its release (system scope) is cumulative over the stores the barrier ordered, so
    // neither the other 255 threads nor this one need a separate system fence
    float tot = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) tot += red[w];
    // the sum of squares travels in a double-buffered slot so a fast peer's next call cannot overwrite it
    const int par = row_epoch & 1;
    const int r = threadIdx.x;
    p.peer_ss[r][(static_cast<long long>(par) * p.T_cap + t) * W + me] = tot;
    red_release_sys_add(p.peer_row_flag[r] + t, 1u);
  }

  // ---- phase B: the whole row is here once all W slices have arrived ----
  if (threadIdx.x == 0) {
    ok_s = ok && do_b && wait_counter(p.my_row_flag + t, (row_epoch + 1u) * static_cast<uint32_t>(W), p.status) ? 1 : 0;
  }
  __syncthreads();
  if (ok_s && p.normed != nullptr) {
    float tot = 0.f;
    const int par = row_epoch & 1;
    for (int r = 0; r < W; ++r) tot += __ldcg(p.my_ss + (static_cast<long long>(par) * p.T_cap + t) * W + r);
    const float inv = rsqrtf(tot / static_cast<float>(p.N) + p.eps);
    for (int v = threadIdx.x; v < p.N / 8; v += kThreads) {
      const uint4 xv = __ldcg(reinterpret_cast<const uint4*>(p.my_x + static_cast<long long>(t) * p.N + v * 8));
      const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + v * 8);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float w0 = __bfloat162float(wp[j].x), w1 = __bfloat162float(wp[j].y);
        if (p.unit_offset) { w0 += 1.f; w1 += 1.f; }
        op[j] = pack_bf16x2(__bfloat162float(xp[j].x) * inv * w0, __bfloat162float(xp[j].y) * inv * w1);
      }
      *reinterpret_cast<uint4*>(p.normed + static_cast<long long>(t) * p.N + v * 8) = o;
    }
  }

  // ---- bookkeeping: the last CTA to finish advances the call-level expectations ----
  __syncthreads();
  if (threadIdx.x == 0) {
    if (do_b) st->row_calls[t] = row_epoch + 1u;
    if (do_a) {
      __threadfence();
      const unsigned int done = atomicAdd(&st->ctas_done, 1u);
      if (done == gridDim.x - 1) {
        st->expected_arrivals = target1;
        st->ctas_done = 0;
        __threadfence();
      }
    }
  }
}

// Vocabulary-parallel arg-max: each rank scans its logits slice, pushes (value, global id) to
// every rank and picks the winner (highest value, lowest id on ties) once all W candidates are in.
__global__ void __launch_bounds__(1024) tp_argmax_kernel(const TpArgmaxParams p) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  const __nv_bfloat16* row = p.logits + static_cast<long long>(t) * p.ld;
  const bool do_push = (p.phases & 1) != 0, do_pick = (p.phases & 2) != 0;
  float best = -CUDART_INF_F;
  int idx = 0x7fffffff;
  // 16-byte loads when the row allows it (8 logits per load, ascending ids: strict > keeps the lowest id)
  const bool vec = (p.ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.logits) & 15) == 0);
  const int nvec = (do_push && vec) ? p.V_local / 8 : 0;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    const uint4 r = *reinterpret_cast<const uint4*>(row + c * 8);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = __bfloat162float(e[j]);
      if (f > best) { best = f; idx = c * 8 + j; }
    }
  }
  for (int i = nvec * 8 + threadIdx.x; do_push && i < p.V_local; i += blockDim.x) {
    const float f = __bfloat162float(row[i]);
    if (f > best || (f == best && i < idx)) { best = f; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x >= 32) return;
  best = threadIdx.x < (blockDim.x >> 5) ? bv[threadIdx.x] : -CUDART_INF_F;
  idx = threadIdx.x < (blockDim.x >> 5) ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if (threadIdx.x != 0) return;
  TpState* st = p.state;
  const uint32_t epoch = st->argmax_calls[t];
  const int par = epoch & 1;
  const int W = p.world;
  if (do_push) {
    for (int r = 0; r < W; ++r) {
      float2* slot = p.peer_cand[r] + (static_cast<long long>(par) * p.T_cap + t) * W + p.rank;
      *slot = make_float2(best, __int_as_float(idx + p.rank * p.V_local));
    }
    __threadfence_system();
    for (int r = 0; r < W; ++r) red_release_sys_add(p.peer_flag[r] + t, 1u);
  }
  if (!do_pick) return;
  if (wait_counter(p.my_flag + t, (epoch + 1u) * static_cast<uint32_t>(W), p.status)) {
    float gb = -CUDART_INF_F;
    int gi = 0x7fffffff;
    for (int r = 0; r < W; ++r) {
      const float2 c = __ldcg(p.my_cand + (static_cast<long long>(par) * p.T_cap + t) * W + r);
      const int ci = __float_as_int(c.y);
      if (c.x > gb || (c.x == gb && ci < gi)) { gb = c.x; gi = ci; }
    }
    p.out[t] = gi;
  }
  st->argmax_calls[t] = epoch + 1u;
}

// ---- one-shot all-reduce finish (decode sizes): 8-CTA cluster per row ----
constexpr int kRowCluster = 8;
constexpr int kRowThreads = 128;

__global__ void __launch_bounds__(kRowThreads) tp_sum_norm_kernel(const TpSumNormParams p) {
  __shared__ float red[kRowThreads / 32];
  __shared__ float cta_ss;
  __shared__ int ok_s;
  pdl_launch_next();
  pdl_wait_prior();
  TpState* st = p.state;
  const long long row = blockIdx.x / kRowCluster;
  uint32_t crank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  const int cols = p.N / kRowCluster;
  const int c = crank * cols + threadIdx.x * 8;
  const bool active = threadIdx.x * 8 < cols;
  const uint32_t target = st->expected_all + p.arrivals_this_call;
  const uint32_t par = st->call_idx & 1u;
  if (threadIdx.x == 0) ok_s = wait_counter(p.my_flag, target, p.status) ? 1 : 0;
  __syncthreads();
  float v[8];
  float ss = 0.f;
  if (active && ok_s) {
    float acc[8];
    const uint4 r = *reinterpret_cast<const uint4*>(p.x + row * p.N + c);
    const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[2 * j] = __bfloat162float(rp[j].x); acc[2 * j + 1] = __bfloat162float(rp[j].y); }
    for (int src = 0; src < p.world; ++src) {
      const float4* pp = reinterpret_cast<const float4*>(
          p.my_recv + ((static_cast<long long>(par) * p.world + src) * p.T_cap + row) * p.N + c);
      const float4 a = __ldcg(pp), b = __ldcg(pp + 1);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      op[j] = pack_bf16x2(acc[2 * j], acc[2 * j + 1]);
      const __nv_bfloat162 b2 = *reinterpret_cast<__nv_bfloat162*>(&op[j]);
      v[2 * j] = __bfloat162float(b2.x);
      v[2 * j + 1] = __bfloat162float(b2.y);
      ss += v[2 * j] * v[2 * j] + v[2 * j + 1] * v[2 * j + 1];
    }
    *reinterpret_cast<uint4*>(p.x + row * p.N + c) = o;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kRowThreads / 32; ++w) t += red[w];
    cta_ss = t;
  }
  cluster_sync_all();
  float tot = 0.f;
  const uint32_t local = smem_u32(&cta_ss);
#pragma unroll
  for (uint32_t r = 0; r < kRowCluster; ++r) {
    float f;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(f) : "r"(mapa_shared(local, r)));
    tot += f;
  }
  cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  if (p.normed != nullptr && active && ok_s) {
    const float inv = rsqrtf(tot / static_cast<float>(p.N) + p.eps);
    const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + c);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float w0 = __bfloat162float(wp[j].x), w1 = __bfloat162float(wp[j].y);
      if (p.unit_offset) { w0 += 1.f; w1 += 1.f; }
      op[j] = pack_bf16x2(v[2 * j] * inv * w0, v[2 * j + 1] * inv * w1);
    }
    *reinterpret_cast<uint4*>(p.normed + row * p.N + c) = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(&st->ctas_done_all, 1u);
    if (done == gridDim.x - 1) {
      st->expected_all = target;
      st->call_idx = st->call_idx + 1u;
      st->ctas_done_all = 0;
      __threadfence();
    }
  }
}

// Wait for the all-gathered residual stream, then RMS-normalise it: one CTA per token row.
__global__ void __launch_bounds__(kThreads) tp_gather_norm_kernel(const TpGatherNormParams p) {
  __shared__ float red[kThreads / 32];
  __shared__ int ok_s;
  pdl_launch_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  if (threadIdx.x == 0) ok_s = wait_counter(p.flag, __ldcg(p.target), p.status) ? 1 : 0;
  __syncthreads();
  if (!ok_s) return;
  const __nv_bfloat16* row = p.x + static_cast<long long>(t) * p.ldx;
  float ss = 0.f;
  for (int v = threadIdx.x; v < p.N / 8; v += kThreads) {
    const uint4 xv = __ldcg(reinterpret_cast<const uint4*>(row + v * 8));
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __bfloat162float(xp[j].x), b = __bfloat162float(xp[j].y);
      ss += a * a + b * b;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < kThreads / 32; ++w) tot += red[w];
  const float inv = rsqrtf(tot / static_cast<float>(p.N) + p.eps);
  for (int v = threadIdx.x; v < p.N / 8; v += kThreads) {
    const uint4 xv = __ldcg(reinterpret_cast<const uint4*>(row + v * 8));
    const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + v * 8);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float w0 = __bfloat162float(wp[j].x), w1 = __bfloat162float(wp[j].y);
      if (p.unit_offset) { w0 += 1.f; w1 += 1.f; }
      op[j] = pack_bf16x2(__bfloat162float(xp[j].x) * inv * w0, __bfloat162float(xp[j].y) * inv * w1);
    }
    *reinterpret_cast<uint4*>(p.normed + static_cast<long long>(t) * p.N + v * 8) = o;
  }
}

}  // namespace

const char* tp_gather_norm(const TpGatherNormParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0) return nullptr;
  if (p.N % 8 || p.ldx % 8 || p.N > 65536) return "tp_gather_norm: row width must be a multiple of 8";
  if ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.normed) | reinterpret_cast<uintptr_t>(p.norm_w)) & 15)
    return "tp_gather_norm: operands must be 16-byte aligned";
  if (p.flag == nullptr || p.target == nullptr || p.norm_w == nullptr || p.normed == nullptr)
    return "tp_gather_norm: missing pointer";
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.T); cfg.blockDim = dim3(kThreads); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, tp_gather_norm_kernel, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* tp_sum_norm(const TpSumNormParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0) return nullptr;
  if (p.T > p.T_cap) return "tp_sum_norm: too many rows for the receive buffer";
  if (p.N % (8 * kRowCluster) || p.N / kRowCluster > kRowThreads * 8) return "tp_sum_norm: unsupported row width";
  if (p.normed != nullptr && p.norm_w == nullptr) return "tp_sum_norm: normed output without weight";
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.T * kRowCluster); cfg.blockDim = dim3(kRowThreads); cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kRowCluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, tp_sum_norm_kernel, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* tp_reduce_ag_norm(const TpReduceParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0) return nullptr;
  if (p.T > p.T_cap || p.T > kTpMaxRows) return "tp_reduce_ag_norm: too many rows for the symmetric buffers";
  if (p.world < 1 || p.world > kMaxTpRanks) return "tp_reduce_ag_norm: bad world size";
  if (p.N % (8 * p.world)) return "tp_reduce_ag_norm: N must be a multiple of 8 * world";
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.T); cfg.blockDim = dim3(kThreads); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, tp_reduce_ag_norm_kernel, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* tp_argmax(const TpArgmaxParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0) return nullptr;
  if (p.T > p.T_cap || p.T > kTpMaxRows) return "tp_argmax: too many rows for the symmetric buffers";
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.T); cfg.blockDim = dim3(1024); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, tp_argmax_kernel, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
