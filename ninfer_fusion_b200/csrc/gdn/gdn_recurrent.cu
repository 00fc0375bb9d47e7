// Gated delta-rule recurrence with the fp32 state held in registers for the
// whole token loop: one CTA per (value head, sequence).  Eight lanes share a
// state row (each owns 16 of its 128 columns as four interleaved float4), so a
// warp instruction moves four fully used 128-byte lines and a thread owns four
// rows -> 64 state registers, <= 128 registers in total, two CTAs per SM, which
// lets one CTA's state load overlap the other's store.  Fused in the same pass:
// q/k L2 normalisation, the gating non-linearities (softplus/exp/sigmoid) and the
// per-head gated RMSNorm epilogue, so a decode step reads and writes each 64 KB
// state exactly once.  Used for decode (1 token per sequence), verify
// (write_state = 0, state untouched, the accepted prefix is replayed afterwards
// with write_state = 1) and as the sequential prefill path.
//
// Reference: include/ninfer/ops/gated_delta_net.h:26-112, gdn_gating.h,
// gated_rmsnorm.h, src/ops/linear_attention/gated_delta_net/recurrent.cuh.
#include "gdn.h"

#include "../common/ptx.cuh"

namespace nfb {

namespace {

constexpr int kDk = 128, kDv = 128;
constexpr int kThreads = 256;
constexpr int kRowsPerThread = 4;

__global__ void __launch_bounds__(kThreads, 2) gdn_recurrent_kernel(const GdnParams p) {
  __shared__ __align__(16) float k_s[kThreads / 32][kDk];
  __shared__ __align__(16) float q_s[kThreads / 32][kDk];
  __shared__ float red[2][kThreads / 32];

  pdl_launch_next();
  // The step description (sequence ranges, state slots) is uploaded before the step's first kernel and the state
  // was last written by this kernel one step earlier, so neither depends on the kernel right before this one: the
  // 64 KB state load is issued BEFORE waiting for that kernel and overlaps its tail.  A replay pass reads
  // per-sequence ends that a kernel of this very step computed: it waits first.
  if (p.seq_end != nullptr) pdl_wait_prior();
  const int hv = blockIdx.x, seq = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, q8 = lane & 7;
  const int hk = hv / (p.n_v_heads / p.n_qk_heads);
  const int t_begin = p.cu_seqlens[seq], t_end = p.seq_end != nullptr ? p.seq_end[seq] : p.cu_seqlens[seq + 1];
  if (t_end <= t_begin) {
    pdl_wait_prior();   // every CTA waits before it leaves: a later kernel's wait then still implies all earlier ones
    return;
  }
  const int slot = p.state_slot[seq];

  // thread's rows: r_j = warp*16 + j*4 + sub ; columns: float4 index q8 + 8*i
  float* sbase = p.state + (static_cast<long long>(slot) * p.n_v_heads + hv) * kDv * kDk;
  float4 S[kRowsPerThread][4];
#pragma unroll
  for (int j = 0; j < kRowsPerThread; ++j) {
    const int r = warp * 16 + j * 4 + sub;
#pragma unroll
    for (int i = 0; i < 4; ++i) S[j][i] = reinterpret_cast<const float4*>(sbase + r * kDk)[q8 + 8 * i];
  }
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const float qscale = rsqrtf(static_cast<float>(kDk));
  if (p.seq_end == nullptr) pdl_wait_prior();   // the projections of this step's tokens come from the previous kernel

  for (int t = t_begin; t < t_end; ++t) {
    // ---- per-warp copy of the normalised q, k of this token ----
    const __nv_bfloat16* row = p.qkv + static_cast<long long>(t) * p.ld_qkv;
    const uint2 kr = *reinterpret_cast<const uint2*>(row + p.k_off + hk * kDk + lane * 4);
    const uint2 qr = *reinterpret_cast<const uint2*>(row + p.q_off + hk * kDk + lane * 4);
    const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kr);
    const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qr);
    const float kf[4] = {__bfloat162float(kp[0].x), __bfloat162float(kp[0].y), __bfloat162float(kp[1].x), __bfloat162float(kp[1].y)};
    const float qf[4] = {__bfloat162float(qp[0].x), __bfloat162float(qp[0].y), __bfloat162float(qp[1].x), __bfloat162float(qp[1].y)};
    const float ssk = warp_sum(kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3]);
    const float ssq = warp_sum(qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3]);
    const float ik = rsqrtf(ssk + 1e-6f), iq = rsqrtf(ssq + 1e-6f) * qscale;
    __syncwarp();
    *reinterpret_cast<float4*>(&k_s[warp][lane * 4]) = make_float4(kf[0] * ik, kf[1] * ik, kf[2] * ik, kf[3] * ik);
    *reinterpret_cast<float4*>(&q_s[warp][lane * 4]) = make_float4(qf[0] * iq, qf[1] * iq, qf[2] * iq, qf[3] * iq);
    __syncwarp();
    float4 k4[4], q4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      k4[i] = reinterpret_cast<const float4*>(k_s[warp])[q8 + 8 * i];
      q4[i] = reinterpret_cast<const float4*>(q_s[warp])[q8 + 8 * i];
    }

    const __nv_bfloat16* prow = p.proj + static_cast<long long>(t) * p.ld_proj;
    const float a = __bfloat162float(prow[p.a_off + hv]);
    const float b = __bfloat162float(prow[p.b_off + hv]);
    const float x = a + dtb;
    const float sp_x = x > 20.f ? x : log1pf(__expf(x));
    const float alpha = __expf(neg_a * sp_x);
    const float beta = 1.f / (1.f + __expf(-b));

    // side-branch tokens (commit[t] == 0) read the state but do not change it:  o = alpha * (S q) + u * (k . q)
    const bool cm = p.commit == nullptr || p.commit[t] != 0;
    float kq = 0.f;
    if (!cm) {
#pragma unroll
      for (int i = 0; i < 4; ++i) kq += k4[i].x * q4[i].x + k4[i].y * q4[i].y + k4[i].z * q4[i].z + k4[i].w * q4[i].w;
      kq += __shfl_xor_sync(0xffffffffu, kq, 1);
      kq += __shfl_xor_sync(0xffffffffu, kq, 2);
      kq += __shfl_xor_sync(0xffffffffu, kq, 4);
    }
    float o[kRowsPerThread];
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < kRowsPerThread; ++j) {
      const int r = warp * 16 + j * 4 + sub;
      const float v = __bfloat162float(row[p.v_off + hv * kDv + r]);
      // same summation tree as the prefill kernels, so decode, prefill and replay stay bit-consistent
      float kp4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        kp4[i] = S[j][i].x * k4[i].x + S[j][i].y * k4[i].y + S[j][i].z * k4[i].z + S[j][i].w * k4[i].w;
      float ks = (kp4[0] + kp4[1]) + (kp4[2] + kp4[3]);
      ks += __shfl_xor_sync(0xffffffffu, ks, 1);
      ks += __shfl_xor_sync(0xffffffffu, ks, 2);
      ks += __shfl_xor_sync(0xffffffffu, ks, 4);
      const float u = beta * (v - alpha * ks);
      float oj = 0.f;
      if (cm) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          S[j][i].x = alpha * S[j][i].x + u * k4[i].x;
          S[j][i].y = alpha * S[j][i].y + u * k4[i].y;
          S[j][i].z = alpha * S[j][i].z + u * k4[i].z;
          S[j][i].w = alpha * S[j][i].w + u * k4[i].w;
          oj += S[j][i].x * q4[i].x + S[j][i].y * q4[i].y + S[j][i].z * q4[i].z + S[j][i].w * q4[i].w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          oj += S[j][i].x * q4[i].x + S[j][i].y * q4[i].y + S[j][i].z * q4[i].z + S[j][i].w * q4[i].w;
        oj *= alpha;
      }
      oj += __shfl_xor_sync(0xffffffffu, oj, 1);
      oj += __shfl_xor_sync(0xffffffffu, oj, 2);
      oj += __shfl_xor_sync(0xffffffffu, oj, 4);
      if (!cm) oj += u * kq;
      oj = __bfloat162float(__float2bfloat16(oj));  // bf16 boundary before the head norm
      o[j] = oj;
      if (q8 == 0) sq += oj * oj;
    }

    // ---- gated RMSNorm over the head's 128 outputs ----
    sq = warp_sum(sq);
    const int par = (t - t_begin) & 1;
    if (lane == 0) red[par][warp] = sq;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) tot += red[par][w];
    const float inv = rsqrtf(tot / kDv + p.eps);
    if (q8 < kRowsPerThread) {
      // lane q8 of each 8-lane group writes row j = q8 (all eight lanes hold all four o[j])
      float oj = o[0];
#pragma unroll
      for (int j = 1; j < kRowsPerThread; ++j) oj = (q8 == j) ? o[j] : oj;
      const int r = warp * 16 + q8 * 4 + sub;
      const float z = __bfloat162float(prow[p.z_off + hv * kDv + r]);
      const float nw = __bfloat162float(p.norm_w[r]);
      const float y = oj * inv * nw * (z / (1.f + __expf(-z)));
      p.out[static_cast<long long>(t) * (p.n_v_heads * kDv) + hv * kDv + r] = __float2bfloat16(y);
    }
  }

  if (p.write_state) {
#pragma unroll
    for (int j = 0; j < kRowsPerThread; ++j) {
      const int r = warp * 16 + j * 4 + sub;
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(sbase + r * kDk)[q8 + 8 * i] = S[j][i];
    }
  }
}

}  // namespace

const char* gdn_recurrent(const GdnParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0 || p.n_seq <= 0) return nullptr;
  if (p.n_v_heads % p.n_qk_heads) return "gdn_recurrent: value heads must be a multiple of qk heads";
  if ((p.q_off | p.k_off | p.ld_qkv) % 4) return "gdn_recurrent: q/k offsets must be multiples of 4";
  if (p.T > p.n_seq && (p.v_off | p.z_off | p.ld_proj) % 4 == 0) return gdn_prefill(p, stream, pdl);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_v_heads, p.n_seq); cfg.blockDim = dim3(kThreads); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gdn_recurrent_kernel, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
