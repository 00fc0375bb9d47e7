// Gated delta-rule recurrence with the fp32 state held in registers for the
// whole token loop: one CTA per (value head, sequence), thread (r, half) owns
// S[r][64*half .. 64*half+63].  Fused in the same pass: q/k L2 normalisation,
// the gating non-linearities (softplus/exp/sigmoid) and the per-head gated
// RMSNorm epilogue, so a decode step is one launch that reads and writes each
// 64 KB state exactly once.  Used for decode (1 token per sequence), verify
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

__global__ void __launch_bounds__(kThreads) gdn_recurrent_kernel(const GdnParams p) {
  __shared__ __align__(16) float k_s[kThreads / 32][kDk];
  __shared__ __align__(16) float q_s[kThreads / 32][kDk];
  __shared__ float red[2][kThreads / 32];

  pdl_launch_next();
  pdl_wait_prior();
  const int hv = blockIdx.x, seq = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = threadIdx.x >> 1, half = threadIdx.x & 1;
  const int hk = hv / (p.n_v_heads / p.n_qk_heads);
  const int t_begin = p.cu_seqlens[seq], t_end = p.cu_seqlens[seq + 1];
  if (t_end <= t_begin) return;
  const int slot = p.state_slot[seq];

  float* sp = p.state + ((static_cast<long long>(slot) * p.n_v_heads + hv) * kDv + r) * kDk + half * 64;
  float S[64];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float4 v = reinterpret_cast<const float4*>(sp)[i];
    S[4 * i] = v.x; S[4 * i + 1] = v.y; S[4 * i + 2] = v.z; S[4 * i + 3] = v.w;
  }
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const float nw = __bfloat162float(p.norm_w[r]);
  const float qscale = rsqrtf(static_cast<float>(kDk));

  for (int t = t_begin; t < t_end; ++t) {
    // ---- per-warp copy of the normalised q, k of this token ----
    const __nv_bfloat16* row = p.qkv + static_cast<long long>(t) * p.ld_qkv;
    const uint2 kr = *reinterpret_cast<const uint2*>(row + p.k_off + hk * kDk + lane * 4);
    const uint2 qr = *reinterpret_cast<const uint2*>(row + p.q_off + hk * kDk + lane * 4);
    const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kr);
    const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qr);
    float kf[4] = {__bfloat162float(kp[0].x), __bfloat162float(kp[0].y), __bfloat162float(kp[1].x), __bfloat162float(kp[1].y)};
    float qf[4] = {__bfloat162float(qp[0].x), __bfloat162float(qp[0].y), __bfloat162float(qp[1].x), __bfloat162float(qp[1].y)};
    const float ssk = warp_sum(kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3]);
    const float ssq = warp_sum(qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3]);
    const float ik = rsqrtf(ssk + 1e-6f), iq = rsqrtf(ssq + 1e-6f) * qscale;
    __syncwarp();
    *reinterpret_cast<float4*>(&k_s[warp][lane * 4]) = make_float4(kf[0] * ik, kf[1] * ik, kf[2] * ik, kf[3] * ik);
    *reinterpret_cast<float4*>(&q_s[warp][lane * 4]) = make_float4(qf[0] * iq, qf[1] * iq, qf[2] * iq, qf[3] * iq);
    __syncwarp();

    const __nv_bfloat16* prow = p.proj + static_cast<long long>(t) * p.ld_proj;
    const float a = __bfloat162float(prow[p.a_off + hv]);
    const float b = __bfloat162float(prow[p.b_off + hv]);
    const float v = __bfloat162float(row[p.v_off + hv * kDv + r]);
    const float x = a + dtb;
    const float sp_x = x > 20.f ? x : log1pf(__expf(x));
    const float alpha = __expf(neg_a * sp_x);
    const float beta = 1.f / (1.f + __expf(-b));

    // kS = (alpha * S) k
    float ks = 0.f;
    const float4* k4 = reinterpret_cast<const float4*>(&k_s[warp][half * 64]);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float4 kk = k4[i];
      ks += S[4 * i] * kk.x + S[4 * i + 1] * kk.y + S[4 * i + 2] * kk.z + S[4 * i + 3] * kk.w;
    }
    ks += __shfl_xor_sync(0xffffffffu, ks, 1);
    const float u = beta * (v - alpha * ks);
    float o = 0.f;
    const float4* q4 = reinterpret_cast<const float4*>(&q_s[warp][half * 64]);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float4 kk = k4[i];
      const float4 qq = q4[i];
      S[4 * i] = alpha * S[4 * i] + u * kk.x;
      S[4 * i + 1] = alpha * S[4 * i + 1] + u * kk.y;
      S[4 * i + 2] = alpha * S[4 * i + 2] + u * kk.z;
      S[4 * i + 3] = alpha * S[4 * i + 3] + u * kk.w;
      o += S[4 * i] * qq.x + S[4 * i + 1] * qq.y + S[4 * i + 2] * qq.z + S[4 * i + 3] * qq.w;
    }
    o += __shfl_xor_sync(0xffffffffu, o, 1);

    // ---- gated RMSNorm over the head's 128 outputs (bf16 boundary first) ----
    o = __bfloat162float(__float2bfloat16(o));
    const float sq = warp_sum(half == 0 ? o * o : 0.f);
    const int par = (t - t_begin) & 1;
    if (lane == 0) red[par][warp] = sq;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) tot += red[par][w];
    if (half == 0) {
      const float z = __bfloat162float(prow[p.z_off + hv * kDv + r]);
      const float y = o * rsqrtf(tot / kDv + p.eps) * nw * (z / (1.f + __expf(-z)));
      p.out[static_cast<long long>(t) * (p.n_v_heads * kDv) + hv * kDv + r] = __float2bfloat16(y);
    }
  }

  if (p.write_state) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      reinterpret_cast<float4*>(sp)[i] = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
  }
}

}  // namespace

const char* gdn_recurrent(const GdnParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0 || p.n_seq <= 0) return nullptr;
  if (p.n_v_heads % p.n_qk_heads) return "gdn_recurrent: value heads must be a multiple of qk heads";
  if ((p.q_off | p.k_off | p.ld_qkv) % 4) return "gdn_recurrent: q/k offsets must be multiples of 4";
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
