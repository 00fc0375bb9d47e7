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
#include "../gemm/nvfp4_act.cuh"

namespace nfb {

namespace {

constexpr int kDk = 128, kDv = 128;
constexpr int kThreads = 256;
constexpr int kRowsPerThread = 4;

__global__ void __launch_bounds__(kThreads, 2) gdn_recurrent_kernel(const GdnParams p) {
  __shared__ __align__(16) float k_s[kThreads / 32][kDk];
  __shared__ __align__(16) float q_s[kThreads / 32][kDk];
  __shared__ float red[2][kThreads / 32];
  __shared__ __align__(16) float conv_q[kDk], conv_k[kDk], conv_v[kDv];   // fused-conv decode: this CTA's q, k, v rows

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
  const int ratio = p.n_v_heads / p.n_qk_heads;
  const bool fused = p.conv_w != nullptr;
  if (t_end <= t_begin) {
    pdl_wait_prior();   // every CTA waits before it leaves: a later kernel's wait then still implies all earlier ones
    if (fused && ratio > 1) cluster_sync_all();   // (the cluster's CTAs share the sequence: all of them are here)
    return;
  }
  const int slot = p.state_slot[seq];
  // fused conv: thread i < 128 owns q channel i and v channel i of this CTA's heads, thread 128 + i k channel i.  The
  // history is as old as the state (written one step ago): it is requested before the dependency wait as well.
  const int ci = threadIdx.x & 127;
  const int ch_a = threadIdx.x < 128 ? p.q_off + hk * kDk + ci : p.k_off + hk * kDk + ci;
  const int ch_v = p.v_off + hv * kDv + ci;
  float hist_a[3] = {0.f, 0.f, 0.f}, hist_v[3] = {0.f, 0.f, 0.f};
  __nv_bfloat16* st_a = nullptr;
  __nv_bfloat16* st_v = nullptr;
  if (fused) {
    st_a = p.conv_state + static_cast<long long>(slot) * 3 * p.conv_C + ch_a;
    st_v = p.conv_state + static_cast<long long>(slot) * 3 * p.conv_C + ch_v;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      hist_a[j] = __bfloat162float(st_a[j * p.conv_C]);
      if (threadIdx.x < 128) hist_v[j] = __bfloat162float(st_v[j * p.conv_C]);
    }
  }

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

  if (fused) {
    // four taps + SiLU on this CTA's 384 channels, rounded to bf16 like the separate kernel's output; then the roll
    const __nv_bfloat16* xrow = p.qkv + static_cast<long long>(t_begin) * p.ld_qkv;
    auto conv1 = [&](int ch, const float* hist, float x) {
      const uint2 wv = *reinterpret_cast<const uint2*>(p.conv_w + static_cast<long long>(ch) * 4);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
      float a = __bfloat162float(wp[0].x) * hist[0];
      a += __bfloat162float(wp[0].y) * hist[1];
      a += __bfloat162float(wp[1].x) * hist[2];
      a += __bfloat162float(wp[1].y) * x;
      a = a / (1.f + __expf(-a));
      return __bfloat162float(__float2bfloat16(a));
    };
    const float xa = __bfloat162float(xrow[ch_a]);
    (threadIdx.x < 128 ? conv_q : conv_k)[ci] = conv1(ch_a, hist_a, xa);
    float xv = 0.f;
    if (threadIdx.x < 128) {
      xv = __bfloat162float(xrow[ch_v]);
      conv_v[ci] = conv1(ch_v, hist_v, xv);
    }
    if (ratio > 1) cluster_sync_all();   // every value head of this key head has read the shared q / k history
    else __syncthreads();
    if (hv % ratio == 0) {
      st_a[0] = __float2bfloat16(hist_a[1]);
      st_a[p.conv_C] = __float2bfloat16(hist_a[2]);
      st_a[2 * p.conv_C] = __float2bfloat16(xa);
    }
    if (threadIdx.x < 128) {
      st_v[0] = __float2bfloat16(hist_v[1]);
      st_v[p.conv_C] = __float2bfloat16(hist_v[2]);
      st_v[2 * p.conv_C] = __float2bfloat16(xv);
    }
  }

  for (int t = t_begin; t < t_end; ++t) {
    // ---- per-warp copy of the normalised q, k of this token ----
    const __nv_bfloat16* row = p.qkv + static_cast<long long>(t) * p.ld_qkv;
    float kf[4], qf[4];
    if (fused) {
      const float4 k4f = *reinterpret_cast<const float4*>(&conv_k[lane * 4]);
      const float4 q4f = *reinterpret_cast<const float4*>(&conv_q[lane * 4]);
      kf[0] = k4f.x; kf[1] = k4f.y; kf[2] = k4f.z; kf[3] = k4f.w;
      qf[0] = q4f.x; qf[1] = q4f.y; qf[2] = q4f.z; qf[3] = q4f.w;
    } else {
      const uint2 kr = *reinterpret_cast<const uint2*>(row + p.k_off + hk * kDk + lane * 4);
      const uint2 qr = *reinterpret_cast<const uint2*>(row + p.q_off + hk * kDk + lane * 4);
      const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kr);
      const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qr);
      kf[0] = __bfloat162float(kp[0].x); kf[1] = __bfloat162float(kp[0].y);
      kf[2] = __bfloat162float(kp[1].x); kf[3] = __bfloat162float(kp[1].y);
      qf[0] = __bfloat162float(qp[0].x); qf[1] = __bfloat162float(qp[0].y);
      qf[2] = __bfloat162float(qp[1].x); qf[3] = __bfloat162float(qp[1].y);
    }
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
      const float v = fused ? conv_v[r] : __bfloat162float(row[p.v_off + hv * kDv + r]);
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
    float yq = 0.f;
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
      yq = __bfloat162float(__float2bfloat16(y));
    }
    if (p.q_codes != nullptr) {
      // a warp owns sixteen consecutive outputs (rows warp * 16 ..): element e = 4 * q8 + sub sits in lane 8 * sub + q8
      float v[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) v[e] = __shfl_sync(0xffffffffu, yq, (e & 3) * 8 + (e >> 2));
      if (lane == 0) nvfp4_store_block(v, t, hv * (kDv / 16) + warp, p.n_v_heads * kDv, p.q_codes, p.q_sf);
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
  const int ratio = p.n_v_heads / p.n_qk_heads;
  if (p.conv_w != nullptr) {
    if (p.T != p.n_seq || p.seq_end != nullptr || p.commit != nullptr || !p.write_state)
      return "gdn_recurrent: the fused convolution is for plain decode steps (one token per sequence, state written)";
    if (p.conv_state == nullptr || p.conv_C <= 0 || ratio > 8) return "gdn_recurrent: bad fused-convolution arguments";
  } else if (p.T > p.n_seq && (p.v_off | p.z_off | p.ld_proj) % 4 == 0) {
    return gdn_prefill(p, stream, pdl);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_v_heads, p.n_seq); cfg.blockDim = dim3(kThreads); cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.conv_w != nullptr && ratio > 1) {   // the value heads of one key head share its q / k history: one cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = ratio;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr; cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gdn_recurrent_kernel, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
