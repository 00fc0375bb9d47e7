// Gated delta-rule recurrence for multi-token sequences (prefill chunks, verify windows, replay of an
// accepted prefix).  Same math and the same register-resident fp32 state as the decode kernel
// (gdn_recurrent.cu), restructured so that the token loop touches no global memory and has no
// block-wide barrier:
//   * token groups of 16: the group's k / q / v / z rows are copied into shared memory by cp.async one
//     group ahead (double buffered);
//   * a short prologue L2-normalises the group's q, k and evaluates alpha = exp(-exp(A) softplus(a+dt)),
//     beta = sigmoid(b) once;
//   * the serial loop then runs 16 delta-rule steps out of shared memory (only 8-lane shuffles);
//   * an epilogue applies the per-head gated RMSNorm to the group's 16 x 128 outputs and stores them
//     with 16-byte writes.
// Reference: src/ops/linear_attention/gated_delta_net/{recurrent.cuh, chunked/*} (the reference switches to
// a chunked WY formulation for full 64-token chunks; this kernel keeps the exact sequential recurrence,
// so prefill, decode and replay stay bit-consistent with one another).
#include "gdn.h"

#include "../common/ptx.cuh"

namespace nfb {

namespace {

constexpr int kD = 128;
constexpr int kThreads = 256;
constexpr int kTG = 16;  // tokens per group

struct PrefillSmem {
  __nv_bfloat16 raw[2][kTG][4][kD];  // k, q, v, z rows of two groups
  float kn[kTG][kD];
  float qn[kTG][kD];
  float o[kTG][kD];
  float alpha[kTG], beta[kTG];
};

__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(kThreads, 1) gdn_prefill_kernel(const GdnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(smem_raw);

  pdl_launch_next();
  pdl_wait_prior();
  const int hv = blockIdx.x, seq = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, q8 = lane & 7;
  const int hk = hv / (p.n_v_heads / p.n_qk_heads);
  const int t_begin = p.cu_seqlens[seq], t_end = p.seq_end != nullptr ? p.seq_end[seq] : p.cu_seqlens[seq + 1];
  if (t_end <= t_begin) return;
  const int slot = p.state_slot[seq];
  const int n_groups = (t_end - t_begin + kTG - 1) / kTG;

  float* sbase = p.state + (static_cast<long long>(slot) * p.n_v_heads + hv) * kD * kD;
  float4 S[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = warp * 16 + j * 4 + sub;
#pragma unroll
    for (int i = 0; i < 4; ++i) S[j][i] = reinterpret_cast<const float4*>(sbase + r * kD)[q8 + 8 * i];
  }
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const float qscale = rsqrtf(static_cast<float>(kD));

  // one group = 16 tokens x 4 rows x 256 bytes = 2048 chunks of 8 bytes, 8 per thread
  auto prefetch = [&](int g) {
    const int buf = g & 1;
    const int t0 = t_begin + g * kTG;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int c = it * kThreads + threadIdx.x;
      const int tok = c >> 7, seg = (c >> 5) & 3, off = (c & 31) * 4;  // 4 bf16 per chunk
      const int t = t0 + tok;
      if (t < t_end) {
        const __nv_bfloat16* src;
        if (seg == 0) src = p.qkv + static_cast<long long>(t) * p.ld_qkv + p.k_off + hk * kD + off;
        else if (seg == 1) src = p.qkv + static_cast<long long>(t) * p.ld_qkv + p.q_off + hk * kD + off;
        else if (seg == 2) src = p.qkv + static_cast<long long>(t) * p.ld_qkv + p.v_off + hv * kD + off;
        else src = p.proj + static_cast<long long>(t) * p.ld_proj + p.z_off + hv * kD + off;
        cp_async8(smem_u32(&sm.raw[buf][tok][seg][off]), src);
      }
    }
    cp_async_commit();
  };

  prefetch(0);
  for (int g = 0; g < n_groups; ++g) {
    const int buf = g & 1;
    const int t0 = t_begin + g * kTG;
    const int n_tok = min(kTG, t_end - t0);
    __syncthreads();  // everybody is done with the previous group (its buffers may be refilled)
    if (g + 1 < n_groups) {
      prefetch(g + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    // ---- prologue: normalised q / k (16 threads per token), gates (one thread per token) ----
    {
      const int tok = threadIdx.x >> 4, part = threadIdx.x & 15;
      const bool valid = tok < n_tok;
      float kf[8], qf[8], ssk = 0.f, ssq = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { kf[i] = 0.f; qf[i] = 0.f; }
      if (valid) {
        const uint4 kr = *reinterpret_cast<const uint4*>(&sm.raw[buf][tok][0][part * 8]);
        const uint4 qr = *reinterpret_cast<const uint4*>(&sm.raw[buf][tok][1][part * 8]);
        const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kr);
        const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qr);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kf[2 * i] = __bfloat162float(kp[i].x); kf[2 * i + 1] = __bfloat162float(kp[i].y);
          qf[2 * i] = __bfloat162float(qp[i].x); qf[2 * i + 1] = __bfloat162float(qp[i].y);
          ssk += kf[2 * i] * kf[2 * i] + kf[2 * i + 1] * kf[2 * i + 1];
          ssq += qf[2 * i] * qf[2 * i] + qf[2 * i + 1] * qf[2 * i + 1];
        }
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {  // the 16 lanes of one token live in one half-warp
        ssk += __shfl_xor_sync(0xffffffffu, ssk, o);
        ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      }
      if (valid) {
        const float ik = rsqrtf(ssk + 1e-6f), iq = rsqrtf(ssq + 1e-6f) * qscale;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          sm.kn[tok][part * 8 + i] = kf[i] * ik;
          sm.qn[tok][part * 8 + i] = qf[i] * iq;
        }
      }
      if (threadIdx.x < n_tok) {
        const __nv_bfloat16* prow = p.proj + static_cast<long long>(t0 + threadIdx.x) * p.ld_proj;
        const float a = __bfloat162float(prow[p.a_off + hv]);
        const float b = __bfloat162float(prow[p.b_off + hv]);
        const float x = a + dtb;
        const float sp_x = x > 20.f ? x : log1pf(__expf(x));
        sm.alpha[threadIdx.x] = __expf(neg_a * sp_x);
        sm.beta[threadIdx.x] = 1.f / (1.f + __expf(-b));
      }
    }
    __syncthreads();

    // ---- serial delta-rule steps, everything out of shared memory ----
    for (int tk = 0; tk < n_tok; ++tk) {
      float4 k4[4], q4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        k4[i] = reinterpret_cast<const float4*>(sm.kn[tk])[q8 + 8 * i];
        q4[i] = reinterpret_cast<const float4*>(sm.qn[tk])[q8 + 8 * i];
      }
      const float alpha = sm.alpha[tk], beta = sm.beta[tk];
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = warp * 16 + j * 4 + sub;
        const float v = __bfloat162float(sm.raw[buf][tk][2][r]);
        float ks = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          ks += S[j][i].x * k4[i].x + S[j][i].y * k4[i].y + S[j][i].z * k4[i].z + S[j][i].w * k4[i].w;
        ks += __shfl_xor_sync(0xffffffffu, ks, 1);
        ks += __shfl_xor_sync(0xffffffffu, ks, 2);
        ks += __shfl_xor_sync(0xffffffffu, ks, 4);
        const float u = beta * (v - alpha * ks);
        float oj = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          S[j][i].x = alpha * S[j][i].x + u * k4[i].x;
          S[j][i].y = alpha * S[j][i].y + u * k4[i].y;
          S[j][i].z = alpha * S[j][i].z + u * k4[i].z;
          S[j][i].w = alpha * S[j][i].w + u * k4[i].w;
          oj += S[j][i].x * q4[i].x + S[j][i].y * q4[i].y + S[j][i].z * q4[i].z + S[j][i].w * q4[i].w;
        }
        oj += __shfl_xor_sync(0xffffffffu, oj, 1);
        oj += __shfl_xor_sync(0xffffffffu, oj, 2);
        oj += __shfl_xor_sync(0xffffffffu, oj, 4);
        o[j] = oj;
      }
      if (q8 < 4) {
        float oj = o[0];
#pragma unroll
        for (int j = 1; j < 4; ++j) oj = (q8 == j) ? o[j] : oj;
        sm.o[tk][warp * 16 + q8 * 4 + sub] = __bfloat162float(__float2bfloat16(oj));  // bf16 boundary
      }
    }
    __syncthreads();

    // ---- epilogue: gated RMSNorm of the group's outputs, 16 threads per token ----
    {
      const int tok = threadIdx.x >> 4, part = threadIdx.x & 15;
      float ov[8], sq = 0.f;
      if (tok < n_tok) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { ov[i] = sm.o[tok][part * 8 + i]; sq += ov[i] * ov[i]; }
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (tok < n_tok) {
        const float inv = rsqrtf(sq / kD + p.eps);
        const uint4 zr = *reinterpret_cast<const uint4*>(&sm.raw[buf][tok][3][part * 8]);
        const uint4 wr = *reinterpret_cast<const uint4*>(p.norm_w + part * 8);
        const __nv_bfloat162* zp = reinterpret_cast<const __nv_bfloat162*>(&zr);
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wr);
        uint4 outv;
        uint32_t* op = reinterpret_cast<uint32_t*>(&outv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float z0 = __bfloat162float(zp[i].x), z1 = __bfloat162float(zp[i].y);
          const float y0 = ov[2 * i] * inv * __bfloat162float(wp[i].x) * (z0 / (1.f + __expf(-z0)));
          const float y1 = ov[2 * i + 1] * inv * __bfloat162float(wp[i].y) * (z1 / (1.f + __expf(-z1)));
          op[i] = pack_bf16x2(y0, y1);
        }
        *reinterpret_cast<uint4*>(p.out + static_cast<long long>(t0 + tok) * (p.n_v_heads * kD) + hv * kD + part * 8) = outv;
      }
    }
  }

  if (p.write_state) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = warp * 16 + j * 4 + sub;
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(sbase + r * kD)[q8 + 8 * i] = S[j][i];
    }
  }
}

}  // namespace

const char* gdn_prefill(const GdnParams& p, cudaStream_t stream, bool pdl) {
  if ((p.q_off | p.k_off | p.v_off | p.z_off) % 4 || p.ld_qkv % 4 || p.ld_proj % 4)
    return "gdn_prefill: row offsets and leading dimensions must be multiples of 4 elements";
  if ((reinterpret_cast<uintptr_t>(p.qkv) | reinterpret_cast<uintptr_t>(p.proj)) & 7)
    return "gdn_prefill: inputs must be 8-byte aligned";
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gdn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         sizeof(PrefillSmem));
    if (e != cudaSuccess) return cudaGetErrorString(e);
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_v_heads, p.n_seq); cfg.blockDim = dim3(kThreads); cfg.stream = stream;
  cfg.dynamicSmemBytes = sizeof(PrefillSmem);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gdn_prefill_kernel, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
