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
  float kdq[kTG];  // k . q of the normalised vectors (side-branch tokens)
  int cm[kTG];     // commit flag per token
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
      {
        // k . q over the token's 16 lanes (raw dot, scaled by both normalisers)
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d += kf[i] * qf[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (valid && part == 0) sm.kdq[tok] = d * rsqrtf(ssk + 1e-6f) * rsqrtf(ssq + 1e-6f) * qscale;
      }
      if (threadIdx.x < n_tok) {
        const __nv_bfloat16* prow = p.proj + static_cast<long long>(t0 + threadIdx.x) * p.ld_proj;
        const float a = __bfloat162float(prow[p.a_off + hv]);
        const float b = __bfloat162float(prow[p.b_off + hv]);
        const float x = a + dtb;
        const float sp_x = x > 20.f ? x : log1pf(__expf(x));
        sm.alpha[threadIdx.x] = __expf(neg_a * sp_x);
        sm.beta[threadIdx.x] = 1.f / (1.f + __expf(-b));
        sm.cm[threadIdx.x] = (p.commit == nullptr || p.commit[t0 + threadIdx.x] != 0) ? 1 : 0;
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
      const bool cm = sm.cm[tk] != 0;
      const float kqv = sm.kdq[tk];
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = warp * 16 + j * 4 + sub;
        const float v = __bfloat162float(sm.raw[buf][tk][2][r]);
        // four independent partial dot products (the state read is on the token-to-token critical path)
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
        } else {   // side branch: the state stays, o = alpha * (S q) + u * (k . q)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            oj += S[j][i].x * q4[i].x + S[j][i].y * q4[i].y + S[j][i].z * q4[i].z + S[j][i].w * q4[i].w;
          oj *= alpha;
        }
        oj += __shfl_xor_sync(0xffffffffu, oj, 1);
        oj += __shfl_xor_sync(0xffffffffu, oj, 2);
        oj += __shfl_xor_sync(0xffffffffu, oj, 4);
        if (!cm) oj += u * kqv;
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

// ---------------------------------------------------------------------------------------------------------
// Row-split variant for few sequences: the rows of the state evolve independently (row r only needs v_r), so a
// head's 128 rows are spread over a cluster of R = 128 / ROWS CTAs and the per-token critical path shrinks to one
// row per thread.  Only the gated RMSNorm couples the rows: per token group every CTA publishes its partial
// sums of squares in shared memory (double buffered by group parity) and reads its peers' through DSMEM after
// one cluster barrier.  The state is bit-identical to the unsplit kernel; the RMS sum is taken in CTA order.
// ---------------------------------------------------------------------------------------------------------
// Optional phase profile of the row-split kernel (performance debugging): clock cycles of CTA (0, 0) summed over
// its token groups: 0 wait for operands, 1 prologue, 2 serial steps, 3 partial sums + cluster barrier, 4 epilogue.
__device__ long long g_gdn_phase[8];
__device__ int g_gdn_trace_on;

constexpr int kTGS = 32;  // tokens per group of the row-split kernel (one cluster barrier per group)

template <int ROWS>
struct SplitSmem {
  __nv_bfloat16 kq[2][kTGS][2][kD];      // k, q rows of two groups
  __nv_bfloat16 vz[2][kTGS][2][ROWS];    // v, z of this CTA's rows
  float kn[kTGS][kD];
  float qn[kTGS][kD];
  float o[kTGS][ROWS];
  float alpha[kTGS], beta[kTGS];
  float kdq[kTGS];                       // k . q of the normalised vectors (side-branch tokens)
  int cm[kTGS];                          // commit flag per token
  float part[2][kTGS];                   // partial sum of squares per token, by group parity
};

template <int ROWS, int THREADS>
__global__ void __launch_bounds__(THREADS, 2) gdn_prefill_split_kernel(const GdnParams p) {
  constexpr int R = kD / ROWS;                 // CTAs per head
  constexpr int RPT = ROWS * 8 / THREADS;      // state rows per thread (8 lanes share a row)
  static_assert(RPT >= 1 && ROWS * 8 % THREADS == 0 && ROWS % 8 == 0, "bad row split");
  extern __shared__ __align__(16) uint8_t smem_raw[];
  SplitSmem<ROWS>& sm = *reinterpret_cast<SplitSmem<ROWS>*>(smem_raw);

  pdl_launch_next();
  pdl_wait_prior();
  const int hv = blockIdx.x / R, seq = blockIdx.y;
  uint32_t crank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  const int row0 = static_cast<int>(crank) * ROWS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, q8 = lane & 7;
  const int hk = hv / (p.n_v_heads / p.n_qk_heads);
  const int t_begin = p.cu_seqlens[seq], t_end = p.seq_end != nullptr ? p.seq_end[seq] : p.cu_seqlens[seq + 1];
  const int n_groups = t_end > t_begin ? (t_end - t_begin + kTGS - 1) / kTGS : 0;  // uniform over the cluster
  const int slot = p.state_slot[seq];

  // local row of (thread, j): warp * 4 * RPT + j * 4 + sub
  float* sbase = p.state + (static_cast<long long>(slot) * p.n_v_heads + hv) * kD * kD;
  float4 S[RPT][4];
  if (n_groups > 0) {
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int r = row0 + warp * 4 * RPT + j * 4 + sub;
#pragma unroll
      for (int i = 0; i < 4; ++i) S[j][i] = reinterpret_cast<const float4*>(sbase + r * kD)[q8 + 8 * i];
    }
  }
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const float qscale = rsqrtf(static_cast<float>(kD));

  auto prefetch = [&](int g) {
    const int buf = g & 1;
    const int t0 = t_begin + g * kTGS;
    // k, q: 16 tokens x 2 rows x 32 chunks of 8 bytes
    for (int c = threadIdx.x; c < kTGS * 2 * 32; c += THREADS) {
      const int tok = c >> 6, seg = (c >> 5) & 1, off = (c & 31) * 4;
      const int t = t0 + tok;
      if (t < t_end) {
        const __nv_bfloat16* src = p.qkv + static_cast<long long>(t) * p.ld_qkv + (seg == 0 ? p.k_off : p.q_off) + hk * kD + off;
        cp_async8(smem_u32(&sm.kq[buf][tok][seg][off]), src);
      }
    }
    // v, z: 16 tokens x 2 rows x ROWS / 4 chunks
    constexpr int kChunks = ROWS / 4;
    for (int c = threadIdx.x; c < kTGS * 2 * kChunks; c += THREADS) {
      const int tok = c / (2 * kChunks), seg = (c / kChunks) & 1, off = (c % kChunks) * 4;
      const int t = t0 + tok;
      if (t < t_end) {
        const __nv_bfloat16* src = seg == 0
            ? p.qkv + static_cast<long long>(t) * p.ld_qkv + p.v_off + hv * kD + row0 + off
            : p.proj + static_cast<long long>(t) * p.ld_proj + p.z_off + hv * kD + row0 + off;
        cp_async8(smem_u32(&sm.vz[buf][tok][seg][off]), src);
      }
    }
    cp_async_commit();
  };

  const bool tracer = g_gdn_trace_on != 0 && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
  long long ph[5] = {0, 0, 0, 0, 0};
  long long t_last = clock64();
  auto mark = [&](int i) {
    if (tracer) {
      const long long now = clock64();
      ph[i] += now - t_last;
      t_last = now;
    }
  };
  // gate inputs (a, b) of a group are fetched one group ahead into registers of threads 0..kTGS-1
  static_assert(THREADS >= kTGS, "one gate thread per token of a group");
  float ga = 0.f, gb = 0.f;
  auto load_gates = [&](int g) {
    const int t = t_begin + g * kTGS + static_cast<int>(threadIdx.x);
    if (threadIdx.x < kTGS && t < t_end) {
      const __nv_bfloat16* prow = p.proj + static_cast<long long>(t) * p.ld_proj;
      ga = __bfloat162float(prow[p.a_off + hv]);
      gb = __bfloat162float(prow[p.b_off + hv]);
    }
  };
  if (n_groups > 0) {
    prefetch(0);
    load_gates(0);
  }
  for (int g = 0; g < n_groups; ++g) {
    const int buf = g & 1;
    const int t0 = t_begin + g * kTGS;
    const int n_tok = min(kTGS, t_end - t0);
    __syncthreads();
    if (g + 1 < n_groups) {
      prefetch(g + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    mark(0);

    // ---- prologue: normalised q / k (16 lanes per token), gates ----
    for (int idx = threadIdx.x; idx < kTGS * 16; idx += THREADS) {
      const int tok = idx >> 4, part = idx & 15;
      const bool valid = tok < n_tok;
      float kf[8], qf[8], ssk = 0.f, ssq = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { kf[i] = 0.f; qf[i] = 0.f; }
      if (valid) {
        const uint4 kr = *reinterpret_cast<const uint4*>(&sm.kq[buf][tok][0][part * 8]);
        const uint4 qr = *reinterpret_cast<const uint4*>(&sm.kq[buf][tok][1][part * 8]);
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
      for (int o = 8; o > 0; o >>= 1) {
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
      {
        // k . q over the token's 16 lanes (raw dot, scaled by both normalisers)
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d += kf[i] * qf[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (valid && part == 0) sm.kdq[tok] = d * rsqrtf(ssk + 1e-6f) * rsqrtf(ssq + 1e-6f) * qscale;
      }
    }
    if (threadIdx.x < n_tok) {
      const float a = ga, b = gb;
      const float x = a + dtb;
      const float sp_x = x > 20.f ? x : log1pf(__expf(x));
      sm.alpha[threadIdx.x] = __expf(neg_a * sp_x);
      sm.beta[threadIdx.x] = 1.f / (1.f + __expf(-b));
      sm.cm[threadIdx.x] = (p.commit == nullptr || p.commit[t0 + threadIdx.x] != 0) ? 1 : 0;
    }
    if (g + 1 < n_groups) load_gates(g + 1);  // lands while the serial steps run
    __syncthreads();
    mark(1);

    // ---- serial delta-rule steps, software pipelined: the operands of token t + 1 are loaded while token t
    //      computes, and the output reduction of token t - 1 (off the critical path) is finished inside
    //      iteration t, so that only  dot(S, k) -> 3 shuffles -> u -> S update  separates two tokens ----
    {
      float4 k4[4], q4[4];
      float vv[RPT], alpha, beta;
      auto load_tok = [&](int tk, float4* kk, float4* qq, float* vr, float& al, float& be, float& kqo, int& cmo) {
        kqo = sm.kdq[tk];
        cmo = sm.cm[tk];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kk[i] = reinterpret_cast<const float4*>(sm.kn[tk])[q8 + 8 * i];
          qq[i] = reinterpret_cast<const float4*>(sm.qn[tk])[q8 + 8 * i];
        }
#pragma unroll
        for (int j = 0; j < RPT; ++j) vr[j] = __bfloat162float(sm.vz[buf][tk][0][warp * 4 * RPT + j * 4 + sub]);
        al = sm.alpha[tk];
        be = sm.beta[tk];
      };
      float kqv = 0.f;
      int cmv = 1;
      load_tok(0, k4, q4, vv, alpha, beta, kqv, cmv);
      float o_pend[RPT];
#pragma unroll
      for (int j = 0; j < RPT; ++j) o_pend[j] = 0.f;
      // one token: `c*` = operands of this token, `n*` = registers that receive the next token's operands
      auto step = [&](int tk, const float4* ck4, const float4* cq4, const float* cv, float calpha, float cbeta,
                      float ckq, int ccm, float4* nk4, float4* nq4, float* nv, float& nalpha, float& nbeta,
                      float& nkq, int& ncm) {
        const int tn = tk + 1 < n_tok ? tk + 1 : tk;
        load_tok(tn, nk4, nq4, nv, nalpha, nbeta, nkq, ncm);
        float ks[RPT];
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          // four independent partial dot products (the state read is on the token-to-token critical path)
          float kp4[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            kp4[i] = S[j][i].x * ck4[i].x + S[j][i].y * ck4[i].y + S[j][i].z * ck4[i].z + S[j][i].w * ck4[i].w;
          ks[j] = (kp4[0] + kp4[1]) + (kp4[2] + kp4[3]);
        }
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          ks[j] += __shfl_xor_sync(0xffffffffu, ks[j], 1);
          ks[j] += __shfl_xor_sync(0xffffffffu, ks[j], 2);
          ks[j] += __shfl_xor_sync(0xffffffffu, ks[j], 4);
        }
        // finish the previous token's output while the shuffles above are in flight
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          float oj = o_pend[j];
          oj += __shfl_xor_sync(0xffffffffu, oj, 1);
          oj += __shfl_xor_sync(0xffffffffu, oj, 2);
          oj += __shfl_xor_sync(0xffffffffu, oj, 4);
          if (q8 == 0 && tk > 0) sm.o[tk - 1][warp * 4 * RPT + j * 4 + sub] = __bfloat162float(__float2bfloat16(oj));
        }
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const float u = cbeta * (cv[j] - calpha * ks[j]);
          float oj = 0.f;
          if (ccm) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              S[j][i].x = calpha * S[j][i].x + u * ck4[i].x;
              S[j][i].y = calpha * S[j][i].y + u * ck4[i].y;
              S[j][i].z = calpha * S[j][i].z + u * ck4[i].z;
              S[j][i].w = calpha * S[j][i].w + u * ck4[i].w;
              oj += S[j][i].x * cq4[i].x + S[j][i].y * cq4[i].y + S[j][i].z * cq4[i].z + S[j][i].w * cq4[i].w;
            }
          } else {
            // side branch: o = alpha * (S q) + u * (k . q); the (k . q) term belongs to one lane of the row only,
            // because the eight lanes' partial sums are added up afterwards
#pragma unroll
            for (int i = 0; i < 4; ++i)
              oj += S[j][i].x * cq4[i].x + S[j][i].y * cq4[i].y + S[j][i].z * cq4[i].z + S[j][i].w * cq4[i].w;
            oj = calpha * oj + (q8 == 0 ? u * ckq : 0.f);
          }
          o_pend[j] = oj;
        }
      };
      // two tokens per trip with ping-pong operand registers (no register-to-register copies)
      float4 k4b[4], q4b[4];
      float vvb[RPT], alphab = 0.f, betab = 0.f, kqb = 0.f;
      int cmb = 1;
      for (int tk = 0; tk < n_tok; tk += 2) {
        step(tk, k4, q4, vv, alpha, beta, kqv, cmv, k4b, q4b, vvb, alphab, betab, kqb, cmb);
        if (tk + 1 < n_tok) step(tk + 1, k4b, q4b, vvb, alphab, betab, kqb, cmb, k4, q4, vv, alpha, beta, kqv, cmv);
      }
#pragma unroll
      for (int j = 0; j < RPT; ++j) {
        float oj = o_pend[j];
        oj += __shfl_xor_sync(0xffffffffu, oj, 1);
        oj += __shfl_xor_sync(0xffffffffu, oj, 2);
        oj += __shfl_xor_sync(0xffffffffu, oj, 4);
        if (q8 == 0) sm.o[n_tok - 1][warp * 4 * RPT + j * 4 + sub] = __bfloat162float(__float2bfloat16(oj));
      }
    }
    __syncthreads();
    mark(2);

    // ---- partial sums of squares of this CTA's rows, one warp-less pass: thread t < 16 sums token t ----
    for (int idx = threadIdx.x; idx < kTGS * 8; idx += THREADS) {  // 8 lanes per token
      const int tok = idx >> 3, l8 = idx & 7;
      float sq = 0.f;
      if (tok < n_tok) {
#pragma unroll
        for (int r = l8; r < ROWS; r += 8) sq += sm.o[tok][r] * sm.o[tok][r];
      }
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      if (l8 == 0) sm.part[g & 1][tok] = sq;
    }
    __syncthreads();
    // publish to the cluster (release) and wait for the peers (acquire)
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");

    mark(3);
    // ---- epilogue: gated RMSNorm, ROWS / 8 threads per token ----
    constexpr int kParts = ROWS / 8;
    for (int idx = threadIdx.x; idx < kTGS * kParts; idx += THREADS) {
      const int tok = idx / kParts, part = idx % kParts;
      if (tok >= n_tok) continue;
      float tot = 0.f;
      const uint32_t local = smem_u32(&sm.part[g & 1][tok]);
#pragma unroll
      for (uint32_t r = 0; r < static_cast<uint32_t>(R); ++r) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(r));
        float f;
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(f) : "r"(remote));
        tot += f;
      }
      const float inv = rsqrtf(tot / kD + p.eps);
      const uint4 zr = *reinterpret_cast<const uint4*>(&sm.vz[buf][tok][1][part * 8]);
      const uint4 wr = *reinterpret_cast<const uint4*>(p.norm_w + row0 + part * 8);
      const __nv_bfloat162* zp = reinterpret_cast<const __nv_bfloat162*>(&zr);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wr);
      uint4 outv;
      uint32_t* op = reinterpret_cast<uint32_t*>(&outv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float z0 = __bfloat162float(zp[i].x), z1 = __bfloat162float(zp[i].y);
        const float y0 = sm.o[tok][part * 8 + 2 * i] * inv * __bfloat162float(wp[i].x) * (z0 / (1.f + __expf(-z0)));
        const float y1 = sm.o[tok][part * 8 + 2 * i + 1] * inv * __bfloat162float(wp[i].y) * (z1 / (1.f + __expf(-z1)));
        op[i] = pack_bf16x2(y0, y1);
      }
      *reinterpret_cast<uint4*>(p.out + static_cast<long long>(t0 + tok) * (p.n_v_heads * kD) + hv * kD + row0 + part * 8) = outv;
    }
  }
  mark(4);
  if (tracer) {
    for (int i = 0; i < 5; ++i) g_gdn_phase[i] = ph[i];
  }
  // nobody leaves while a peer may still read its partial sums
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");

  if (p.write_state && n_groups > 0) {
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int r = row0 + warp * 4 * RPT + j * 4 + sub;
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(sbase + r * kD)[q8 + 8 * i] = S[j][i];
    }
  }
}

template <int ROWS, int THREADS>
cudaError_t launch_split(const GdnParams& p, cudaStream_t stream, bool pdl) {
  constexpr int R = kD / ROWS;
  auto kern = gdn_prefill_split_kernel<ROWS, THREADS>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(SplitSmem<ROWS>));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_v_heads * R, p.n_seq); cfg.blockDim = dim3(THREADS); cfg.stream = stream;
  cfg.dynamicSmemBytes = sizeof(SplitSmem<ROWS>);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = R; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

int sm_count_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

}  // namespace

void gdn_prefill_trace(bool enable, long long* host5) {
  const int on = enable ? 1 : 0;
  cudaMemcpyToSymbol(g_gdn_trace_on, &on, sizeof(int));
  if (host5 != nullptr) cudaMemcpyFromSymbol(host5, g_gdn_phase, 5 * sizeof(long long));
}

const char* gdn_prefill(const GdnParams& p, cudaStream_t stream, bool pdl) {
  if ((p.q_off | p.k_off | p.v_off | p.z_off) % 4 || p.ld_qkv % 4 || p.ld_proj % 4)
    return "gdn_prefill: row offsets and leading dimensions must be multiples of 4 elements";
  if ((reinterpret_cast<uintptr_t>(p.qkv) | reinterpret_cast<uintptr_t>(p.proj)) & 7)
    return "gdn_prefill: inputs must be 8-byte aligned";
  // few (head, sequence) pairs: spread each head's independent state rows over a cluster of CTAs
  {
    const int work = p.n_v_heads * p.n_seq;
    const int sms = sm_count_cached();
    cudaError_t e = cudaSuccess;
    bool done = true;
    // (measured on the 27B geometry, 2048 tokens of one sequence: 48 heads split 4 ways = 1.0 ms against 1.5 ms
    // unsplit; an 8-way split is faster in isolation (0.92 ms) but its 8-CTA clusters schedule worse between
    // the neighbouring GEMMs, so it is kept for shards with few heads only.  The loop is instruction-issue
    // bound: ~146 warp instructions per token and 4 rows.)
    if (work * 8 <= sms + sms / 2) e = launch_split<16, 128>(p, stream, pdl);
    else if (work * 4 <= sms + sms / 2) e = launch_split<32, 256>(p, stream, pdl);
    else if (work * 2 <= sms + sms / 2) e = launch_split<64, 256>(p, stream, pdl);
    else done = false;
    if (done) return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  }
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
