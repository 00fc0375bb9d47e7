// Chunked (WY) gated delta rule for prefill: the recurrence over 64-token chunks as tensor-core matrix products.
//
// Per value head, with the chunk's incoming state S0 [dv, dk], cumulative log decays G_i (inclusive) and
// L2-normalised q, k:
//
//   A_ij = beta_i (k_i . k_j) exp(G_i - G_j)  (j < i),   X = (I + A)^-1
//   W = X (beta exp(G) k),  U = X (beta v),  P_ij = (q_i . k_j) exp(G_i - G_j) / sqrt(dk)  (j <= i)
//   u~ = U - W S0^T                                   (the per-token delta-rule updates, all at once)
//   O  = exp(G) (q S0^T) / sqrt(dk) + P u~
//   S1 = exp(G_C) S0 + (exp(G_C - G) u~)^T k
//
// which is algebraically the token-by-token rule `S = a S; u = beta (v - S k); S += u (x) k; o = S q / sqrt(dk)`.
//
// Three launches:
//   gdn_chunk_prepare  one CTA per (chunk, value head), all chunks in parallel: K K^T and Q K^T on mma.sync,
//                      the triangular inverse by forward substitution in registers, W / U / P and the row scales
//                      into a workspace;
//   gdn_chunk_scan     one CTA per (sequence, value head, half of dv), sequential over the chunks: the state slice
//                      lives in MMA accumulator registers (fp32), the four products per chunk run on mma.sync
//                      out of a two-deep cp.async ring;
//   gdn_gated_norm     per (token, head) gated RMSNorm of the raw outputs in place.
//
// Operands of the products are bf16 (the inverse X as a hi + lo pair), accumulation and the state are fp32.
// mma.sync is used because the per-chunk products are 64 x 64 x 128 and run in a serial chain per head, where
// issue latency, not tensor throughput, sets the pace; a tcgen05 tile (M = 128) would be half empty.
//
// Reference: src/ops/linear_attention/gated_delta_net/chunked/{prepare_wy_wu,state_passing,output}.cuh
// (chunk 64, sub-block 16; same three-phase split).
#include "gdn.h"

#include <math_constants.h>

#include "../common/ptx.cuh"

namespace nfb {

namespace {

constexpr int kC = 64;          // tokens per chunk
constexpr int kD = 128;         // dk = dv
constexpr int kLdR = kD + 8;    // bf16 row pitch of [*, 128] tiles: 272 B, eight ldmatrix rows hit distinct banks
constexpr int kLdP = kC + 8;    // bf16 row pitch of [*, 64] tiles
constexpr int kLdA = kC + 4;    // fp32 row pitch of the A matrix (16-byte aligned rows)
constexpr int kLdU = kC + 4;    // fp32 row pitch of the U slice in the scan kernel

struct WsView {
  __nv_bfloat16* W;   // [chunks * Hv, 64, 128]
  float* U;           // [chunks * Hv, 64, 128]
  __nv_bfloat16* P;   // [chunks * Hv, 64, 64]
  float* vec;         // [chunks * Hv, 3, 64]: q row scale, k row scale, exp(G_C) (broadcast)
};

struct ChunkParams {
  GdnParams g;
  WsView ws;
  int max_chunks;
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Chunk `ci` of the step (chunks are numbered sequence by sequence): its sequence, first token and token count.
__device__ __forceinline__ bool find_chunk(const int* cu, int n_seq, int ci, int& seq, int& t0, int& n) {
  int base = 0;
  for (int s = 0; s < n_seq; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int nc = (max(e - b, 0) + kC - 1) / kC;
    if (ci < base + nc) {
      seq = s;
      t0 = b + (ci - base) * kC;
      n = min(kC, e - t0);
      return true;
    }
    base += nc;
  }
  return false;
}

// ------------------------------------------------------------------------------------------------ prepare
struct PrepSmem {
  __nv_bfloat16 k[kC][kLdR];    // raw k rows (zero past the chunk's end)
  __nv_bfloat16 q[kC][kLdR];
  __nv_bfloat16 v[kC][kLdR];    // raw v, scaled in place to beta v
  __nv_bfloat16 bk[kC][kLdR];   // beta exp(G) k / |k|
  float a[kC][kLdA];
  __nv_bfloat16 xh[kC][kLdP];
  __nv_bfloat16 xl[kC][kLdP];
  float g[kC], beta[kC], G[kC], rk[kC], rq[kC];
};

__global__ void __launch_bounds__(128) gdn_chunk_prepare_kernel(const ChunkParams cp) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  PrepSmem& sm = *reinterpret_cast<PrepSmem*>(smem_raw);
  const GdnParams& p = cp.g;
  int seq, t0, n_tok;
  if (!find_chunk(p.cu_seqlens, p.n_seq, blockIdx.x, seq, t0, n_tok)) return;
  const int hv = blockIdx.y;
  const int hk = hv / (p.n_v_heads / p.n_qk_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long item = static_cast<long long>(blockIdx.x) * p.n_v_heads + hv;

  // ---- raw rows by cp.async (zero-filled past the chunk), gates by the first 64 threads ----
  for (int i = tid; i < 3 * kC * (kD / 8); i += blockDim.x) {
    const int which = i / (kC * (kD / 8)), r = (i / (kD / 8)) % kC, c = i % (kD / 8);
    const bool ok = r < n_tok;
    const int off = which == 0 ? p.k_off + hk * kD : (which == 1 ? p.q_off + hk * kD : p.v_off + hv * kD);
    const __nv_bfloat16* src = p.qkv + static_cast<long long>(t0 + (ok ? r : 0)) * p.ld_qkv + off + c * 8;
    __nv_bfloat16(*dst)[kLdR] = which == 0 ? sm.k : (which == 1 ? sm.q : sm.v);
    cp_async_16(smem_u32(&dst[r][c * 8]), src, ok ? 16 : 0);
  }
  cp_async_commit();
  if (tid < kC) {
    float g = 0.f, beta = 0.f;
    if (tid < n_tok) {
      const __nv_bfloat16* prow = p.proj + static_cast<long long>(t0 + tid) * p.ld_proj;
      const float a = __bfloat162float(prow[p.a_off + hv]);
      const float b = __bfloat162float(prow[p.b_off + hv]);
      const float x = a + p.dt_bias[hv];
      const float sp = x > 20.f ? x : log1pf(__expf(x));
      g = -__expf(p.A_log[hv]) * sp;
      beta = 1.f / (1.f + __expf(-b));
    }
    sm.g[tid] = g;
    sm.beta[tid] = beta;
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- row norms (16 rows per warp), inclusive scan of the log decays (warp 0) ----
  for (int r = warp * 16; r < warp * 16 + 16; ++r) {
    float sk = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float kv = __bfloat162float(sm.k[r][lane * 4 + i]), qv = __bfloat162float(sm.q[r][lane * 4 + i]);
      sk += kv * kv;
      sq += qv * qv;
    }
    sk = warp_sum(sk);
    sq = warp_sum(sq);
    if (lane == 0) {
      sm.rk[r] = rsqrtf(sk + 1e-6f);
      sm.rq[r] = rsqrtf(sq + 1e-6f);
    }
  }
  if (warp == 0) {
    float a = sm.g[lane], b = sm.g[lane + 32];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) { a += ua; b += ub; }
    }
    const float total = __shfl_sync(0xffffffffu, a, 31);
    sm.G[lane] = a;
    sm.G[lane + 32] = b + total;
  }
  __syncthreads();

  // ---- K K^T and Q K^T for this warp's 16 rows; tiles above the diagonal are skipped ----
  const int row0 = lane >> 2, cq = lane & 3;
  {
    float kk[8][4], qk[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) { kk[n][j] = 0.f; qk[n][j] = 0.f; }
    const uint32_t ak_addr = smem_u32(&sm.k[warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
    const uint32_t aq_addr = smem_u32(&sm.q[warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      uint32_t a[4], b[4];
      ldsm_x4(ak_addr + ks * 32, a[0], a[1], a[2], a[3]);
      ldsm_x4(aq_addr + ks * 32, b[0], b[1], b[2], b[3]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        if (np <= warp) {
          uint32_t c0, c1, c2, c3;
          ldsm_x4(smem_u32(&sm.k[np * 16 + (lane & 7) + 8 * (lane >> 4)][ks * 16 + 8 * ((lane >> 3) & 1)]), c0, c1, c2, c3);
          mma_bf16(kk[2 * np], a[0], a[1], a[2], a[3], c0, c1);
          mma_bf16(kk[2 * np + 1], a[0], a[1], a[2], a[3], c2, c3);
          mma_bf16(qk[2 * np], b[0], b[1], b[2], b[3], c0, c1);
          mma_bf16(qk[2 * np + 1], b[0], b[1], b[2], b[3], c2, c3);
        }
      }
    }
    const float qscale = rsqrtf(static_cast<float>(kD));
    __nv_bfloat16* Pg = cp.ws.P + item * (kC * kC);
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = warp * 16 + row0 + 8 * h;
        const int j = n * 8 + 2 * cq;
        float av[2], pv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int jj = j + e;
          const float dec = jj <= i ? __expf(sm.G[i] - sm.G[jj]) : 0.f;
          const float rkj = sm.rk[jj];
          av[e] = jj < i ? sm.beta[i] * sm.rk[i] * rkj * kk[n][2 * h + e] * dec : 0.f;
          pv[e] = jj <= i ? sm.rq[i] * rkj * qk[n][2 * h + e] * dec * qscale : 0.f;
        }
        *reinterpret_cast<float2*>(&sm.a[i][j]) = make_float2(av[0], av[1]);
        *reinterpret_cast<uint32_t*>(Pg + i * kC + j) = pack_bf16x2(pv[0], pv[1]);
      }
  }
  __syncthreads();

  // ---- X = (I + A)^-1: thread c owns column c (forward substitution in registers); the other half of the CTA
  //      scales the right-hand sides meanwhile ----
  if (tid < kC) {
    const int c = tid;
    float x[kC];
#pragma unroll
    for (int i = 0; i < kC; ++i) {
      float acc[4] = {i == c ? 1.f : 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < i; ++j) acc[j & 3] -= sm.a[i][j] * x[j];
      x[i] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
#pragma unroll
    for (int i = 0; i < kC; ++i) {
      const __nv_bfloat16 hi = __float2bfloat16(x[i]);
      sm.xh[i][c] = hi;
      sm.xl[i][c] = __float2bfloat16(x[i] - __bfloat162float(hi));
    }
  } else {
    for (int i = tid - kC; i < kC * (kD / 2); i += blockDim.x - kC) {
      const int r = i / (kD / 2), c2 = (i % (kD / 2)) * 2;
      const float sk = sm.beta[r] * __expf(sm.G[r]) * sm.rk[r], sv = sm.beta[r];
      const __nv_bfloat162 kv = *reinterpret_cast<const __nv_bfloat162*>(&sm.k[r][c2]);
      const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(&sm.v[r][c2]);
      *reinterpret_cast<uint32_t*>(&sm.bk[r][c2]) = pack_bf16x2(__bfloat162float(kv.x) * sk, __bfloat162float(kv.y) * sk);
      *reinterpret_cast<uint32_t*>(&sm.v[r][c2]) = pack_bf16x2(__bfloat162float(vv.x) * sv, __bfloat162float(vv.y) * sv);
    }
  }
  __syncthreads();

  // ---- W = X (beta exp(G) k^), U = X (beta v); X is lower triangular, so k-steps past the diagonal are skipped ----
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    float acc[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[n][j] = 0.f;
    __nv_bfloat16(*rhs)[kLdR] = pass == 0 ? sm.bk : sm.v;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      if (kk <= warp) {
        uint32_t h[4], l[4];
        const int xr = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), xc = kk * 16 + 8 * (lane >> 4);
        ldsm_x4(smem_u32(&sm.xh[xr][xc]), h[0], h[1], h[2], h[3]);
        ldsm_x4(smem_u32(&sm.xl[xr][xc]), l[0], l[1], l[2], l[3]);
        const int br = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(smem_u32(&rhs[br][np * 16 + 8 * (lane >> 4)]), b0, b1, b2, b3);
          mma_bf16(acc[2 * np], h[0], h[1], h[2], h[3], b0, b1);
          mma_bf16(acc[2 * np + 1], h[0], h[1], h[2], h[3], b2, b3);
          mma_bf16(acc[2 * np], l[0], l[1], l[2], l[3], b0, b1);
          mma_bf16(acc[2 * np + 1], l[0], l[1], l[2], l[3], b2, b3);
        }
      }
    }
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = warp * 16 + row0 + 8 * h, j = n * 8 + 2 * cq;
        if (pass == 0)
          *reinterpret_cast<uint32_t*>(cp.ws.W + item * (kC * kD) + i * kD + j) = pack_bf16x2(acc[n][2 * h], acc[n][2 * h + 1]);
        else
          *reinterpret_cast<float2*>(cp.ws.U + item * (kC * kD) + i * kD + j) = make_float2(acc[n][2 * h], acc[n][2 * h + 1]);
      }
  }

  // ---- row scales for the scan ----
  if (tid < kC) {
    float* vec = cp.ws.vec + item * (3 * kC);
    const float Gc = sm.G[kC - 1];
    vec[tid] = __expf(sm.G[tid]) * sm.rq[tid] * rsqrtf(static_cast<float>(kD));
    vec[kC + tid] = sm.rk[tid] * __expf(Gc - sm.G[tid]);
    vec[2 * kC + tid] = __expf(Gc);
  }
}

// ------------------------------------------------------------------------------------------------ scan
constexpr int kScanThreads = 256;
constexpr int kHalf = kD / 2;   // dv columns per CTA

struct ScanStage {
  __nv_bfloat16 w[kC][kLdR];
  __nv_bfloat16 q[kC][kLdR];
  __nv_bfloat16 k[kC][kLdR];
  __nv_bfloat16 p[kC][kLdP];
  float u[kC][kLdU];
  float vec[3][kC];
};

struct ScanSmem {
  ScanStage st[2];
  __nv_bfloat16 sb[kHalf][kLdR];    // state slice as bf16, [dv][dk]
  __nv_bfloat16 vn[kC][kLdP];       // u~ (bf16)
  __nv_bfloat16 vnd[kC][kLdP];      // exp(G_C - G) / |k| scaled u~
};

__global__ void __launch_bounds__(kScanThreads, 1) gdn_chunk_scan_kernel(const ChunkParams cp) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  ScanSmem& sm = *reinterpret_cast<ScanSmem*>(smem_raw);
  const GdnParams& p = cp.g;
  const int hv = blockIdx.x, half = blockIdx.y, seq = blockIdx.z;
  const int hk = hv / (p.n_v_heads / p.n_qk_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = lane >> 2, cq = lane & 3;
  const int mt = warp & 3, nh = warp >> 2;   // products with 64 x 64 outputs: row tile, half of the columns

  const int seq_b = p.cu_seqlens[seq], seq_e = p.cu_seqlens[seq + 1];
  if (seq_e <= seq_b) return;
  const int n_chunks = (seq_e - seq_b + kC - 1) / kC;
  int chunk0 = 0;
  for (int s = 0; s < seq; ++s) chunk0 += (max(p.cu_seqlens[s + 1] - p.cu_seqlens[s], 0) + kC - 1) / kC;

  auto load_stage = [&](int c, int stg) {
    ScanStage& st = sm.st[stg];
    const int t0 = seq_b + c * kC;
    const int n_tok = min(kC, seq_e - t0);
    const long long item = static_cast<long long>(chunk0 + c) * p.n_v_heads + hv;
    const __nv_bfloat16* Wg = cp.ws.W + item * (kC * kD);
    const __nv_bfloat16* Pg = cp.ws.P + item * (kC * kC);
    const float* Ug = cp.ws.U + item * (kC * kD) + half * kHalf;
    const float* Vg = cp.ws.vec + item * (3 * kC);
    for (int i = tid; i < kC * (kD / 8); i += kScanThreads) {
      const int r = i / (kD / 8), c8 = (i % (kD / 8)) * 8;
      cp_async_16(smem_u32(&st.w[r][c8]), Wg + r * kD + c8, 16);
      const bool ok = r < n_tok;
      const __nv_bfloat16* row = p.qkv + static_cast<long long>(t0 + (ok ? r : 0)) * p.ld_qkv + hk * kD + c8;
      cp_async_16(smem_u32(&st.q[r][c8]), row + p.q_off, ok ? 16 : 0);
      cp_async_16(smem_u32(&st.k[r][c8]), row + p.k_off, ok ? 16 : 0);
      cp_async_16(smem_u32(&st.u[r][(i % (kD / 8)) * 4]), Ug + r * kD + (i % (kD / 8)) * 4, 16);
    }
    for (int i = tid; i < kC * (kC / 8); i += kScanThreads) {
      const int r = i / (kC / 8), c8 = (i % (kC / 8)) * 8;
      cp_async_16(smem_u32(&st.p[r][c8]), Pg + r * kC + c8, 16);
    }
    if (tid < 3 * kC / 4) cp_async_16(smem_u32(&st.vec[0][tid * 4]), Vg + tid * 4, 16);
  };

  load_stage(0, 0);
  cp_async_commit();

  // state slice S[dv 64*half .. +63][dk] in accumulator layout: warp w owns dk columns 16w..16w+15
  float* sbase = p.state + ((static_cast<long long>(p.state_slot[seq]) * p.n_v_heads + hv) * kD + half * kHalf) * kD;
  float S[4][2][4];
#pragma unroll
  for (int mi = 0; mi < 4; ++mi)
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int dv = mi * 16 + row0 + 8 * h, dk = warp * 16 + n * 8 + 2 * cq;
        const float2 v = *reinterpret_cast<const float2*>(sbase + dv * kD + dk);
        S[mi][n][2 * h] = v.x;
        S[mi][n][2 * h + 1] = v.y;
        *reinterpret_cast<uint32_t*>(&sm.sb[dv][dk]) = pack_bf16x2(v.x, v.y);
      }

  for (int c = 0; c < n_chunks; ++c) {
    const int stg = c & 1;
    ScanStage& st = sm.st[stg];
    if (c + 1 < n_chunks) {
      load_stage(c + 1, stg ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();   // this chunk's operands and the bf16 state are visible

    // ---- M1 = W S^T and O1 = Q S^T: rows 16 mt.., dv columns 32 nh.. ----
    float m1[4][4], o1[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) { m1[n][j] = 0.f; o1[n][j] = 0.f; }
    {
      const uint32_t aw = smem_u32(&st.w[mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
      const uint32_t aq = smem_u32(&st.q[mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
      const uint32_t bs = smem_u32(&sm.sb[nh * 32 + (lane & 7) + 8 * (lane >> 4)][8 * ((lane >> 3) & 1)]);
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        uint32_t a[4], b[4];
        ldsm_x4(aw + ks * 32, a[0], a[1], a[2], a[3]);
        ldsm_x4(aq + ks * 32, b[0], b[1], b[2], b[3]);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t c0, c1, c2, c3;
          ldsm_x4(bs + np * 16 * kLdR * 2 + ks * 32, c0, c1, c2, c3);
          mma_bf16(m1[2 * np], a[0], a[1], a[2], a[3], c0, c1);
          mma_bf16(m1[2 * np + 1], a[0], a[1], a[2], a[3], c2, c3);
          mma_bf16(o1[2 * np], b[0], b[1], b[2], b[3], c0, c1);
          mma_bf16(o1[2 * np + 1], b[0], b[1], b[2], b[3], c2, c3);
        }
      }
    }
    // ---- u~ = U - M1 (fp32), published as bf16 twice: plain and row-scaled for the state update ----
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = mt * 16 + row0 + 8 * h, col = nh * 32 + n * 8 + 2 * cq;
        const float2 u = *reinterpret_cast<const float2*>(&st.u[r][col]);
        const float v0 = u.x - m1[n][2 * h], v1 = u.y - m1[n][2 * h + 1];
        const float dk = st.vec[1][r], dq = st.vec[0][r];
        *reinterpret_cast<uint32_t*>(&sm.vn[r][col]) = pack_bf16x2(v0, v1);
        *reinterpret_cast<uint32_t*>(&sm.vnd[r][col]) = pack_bf16x2(v0 * dk, v1 * dk);
        o1[n][2 * h] *= dq;
        o1[n][2 * h + 1] *= dq;
      }
    __syncthreads();

    // ---- O = O1 + P u~ ----
    {
      const uint32_t ap = smem_u32(&st.p[mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
#pragma unroll
      for (int kk = 0; kk < kC / 16; ++kk) {
        uint32_t a[4];
        ldsm_x4(ap + kk * 32, a[0], a[1], a[2], a[3]);
        const int br = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t c0, c1, c2, c3;
          ldsm_x4_trans(smem_u32(&sm.vn[br][nh * 32 + np * 16 + 8 * (lane >> 4)]), c0, c1, c2, c3);
          mma_bf16(o1[2 * np], a[0], a[1], a[2], a[3], c0, c1);
          mma_bf16(o1[2 * np + 1], a[0], a[1], a[2], a[3], c2, c3);
        }
      }
      const int t0 = seq_b + c * kC;
      const int n_tok = min(kC, seq_e - t0);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = mt * 16 + row0 + 8 * h;
        if (r < n_tok) {
          __nv_bfloat16* dst = p.out + static_cast<long long>(t0 + r) * (p.n_v_heads * kD) + hv * kD + half * kHalf + nh * 32 + 2 * cq;
#pragma unroll
          for (int n = 0; n < 4; ++n)
            *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16x2(o1[n][2 * h], o1[n][2 * h + 1]);
        }
      }
    }

    // ---- S = exp(G_C) S + (scaled u~)^T K: all 64 dv rows, dk columns 16 warp.. ----
    {
      const float gamma = st.vec[2][0];
#pragma unroll
      for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int j = 0; j < 4; ++j) S[mi][n][j] *= gamma;
#pragma unroll
      for (int kk = 0; kk < kC / 16; ++kk) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(smem_u32(&st.k[kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][warp * 16 + 8 * (lane >> 4)]), b0, b1, b2, b3);
#pragma unroll
        for (int mi = 0; mi < 4; ++mi) {
          uint32_t a[4];
          ldsm_x4_trans(smem_u32(&sm.vnd[kk * 16 + (lane & 7) + 8 * (lane >> 4)][mi * 16 + 8 * ((lane >> 3) & 1)]),
                        a[0], a[1], a[2], a[3]);
          mma_bf16(S[mi][0], a[0], a[1], a[2], a[3], b0, b1);
          mma_bf16(S[mi][1], a[0], a[1], a[2], a[3], b2, b3);
        }
      }
    }
    __syncthreads();   // every warp is done with sb, vn / vnd and this stage
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int dv = mi * 16 + row0 + 8 * h, dk = warp * 16 + n * 8 + 2 * cq;
          *reinterpret_cast<uint32_t*>(&sm.sb[dv][dk]) = pack_bf16x2(S[mi][n][2 * h], S[mi][n][2 * h + 1]);
        }
  }

  if (p.write_state) {
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int dv = mi * 16 + row0 + 8 * h, dk = warp * 16 + n * 8 + 2 * cq;
          *reinterpret_cast<float2*>(sbase + dv * kD + dk) = make_float2(S[mi][n][2 * h], S[mi][n][2 * h + 1]);
        }
  }
}

// ------------------------------------------------------------------------------------------------ gated norm
// y = o * rsqrt(mean(o^2) + eps) * norm_w * silu(z), one warp per (token, head), in place on `out`.
__global__ void __launch_bounds__(256) gdn_gated_norm_kernel(const GdnParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long idx = static_cast<long long>(blockIdx.x) * 8 + warp;
  if (idx >= static_cast<long long>(p.T) * p.n_v_heads) return;
  const int t = static_cast<int>(idx / p.n_v_heads), hv = static_cast<int>(idx % p.n_v_heads);
  __nv_bfloat16* o = p.out + static_cast<long long>(t) * (p.n_v_heads * kD) + hv * kD + lane * 4;
  const __nv_bfloat16* z = p.proj + static_cast<long long>(t) * p.ld_proj + p.z_off + hv * kD + lane * 4;
  const uint2 ov = *reinterpret_cast<const uint2*>(o);
  const uint2 zv = *reinterpret_cast<const uint2*>(z);
  const uint2 wv = *reinterpret_cast<const uint2*>(p.norm_w + lane * 4);
  const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
  const __nv_bfloat162* z2 = reinterpret_cast<const __nv_bfloat162*>(&zv);
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
  float of[4], zf[4], wf[4], sq = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    of[2 * i] = __bfloat162float(o2[i].x); of[2 * i + 1] = __bfloat162float(o2[i].y);
    zf[2 * i] = __bfloat162float(z2[i].x); zf[2 * i + 1] = __bfloat162float(z2[i].y);
    wf[2 * i] = __bfloat162float(w2[i].x); wf[2 * i + 1] = __bfloat162float(w2[i].y);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) sq += of[i] * of[i];
  sq = warp_sum(sq);
  const float inv = rsqrtf(sq / kD + p.eps);
  float y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) y[i] = of[i] * inv * wf[i] * (zf[i] / (1.f + __expf(-zf[i])));
  uint2 out;
  out.x = pack_bf16x2(y[0], y[1]);
  out.y = pack_bf16x2(y[2], y[3]);
  *reinterpret_cast<uint2*>(o) = out;
}

}  // namespace

size_t gdn_chunked_workspace_bytes(int max_chunks, int n_v_heads) {
  const size_t items = static_cast<size_t>(max_chunks) * n_v_heads;
  return items * (kC * kD * 2 + kC * kD * 4 + kC * kC * 2 + 3 * kC * 4);
}

int gdn_chunked_max_chunks(int T, int n_seq) { return (T + kC - 1) / kC + n_seq; }

const char* gdn_chunked(const GdnParams& p, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (p.T <= 0 || p.n_seq <= 0) return nullptr;
  if (p.seq_end != nullptr || p.commit != nullptr) return "gdn_chunked: partial-sequence and tree passes use the recurrent kernels";
  if (p.n_v_heads % p.n_qk_heads) return "gdn_chunked: value heads must be a multiple of qk heads";
  if ((p.q_off | p.k_off | p.v_off | p.z_off) % 8 || p.ld_qkv % 8 || p.ld_proj % 4)
    return "gdn_chunked: row offsets and leading dimensions must be multiples of 8 elements";
  if ((reinterpret_cast<uintptr_t>(p.qkv) | reinterpret_cast<uintptr_t>(workspace)) & 15)
    return "gdn_chunked: inputs must be 16-byte aligned";
  if ((reinterpret_cast<uintptr_t>(p.proj) | reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.norm_w)) & 7)
    return "gdn_chunked: proj / out / norm_w must be 8-byte aligned";
  ChunkParams cp;
  cp.g = p;
  cp.max_chunks = gdn_chunked_max_chunks(p.T, p.n_seq);
  if (workspace_bytes < gdn_chunked_workspace_bytes(cp.max_chunks, p.n_v_heads)) return "gdn_chunked: workspace too small";
  const size_t items = static_cast<size_t>(cp.max_chunks) * p.n_v_heads;
  uint8_t* base = static_cast<uint8_t*>(workspace);
  cp.ws.U = reinterpret_cast<float*>(base);
  base += items * kC * kD * 4;
  cp.ws.W = reinterpret_cast<__nv_bfloat16*>(base);
  base += items * kC * kD * 2;
  cp.ws.P = reinterpret_cast<__nv_bfloat16*>(base);
  base += items * kC * kC * 2;
  cp.ws.vec = reinterpret_cast<float*>(base);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gdn_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(PrepSmem))) != cudaSuccess ||
        cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(ScanSmem))) != cudaSuccess)
      return "gdn_chunked: cannot raise the shared-memory limit";
    attr_set = true;
  }
  gdn_chunk_prepare_kernel<<<dim3(cp.max_chunks, p.n_v_heads), 128, sizeof(PrepSmem), stream>>>(cp);
  gdn_chunk_scan_kernel<<<dim3(p.n_v_heads, 2, p.n_seq), kScanThreads, sizeof(ScanSmem), stream>>>(cp);
  const long long warps = static_cast<long long>(p.T) * p.n_v_heads;
  gdn_gated_norm_kernel<<<static_cast<unsigned int>((warps + 7) / 8), 256, 0, stream>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
