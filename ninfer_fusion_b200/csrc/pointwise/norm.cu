// Row kernels on the residual stream: embedding gather, RMSNorm, fused
// residual-add + RMSNorm, and the split-K reduction that finishes a
// row-parallel GEMM (sum of fp32 partials + residual + next layer's RMSNorm in
// one pass over the row).  All are bandwidth-bound: one CTA per token row,
// 16-byte accesses, fp32 math, bf16 at the boundaries.
//
// Math contract (reference: include/ninfer/ops/rmsnorm.h, launcher/rmsnorm.cu):
//   y = x * rsqrt(mean(x^2) + eps) * (unit_offset ? 1 + w : w)
#include "pointwise.h"

#include "../gemm/gemm_quant.h"
#include "../kv/codec.cuh"

#include "../common/ptx.cuh"

namespace nfb {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// x row held in registers as up to kMaxVec 8-wide vectors per thread.
constexpr int kMaxVec = 4;  // 256 threads * 4 * 8 = 8192 columns max

template <bool kHasPartial>
__global__ void __launch_bounds__(kThreads) add_rmsnorm_kernel(
    const float* __restrict__ partial, int splits, long long split_stride,  // [splits][T][N] fp32
    const __nv_bfloat16* __restrict__ delta,                                // optional bf16 [T, N] to add
    const __nv_bfloat16* __restrict__ resid_in, __nv_bfloat16* __restrict__ resid_out,
    const __nv_bfloat16* __restrict__ norm_w, __nv_bfloat16* __restrict__ normed, int N, float eps,
    int unit_offset) {
  __shared__ float red[32];
  pdl_launch_next();
  pdl_wait_prior();
  const long long row = blockIdx.x;
  const int nvec = N / 8;
  float v[kMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      if (resid_in != nullptr) {
        const uint4 r = *reinterpret_cast<const uint4*>(resid_in + row * N + c * 8);
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] = __bfloat162float(rp[j].x);
          acc[2 * j + 1] = __bfloat162float(rp[j].y);
        }
      }
      if (delta != nullptr) {
        const uint4 r = *reinterpret_cast<const uint4*>(delta + row * N + c * 8);
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += __bfloat162float(rp[j].x);
          acc[2 * j + 1] += __bfloat162float(rp[j].y);
        }
      }
      if (kHasPartial) {
        for (int z = 0; z < splits; ++z) {
          const float4* pp = reinterpret_cast<const float4*>(partial + z * split_stride + row * N + c * 8);
          const float4 a = pp[0], b = pp[1];
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
          acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
      }
      // The residual stream is bf16: round first so the norm sees what is stored.
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        op[j] = pack_bf16x2(acc[2 * j], acc[2 * j + 1]);
        const __nv_bfloat162 b2 = *reinterpret_cast<__nv_bfloat162*>(&op[j]);
        v[i][2 * j] = __bfloat162float(b2.x);
        v[i][2 * j + 1] = __bfloat162float(b2.y);
        ss += v[i][2 * j] * v[i][2 * j] + v[i][2 * j + 1] * v[i][2 * j + 1];
      }
      if (resid_out != nullptr) *reinterpret_cast<uint4*>(resid_out + row * N + c * 8) = o;
    }
  }
  if (normed == nullptr) return;
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / static_cast<float>(N) + eps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) {
      const uint4 wv = *reinterpret_cast<const uint4*>(norm_w + c * 8);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float w0 = __bfloat162float(wp[j].x), w1 = __bfloat162float(wp[j].y);
        if (unit_offset) { w0 += 1.f; w1 += 1.f; }
        op[j] = pack_bf16x2(v[i][2 * j] * inv * w0, v[i][2 * j + 1] * inv * w1);
      }
      *reinterpret_cast<uint4*>(normed + row * N + c * 8) = o;
    }
  }
}

__global__ void __launch_bounds__(kThreads) embed_gather_kernel(const int* __restrict__ ids,
                                                                 const __nv_bfloat16* __restrict__ table,
                                                                 __nv_bfloat16* __restrict__ out, int N,
                                                                 int vocab) {
  pdl_launch_next();
  pdl_wait_prior();
  const long long row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<long long>(id) * N);
  uint4* dst = reinterpret_cast<uint4*>(out + row * N);
  for (int c = threadIdx.x; c < N / 8; c += kThreads) dst[c] = src[c];
}

// Generic strided per-head RMSNorm for small rows (head_dim 64..256): one warp per row.
__global__ void head_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long long row_stride,
                                    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                    long long out_stride, int rows, int D, float eps, int unit_offset) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * row_stride;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) { const float f = __bfloat162float(xr[d]); ss += f * f; }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / D + eps);
  for (int d = lane; d < D; d += 32) {
    float wd = __bfloat162float(w[d]);
    if (unit_offset) wd += 1.f;
    y[row * out_stride + d] = __float2bfloat16(__bfloat162float(xr[d]) * inv * wd);
  }
}

// Decode-sized variant (few rows): a thread-block cluster of kClusterRow CTAs shares one row, each
// CTA reduces and normalises N / kClusterRow columns and the row's sum of squares is combined
// through distributed shared memory.  32 rows then occupy 256 CTAs instead of 32.
constexpr int kClusterRow = 8;
constexpr int kClThreads = 128;

template <bool kHasPartial>
__global__ void __launch_bounds__(kClThreads) add_rmsnorm_cluster_kernel(
    const float* __restrict__ partial, int splits, long long split_stride,
    const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ resid_in,
    __nv_bfloat16* __restrict__ resid_out, const __nv_bfloat16* __restrict__ norm_w,
    __nv_bfloat16* __restrict__ normed, int N, float eps, int unit_offset, uint8_t* __restrict__ q_codes,
    uint8_t* __restrict__ q_sf) {
  __shared__ float red[kClThreads / 32];
  __shared__ float cta_ss;
  pdl_launch_next();
  pdl_wait_prior();
  const long long row = blockIdx.x / kClusterRow;
  uint32_t crank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  const int cols = N / kClusterRow;           // columns of this CTA
  const int c_begin = crank * cols;
  const int c = c_begin + threadIdx.x * 8;    // one 8-wide vector per thread (cols <= 1024)
  const bool active = threadIdx.x * 8 < cols;
  float v[8];
  float ss = 0.f;
  if (active) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (resid_in != nullptr) {
      const uint4 r = *reinterpret_cast<const uint4*>(resid_in + row * N + c);
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[2 * j] = __bfloat162float(rp[j].x); acc[2 * j + 1] = __bfloat162float(rp[j].y); }
    }
    if (delta != nullptr) {
      const uint4 r = *reinterpret_cast<const uint4*>(delta + row * N + c);
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[2 * j] += __bfloat162float(rp[j].x); acc[2 * j + 1] += __bfloat162float(rp[j].y); }
    }
    if (kHasPartial) {
#pragma unroll 8
      for (int z = 0; z < splits; ++z) {
        const float4* pp = reinterpret_cast<const float4*>(partial + z * split_stride + row * N + c);
        const float4 a = __ldcs(pp), b = __ldcs(pp + 1);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
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
    if (resid_out != nullptr) *reinterpret_cast<uint4*>(resid_out + row * N + c) = o;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kClThreads / 32; ++w) t += red[w];
    cta_ss = t;
  }
  // every CTA of the cluster publishes its partial sum, then reads all eight in rank order
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  float tot = 0.f;
  const uint32_t local = smem_u32(&cta_ss);
#pragma unroll
  for (uint32_t r = 0; r < kClusterRow; ++r) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(r));
    float f;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(f) : "r"(remote));
    tot += f;
  }
  // nobody may exit (and release its shared memory) before all peers have read it
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (normed == nullptr) return;
  const float inv = rsqrtf(tot / static_cast<float>(N) + eps);
  float nv[8];
  float amax = 0.f;
  if (active) {
    const uint4 wv = *reinterpret_cast<const uint4*>(norm_w + c);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float w0 = __bfloat162float(wp[j].x), w1 = __bfloat162float(wp[j].y);
      if (unit_offset) { w0 += 1.f; w1 += 1.f; }
      op[j] = pack_bf16x2(v[2 * j] * inv * w0, v[2 * j + 1] * inv * w1);
      const __nv_bfloat162 b2 = *reinterpret_cast<__nv_bfloat162*>(&op[j]);
      nv[2 * j] = __bfloat162float(b2.x);
      nv[2 * j + 1] = __bfloat162float(b2.y);
      amax = fmaxf(amax, fmaxf(fabsf(nv[2 * j]), fabsf(nv[2 * j + 1])));
    }
    *reinterpret_cast<uint4*>(normed + row * N + c) = o;
  }
  if (q_codes == nullptr) return;
  // nvfp4 copy of the normalised row for a block-scaled GEMM: two neighbouring threads share a 16-value block
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  if (!active) return;
  const uint8_t sc = float_to_e4m3(amax / 6.f);
  const float sf = e4m3_to_float(sc);
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) packed |= float_to_e2m1(sf > 0.f ? __fdiv_rn(nv[j], sf) : 0.f) << (4 * j);
  *reinterpret_cast<uint32_t*>(q_codes + row * (N / 2) + c / 2) = packed;
  if ((threadIdx.x & 1) == 0) {
    const int g = c / 16;
    const int t = static_cast<int>(row);
    q_sf[(static_cast<long long>(t / 128) * (N / 64) + g / 4) * 512 + (t % 32) * 16 + ((t % 128) / 32) * 4 + (g % 4)] = sc;
  }
}

template <typename K, typename... Args>
cudaError_t launch_cluster(K kern, dim3 grid, dim3 block, cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kClusterRow; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <typename K, typename... Args>
cudaError_t launch_pdl(K kern, dim3 grid, dim3 block, cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

const char* add_rmsnorm(const float* partial, int splits, const void* delta, const void* resid_in,
                        void* resid_out, const void* norm_w, void* normed, int T, int N, float eps,
                        int unit_offset, cudaStream_t stream, bool pdl, uint8_t* q_codes, uint8_t* q_sf) {
  if (T <= 0) return nullptr;
  if (q_codes != nullptr && (q_sf == nullptr || normed == nullptr || N % 64))
    return "add_rmsnorm: the nvfp4 copy needs the scale plane, the bf16 output and N % 64 == 0";
  if (N % 8 || N > kThreads * kMaxVec * 8) return "add_rmsnorm: N must be a multiple of 8 and <= 8192";
  if (normed != nullptr && norm_w == nullptr) return "add_rmsnorm: normed output without weight";
  cudaError_t e;
  const long long stride = static_cast<long long>(T) * N;
  auto* d = static_cast<const __nv_bfloat16*>(delta);
  auto* ri = static_cast<const __nv_bfloat16*>(resid_in);
  auto* ro = static_cast<__nv_bfloat16*>(resid_out);
  auto* w = static_cast<const __nv_bfloat16*>(norm_w);
  auto* no = static_cast<__nv_bfloat16*>(normed);
  if (T <= 128 && N % (16 * kClusterRow) == 0 && N / kClusterRow <= kClThreads * 8) {
    const dim3 grid(T * kClusterRow);
    if (partial != nullptr && splits > 0)
      e = launch_cluster(add_rmsnorm_cluster_kernel<true>, grid, dim3(kClThreads), stream, pdl, partial, splits,
                         stride, d, ri, ro, w, no, N, eps, unit_offset, q_codes, q_sf);
    else
      e = launch_cluster(add_rmsnorm_cluster_kernel<false>, grid, dim3(kClThreads), stream, pdl, partial, 0, stride,
                         d, ri, ro, w, no, N, eps, unit_offset, q_codes, q_sf);
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  }
  if (partial != nullptr && splits > 0)
    e = launch_pdl(add_rmsnorm_kernel<true>, dim3(T), dim3(kThreads), stream, pdl, partial, splits, stride,
                   d, ri, ro, w, no, N, eps, unit_offset);
  else
    e = launch_pdl(add_rmsnorm_kernel<false>, dim3(T), dim3(kThreads), stream, pdl, partial, 0, stride, d,
                   ri, ro, w, no, N, eps, unit_offset);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  if (q_codes != nullptr) return quant_act_nvfp4(no, N, T, N, q_codes, q_sf, stream, pdl);
  return nullptr;
}

const char* embed_gather(const int* ids, const void* table, void* out, int T, int N, int vocab,
                         cudaStream_t stream, bool pdl) {
  if (T <= 0) return nullptr;
  if (N % 8) return "embed_gather: N must be a multiple of 8";
  cudaError_t e = launch_pdl(embed_gather_kernel, dim3(T), dim3(kThreads), stream, pdl, ids,
                             static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), N,
                             vocab);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* head_rmsnorm(const void* x, long long row_stride, const void* w, void* y, long long out_stride,
                         int rows, int D, float eps, int unit_offset, cudaStream_t stream) {
  if (rows <= 0) return nullptr;
  const int warps = 4;
  head_rmsnorm_kernel<<<(rows + warps - 1) / warps, warps * 32, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), row_stride, static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(y), out_stride, rows, D, eps, unit_offset);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nfb
