// Depthwise causal conv1d (4 taps) + SiLU for the GDN q/k/v channels, ragged
// batches, with the per-sequence 3-column history.  One thread owns a channel
// pair of one token and gathers its four taps from the projection rows (or the
// history for taps that fall before the sequence's first token of this call).
//
// Reference: include/ninfer/ops/causal_conv1d_silu.h, src/ops/kernel/causal_conv1d.cuh
// (state = last 3 columns, oldest -> newest).
#include "gdn.h"

#include "../common/ptx.cuh"

namespace nfb {

namespace {

__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
  return make_float2(__bfloat162float(v.x), __bfloat162float(v.y));
}

// input of sequence `seq` at token index tau (global index), channel pair c.
__device__ __forceinline__ float2 tap(const ConvParams& p, int tau, int seq_start, int slot, int c) {
  if (tau >= seq_start) return ld2(p.x + static_cast<long long>(tau) * p.ld_x + p.c_off + c);
  const int j = tau - seq_start + 3;  // 0..2
  return ld2(p.conv_state + (static_cast<long long>(slot) * 3 + j) * p.C + c);
}

// Token index `back` steps before t: along the draft tree's parent links while inside the window, then into the
// history (indices below seq_start).
__device__ __forceinline__ int ancestor(const ConvParams& p, int t, int back, int seq_start) {
  int cur = t;
  for (int i = 0; i < back; ++i) {
    if (p.parent != nullptr && cur >= seq_start) {
      const int par = p.parent[cur];
      cur = par >= 0 ? par : seq_start - 1;
    } else {
      cur -= 1;
    }
  }
  return cur;
}

__global__ void __launch_bounds__(128) conv1d_silu_kernel(const ConvParams p) {
  pdl_launch_next();
  pdl_wait_prior();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  const int t = blockIdx.x;
  if (c >= p.C) return;
  const int seq = p.token_seq[t];
  if (seq < 0) return;
  const int start = p.cu_seqlens[seq];
  const int slot = p.state_slot[seq];
  const uint4 wv = *reinterpret_cast<const uint4*>(p.w + static_cast<long long>(c) * 4);  // 2 channels x 4 taps
  const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 x = tap(p, ancestor(p, t, 3 - j, start), start, slot, c);
    a0 += __bfloat162float(wp[j]) * x.x;
    a1 += __bfloat162float(wp[4 + j]) * x.y;
  }
  a0 = a0 / (1.f + __expf(-a0));
  a1 = a1 / (1.f + __expf(-a1));
  *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.C + c) = pack_bf16x2(a0, a1);
}

// Prefill variant: one thread owns 8 channels of a run of 16 consecutive tokens and slides the three previous
// inputs through registers, so every input row is read once (16-byte loads) instead of four times, and the grid is
// T / 16 x C / 1024 CTAs instead of T x C / 256.  Sequence boundaries inside a run reload the window from the new
// sequence's history.  (2048 tokens x 10240 channels: 97 us with the per-token kernel against 13 us of traffic.)
constexpr int kConvRun = 16;

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __bfloat162float(h[i].x);
    v[2 * i + 1] = __bfloat162float(h[i].y);
  }
}

__global__ void __launch_bounds__(128) conv1d_silu_rows_kernel(const ConvParams p) {
  pdl_launch_next();
  pdl_wait_prior();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= p.C) return;
  const int t0 = blockIdx.x * kConvRun, t1 = min(p.T, t0 + kConvRun);
  float w[8][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {   // 8 channels x 4 taps = 64 bytes
    float v[8];
    ld8(p.w + static_cast<long long>(c) * 4 + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) w[(i * 8 + j) >> 2][(i * 8 + j) & 3] = v[j];
  }
  float win[3][8];
  int seq = -2;
  for (int t = t0; t < t1; ++t) {
    const int s = p.token_seq[t];
    if (s < 0) {
      seq = -2;
      continue;
    }
    if (s != seq) {   // first token of this run, or a new sequence starts here
      seq = s;
      const int start = p.cu_seqlens[s];
      const int slot = p.state_slot[s];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int tau = t - 3 + j;
        if (tau >= start) ld8(p.x + static_cast<long long>(tau) * p.ld_x + p.c_off + c, win[j]);
        else ld8(p.conv_state + (static_cast<long long>(slot) * 3 + (tau - start + 3)) * p.C + c, win[j]);
      }
    }
    float cur[8];
    ld8(p.x + static_cast<long long>(t) * p.ld_x + p.c_off + c, cur);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int ch = 2 * i + h;
        const float v = w[ch][0] * win[0][ch] + w[ch][1] * win[1][ch] + w[ch][2] * win[2][ch] + w[ch][3] * cur[ch];
        a[h] = v / (1.f + __expf(-v));
      }
      o[i] = pack_bf16x2(a[0], a[1]);
    }
    *reinterpret_cast<uint4*>(p.out + static_cast<long long>(t) * p.C + c) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      win[0][ch] = win[1][ch];
      win[1][ch] = win[2][ch];
      win[2][ch] = cur[ch];
    }
  }
}

__global__ void __launch_bounds__(128) conv1d_state_kernel(const ConvParams p) {
  pdl_launch_next();
  pdl_wait_prior();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  const int seq = blockIdx.x;
  if (c >= p.C) return;
  const int start = p.cu_seqlens[seq], end = p.seq_end != nullptr ? p.seq_end[seq] : p.cu_seqlens[seq + 1];
  if (end <= start) return;
  const int slot = p.state_slot[seq];
  // the new history = the last three inputs along the (accepted) path that ends at `last`
  const int last = p.last_token != nullptr ? p.last_token[seq] : end - 1;
  float2 v[3];
#pragma unroll
  for (int j = 0; j < 3; ++j) v[j] = tap(p, ancestor(p, last, 2 - j, start), start, slot, c);
#pragma unroll
  for (int j = 0; j < 3; ++j)
    *reinterpret_cast<uint32_t*>(p.conv_state + (static_cast<long long>(slot) * 3 + j) * p.C + c) =
        pack_bf16x2(v[j].x, v[j].y);
}

// Decode fast path (exactly one token per sequence): conv, SiLU and the history roll in one
// launch.  The thread that owns (sequence, channel pair) is the only reader and writer of that
// history column, so there is no ordering problem.
__global__ void __launch_bounds__(128) conv1d_silu_decode_kernel(const ConvParams p) {
  pdl_launch_next();
  pdl_wait_prior();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  const int t = blockIdx.x;  // token index == sequence index
  if (c >= p.C) return;
  const int slot = p.state_slot[t];
  __nv_bfloat16* st = p.conv_state + static_cast<long long>(slot) * 3 * p.C + c;
  const uint4 wv = *reinterpret_cast<const uint4*>(p.w + static_cast<long long>(c) * 4);
  const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
  float2 x[4];
  x[0] = ld2(st);
  x[1] = ld2(st + p.C);
  x[2] = ld2(st + 2 * p.C);
  x[3] = ld2(p.x + static_cast<long long>(t) * p.ld_x + p.c_off + c);
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    a0 += __bfloat162float(wp[j]) * x[j].x;
    a1 += __bfloat162float(wp[4 + j]) * x[j].y;
  }
  a0 = a0 / (1.f + __expf(-a0));
  a1 = a1 / (1.f + __expf(-a1));
  *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t) * p.C + c) = pack_bf16x2(a0, a1);
#pragma unroll
  for (int j = 0; j < 3; ++j)
    *reinterpret_cast<uint32_t*>(st + j * p.C) = pack_bf16x2(x[j + 1].x, x[j + 1].y);
}

}  // namespace

const char* causal_conv1d_silu(const ConvParams& p, cudaStream_t stream, bool pdl) {
  if (p.T <= 0) return nullptr;
  if (p.C % 2 || p.c_off % 2 || p.ld_x % 2) return "causal_conv1d_silu: channel counts/offsets must be even";
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(128); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  cfg.gridDim = dim3(p.T, (p.C / 2 + 127) / 128);
  if (p.update_state && p.one_token_per_seq) {
    if (p.T != p.n_seq) return "causal_conv1d_silu: one_token_per_seq needs T == n_seq";
    cudaError_t e1 = cudaLaunchKernelEx(&cfg, conv1d_silu_decode_kernel, p);
    return e1 == cudaSuccess ? nullptr : cudaGetErrorString(e1);
  }
  cudaError_t e = cudaSuccess;
  const bool rows_ok = p.parent == nullptr && p.T >= 64 && p.C % 8 == 0 && p.c_off % 8 == 0 && p.ld_x % 8 == 0 &&
                       ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.out) |
                         reinterpret_cast<uintptr_t>(p.conv_state) | reinterpret_cast<uintptr_t>(p.w)) & 15) == 0;
  if (!p.state_only && rows_ok) {
    cfg.gridDim = dim3((p.T + kConvRun - 1) / kConvRun, (p.C / 8 + 127) / 128);
    e = cudaLaunchKernelEx(&cfg, conv1d_silu_rows_kernel, p);
    cfg.gridDim = dim3(p.T, (p.C / 2 + 127) / 128);
  } else if (!p.state_only) {
    e = cudaLaunchKernelEx(&cfg, conv1d_silu_kernel, p);
  }
  if (e != cudaSuccess) return cudaGetErrorString(e);
  if (p.update_state) {
    cfg.gridDim = dim3(p.n_seq, (p.C / 2 + 127) / 128);
    e = cudaLaunchKernelEx(&cfg, conv1d_state_kernel, p);
    if (e != cudaSuccess) return cudaGetErrorString(e);
  }
  return nullptr;
}

}  // namespace nfb
