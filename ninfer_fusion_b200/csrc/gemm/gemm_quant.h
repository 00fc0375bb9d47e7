// Host entry points of the quantised-weight tcgen05 GEMMs and of the activation quantisers (plain C++ ABI).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm.h"

namespace nfb {

enum QuantType : int {
  kQFp8Row = 1,  // e4m3 codes, one fp32 scale per weight row / per token
  kQNvfp4 = 2,   // e2m1 codes, e4m3 scale per 16 values in 128x4 tiles, global divisor d_w
};

struct QGemmArgs {
  int qtype = kQFp8Row;
  const void* w = nullptr;        // fp8: [N, K] bytes; nvfp4: [N, K/2] bytes (low nibble = even k); leading dimension ldw bytes
  const void* w_scale = nullptr;  // fp8: float [N]; nvfp4: scale plane [ceil(N/128)][K/64][512] bytes
  float w_divisor = 1.f;          // nvfp4: d_w (W = e2m1 * e4m3 / d_w)
  const void* x = nullptr;        // quantised activations, same code format; leading dimension ldx bytes
  const void* x_scale = nullptr;  // fp8: float [T]; nvfp4: scale plane [ceil(T/256)*2][K/64][512] bytes
  int64_t N = 0, K = 0, T = 0, ldw = 0, ldx = 0;
  void* out = nullptr;            // bf16 [T, N] (SwiGLU: [T, N/2]; weight rows tile-interleaved [64 gate; 64 up])
  int64_t ldo = 0;
  const void* resid = nullptr;
  int64_t ldr = 0;
  int epi = kEpiStore;            // kEpiStore, kEpiResidual, kEpiSwiglu, kEpiPushAll or kEpiPushPartial
  // tensor-parallel epilogues (same protocol as the bf16 kernel, gemm.h)
  int world = 1, rank = 0, T_cap = 0;
  const unsigned int* call_idx = nullptr;
  float* peer_recv[kMaxRanks] = {};
  unsigned int* peer_flag[kMaxRanks] = {};
  int splits = 1;                 // in-cluster split-K
  // nvfp4 SwiGLU only: also write the activation [T, N/2] as the next GEMM's W4A4 operand (codes [T][N/4] bytes and
  // the scale plane of nvfp4_act_scale_bytes(T, N/2) bytes); nullptr = bf16 output only
  void* next_codes = nullptr;
  void* next_sf = nullptr;
  int* status = nullptr;
  cudaStream_t stream = nullptr;
  bool pdl = false;
};
const char* gemm_quant(const QGemmArgs& a);

// Bytes of the nvfp4 activation scale plane for T tokens of K values.
int64_t nvfp4_act_scale_bytes(int64_t T, int64_t K);

// Activation quantisers.  fp8: scale[t] = amax/448 (fp32), code = e4m3(x / scale).  nvfp4: per 16 values
// scale = e4m3(amax/6), code = e2m1(x / scale), scales written in the 128x4 tile order.
const char* quant_act_fp8(const __nv_bfloat16* x, int64_t ldx, int64_t T, int64_t K, uint8_t* codes, float* scale,
                          cudaStream_t stream, bool pdl = false);
const char* quant_act_nvfp4(const __nv_bfloat16* x, int64_t ldx, int64_t T, int64_t K, uint8_t* codes, uint8_t* sf_plane,
                            cudaStream_t stream, bool pdl = false);

}  // namespace nfb
