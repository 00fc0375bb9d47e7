// Host entry points of the tcgen05 GEMM family (plain C++ ABI, no torch types).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfb {

enum GemmEpilogue : int {
  kEpiStore = 0,     // out = act(acc (+ bias[n]))
  kEpiResidual = 1,  // out = resid + acc (+ bias[n])
  kEpiSwiglu = 2,    // W = [gate; up] (N rows), out[T, N/2] = silu(gate) * up
  kEpiPartial = 3,   // partial[z, T, N] = acc over this split's K range (fp32)
  kEpiPushPartial = 4,  // tensor parallel: fp32 partial tiles are stored into the OWNER rank's receive
                        // buffer [src_rank][split][T][N/world] over NVLink, then the owner's arrival
                        // counter is incremented (GEMM -> reduce-scatter in one kernel)
  kEpiPushAll = 5,      // tensor parallel, decode sizes: the fp32 tile is stored into EVERY rank's receive
                        // buffer [parity][src_rank][T_cap][N] (one-shot all-reduce by push) and every
                        // rank's arrival counter is incremented (GEMM -> all-reduce in one kernel)
};

enum GemmActivation : int { kActNone = 0, kActGeluTanh = 1, kActGeluErf = 2 };

constexpr int kMaxRanks = 8;

struct GemmArgs {
  const void* w = nullptr;  // [N, K] bf16 row-major, leading dimension ldw
  int64_t N = 0, K = 0, ldw = 0;
  const void* x = nullptr;  // [T, K] bf16 row-major, leading dimension ldx
  int64_t T = 0, ldx = 0;
  void* out = nullptr;      // bf16 [T, N] (or [T, N/2] for SwiGLU), leading dimension ldo
  int64_t ldo = 0;
  const void* resid = nullptr;
  int64_t ldr = 0;
  const float* bias = nullptr;   // [N] fp32, added by kEpiStore and kEpiResidual
  int act = kActNone;            // kEpiStore: out = act(acc + bias)
  float* partial = nullptr;
  int splits = 1;
  int epi = kEpiStore;
  int* status = nullptr;    // device status word (see common/ptx.cuh)
  cudaStream_t stream = nullptr;
  bool pdl = false;         // launch with programmatic stream serialization
  // `splits` > 1 with kEpiStore / kEpiResidual / kEpiSwiglu / kEpiPushAll = in-cluster split-K: that many
  // CTAs (a power of two, see gemm_max_cluster) share one output tile and reduce through DSMEM.
  // kEpiPushPartial / kEpiPushAll only
  int world = 1, rank = 0;
  int T_cap = 0;                          // rows of the receive buffer (kEpiPushAll)
  const unsigned int* call_idx = nullptr; // device counter whose parity selects the receive buffer
  float* peer_recv[kMaxRanks] = {};
  unsigned int* peer_flag[kMaxRanks] = {};
};

// Returns nullptr on success, else a static error string.
const char* gemm_bf16(const GemmArgs& args);

// Token-tile width the kernel will use for T tokens (16, 32, 64, 128 or 256).
// Performance debugging: per-CTA phase timeline (ns, globaltimer): 0 start, 1 set-up done, 2 main loop done,
// 3 peer tile sent, 4 cluster exchange done, 5 epilogue done, 6 exit.
void gemm_trace_enable(bool on);
int gemm_trace_read(unsigned long long* host, int n_ctas);
int gemm_tile_tokens(int T);
int gemm_max_cluster(int tile_tokens);
// Split-K factor that fills `sm_count` SMs for a decode-shaped problem.
int gemm_pick_splits(int T, int N, int K, int epi, int sm_count);

}  // namespace nfb
