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
  kEpiRsAg = 6,         // tensor parallel, decode sizes, two hops inside one kernel: every CTA whose column
                        // tile belongs to another rank stores its fp32 tile into that owner's receive buffer
                        // [src_rank][T_cap][N/world] as (value, epoch) pairs (the data says by itself when it is
                        // complete: no fence, no counter); the CTA that owns its tile polls the world-1 peer
                        // tiles until they carry this call's epoch, adds them and the residual, rounds to
                        // bf16, stores the new residual tile and the tile's per-token sums of squares into
                        // EVERY rank's residual buffer and bumps every rank's residual counter
                        // (GEMM -> reduce-scatter -> all-gather in one kernel).  The next column-parallel
                        // GEMM waits on that counter itself (GemmGather below).
};

// Rank-local bookkeeping of kEpiRsAg and of the gathered consumer (ordinary device memory, zero-initialised).
constexpr int kRsMaxTiles = 64;      // column tiles of 128 (N <= 8192)
constexpr int kRsMaxTokenTiles = 16;
constexpr int kRsSsStride = 64;      // column tiles per row of the sums-of-squares table (N <= 8192)
struct RsState {
  unsigned int tile_epoch[kRsMaxTiles * kRsMaxTokenTiles];  // finished calls per (column tile, token tile); every
                                                            // rank runs the same calls, so the words agree
  unsigned int x_expected;   // cumulative residual-tile arrivals the next consumer has to see
};

// A column-parallel GEMM that consumes the residual stream straight from the all-gather of kEpiRsAg: its TMA
// producer first streams weights into every pipeline stage, then waits until `*flag - *target >= 0` (all residual
// tiles of all owners have landed in this rank's buffer) and only then loads activations; the epilogue multiplies
// token t by rsqrt(sum_j ss[t][j] / n_features + eps), i.e. applies the RMS norm as a row scale (the norm's
// column weights must have been folded into the GEMM weight).
struct GemmGather {
  const unsigned int* flag = nullptr;    // this rank's residual arrival counter (symmetric buffer)
  const unsigned int* target = nullptr;  // RsState::x_expected
  const float* ss = nullptr;             // [T_cap][kRsSsStride] per-tile sums of squares (symmetric buffer)
  int ss_tiles = 0;                      // tiles per row that hold data (n_features / 128)
  int n_features = 0;
  float eps = 0.f;
};

enum GemmActivation : int { kActNone = 0, kActGeluTanh = 1, kActGeluErf = 2 };

constexpr int kMaxRanks = 8;

// kEpiStore at decode (token t is sequence t): output columns [0, C) are the inputs of a depthwise causal
// conv (4 taps) + SiLU with a 3-column history per sequence slot.  The epilogue thread that holds (token, channel)
// applies the taps, rolls the history forward and writes the activation to `out` [T, C]; columns >= C go to the
// GEMM's ordinary output.  Same arithmetic as the stand-alone decode kernel (gdn/conv1d.cu); C % 128 == 0.
struct GemmConv {
  const void* w = nullptr;      // bf16 [C, 4], tap 3 multiplies the newest input
  void* state = nullptr;        // bf16 [slots, 3, C], oldest -> newest
  const int* slot = nullptr;    // [T] history slot of each token's sequence
  void* out = nullptr;          // bf16 [T, C]
  int C = 0;
};

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
  // kEpiRsAg only (peer_recv then holds (fp32 bits, epoch) pairs, 8 bytes per value; peer_flag is unused):
  // every rank's residual buffer [T_cap][N] bf16, sums-of-squares table, residual counter; this
  // rank's bookkeeping; `rs_phase` 0 = fused (production), 1 = push tiles only (owned tiles are pushed to this
  // rank's own receive buffer too), 2 = no GEMM, owners reduce the `world` tiles that phase 1 left.  Phases 1 and
  // 2 exist so that several ranks can be walked through on ONE GPU without any kernel waiting on another.
  void* peer_x[kMaxRanks] = {};            // bf16 [T_cap][ldx_resid]
  int64_t ld_resid = 0;                    // leading dimension of the residual buffers (elements)
  float* peer_ss[kMaxRanks] = {};          // [T_cap][kRsSsStride]
  unsigned int* peer_xflag[kMaxRanks] = {};
  RsState* rs_state = nullptr;
  int rs_phase = 0;
  // kEpiStore / kEpiSwiglu: consume the gathered residual stream (see GemmGather); flag == nullptr = off
  GemmGather gather;
  GemmConv conv;   // kEpiStore only; state == nullptr = off
  // Optional: memory the NEXT kernel will stream (its weights).  Once a CTA has issued its own last load it asks
  // L2 to fetch its share of this range, so that HBM keeps working through this kernel's tail and epilogue and
  // the next kernel's pipeline fills from L2.  A hint only: nothing waits for it.
  const void* prefetch = nullptr;
  int64_t prefetch_bytes = 0;
};

// Returns nullptr on success, else a static error string.
const char* gemm_bf16(const GemmArgs& args);

// Token-tile width the kernel will use for T tokens (16, 32, 64, 128 or 256).
// Performance debugging: per-CTA phase timeline (ns, globaltimer): 0 start, 1 set-up done, 2 main loop done,
// 3 peer tile sent, 4 cluster exchange done, 5 epilogue done, 6 exit; kEpiRsAg also 7 tile pushed and signalled,
// 8 owner: tile staged and peers' tiles here, 9 rows reduced and stored, 10 barrier, 11 residual counters signalled.
// Twelve stamps per CTA.
void gemm_trace_enable(bool on);
int gemm_trace_read(unsigned long long* host, int n_ctas);
// Timeline over several launches: between begin and end, GEMM launch i records the stamps of its first 256 CTAs in
// slot i % 64 (a launch captured into a CUDA graph keeps its slot at every replay).  `end` copies
// [64][256][12] stamps (ns, globaltimer; 0 = not written) to `host` and returns the number of launches seen.
void gemm_timeline_begin();
int gemm_timeline_end(unsigned long long* host, int* n_slots, int* n_ctas);
int gemm_tile_tokens(int T);
int gemm_max_cluster(int tile_tokens);
// Split-K factor that fills `sm_count` SMs for a decode-shaped problem.
int gemm_pick_splits(int T, int N, int K, int epi, int sm_count);

}  // namespace nfb
