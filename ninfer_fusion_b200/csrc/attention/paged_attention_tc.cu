// Split-KV paged decode / verify attention on the 5th-generation tensor cores, fp8-row KV pages, head_dim 256.
//
// The e4m3 codes of the cache are the MMA operands as they lie in the pages: no dequantisation, no register
// staging.  A persistent CTA (one per SM) takes an equal share of the 128-key tiles of all (query token, kv head)
// rows -- rows are cut where CTA boundaries fall, each piece fills one partial-result slot of its row -- and runs
// the whole problem TRANSPOSED, so that the 128 MMA rows are keys instead of the handful of query rows of a GQA
// group:
//
//   S^T[128 keys, 16 rows]  = K_tile[128 keys, 256 d]   . Q^T          kind::f8f6f4, K-major A from TMA, 16 k-steps
//   O^T[256 d, 16 rows]    += V_tile^T[256 d, 128 keys] . P^T          V as it lies in the page = MN-major A operand
//
// * K and V tiles come through TMA as boxes of [64 keys][128 bytes] with the 128-byte swizzle: the same bytes are
//   a K-major operand (rows = keys, contraction over d) for the first product and an MN-major operand (rows = keys
//   = contraction) for the second, so V needs no transpose pass.  Three 64 KB stages per CTA keep ~190 KB of loads
//   in flight per SM; the producer runs ahead across item boundaries, so there is no drain between items.
// * Row scales never touch the operands: the K scale multiplies a key's row of S^T (one scalar per thread, the
//   thread owns a key), the V scale multiplies the key's probabilities before they are quantised.
// * Q and P are not fp8 in the model.  Each is split into two e4m3 terms (x ~ hi + lo, ~2^-8 relative).  Q: both
//   terms go into the same accumulator.  P: p' = p * v_scale / V-scale frame; hi = e4m3(p') accumulates into
//   O_hi, lo = e4m3(128 * (p' - hi)) into O_lo, and the result is O_hi + O_lo / 128 -- the second accumulator extends
//   the smallest representable probability to ~2^-17 of the frame, so a long tail of small weights is not dropped.
// * Frames instead of running maxima: the softmax frame m and the V-scale frame R of a row are only moved when a
//   tile's maximum exceeds them by more than 2^4 (scores) or 2 (scales), so p <= 16 and p' <= 32 always fit e4m3.
//   Moving a frame rescales the O^T columns in TMEM (tcgen05.ld / tcgen05.st) and needs the previous product to be
//   complete; with lazy frames that happens in the first tile or two of an item, and every other tile's softmax
//   overlaps the previous tile's P.V.
// * S^T (2 buffers x 4 partial accumulators x 16 columns), O_hi and O_lo (2 x 16 columns each) live in TMEM.  The
//   N = 16 instructions are latency bound, so no two consecutive ones share an accumulator: S^T is summed from four
//   partials by the softmax threads, and P.V walks its four accumulators inside every key step.
// * Warps: 0-7 softmax (two threads per key = TMEM lane, each with half of the query rows: one warp per scheduler
//   could not hide its own latencies), 8 TMA producer, 9 issuer of S^T + TMEM owner, 10 query staging (bf16 -> two
//   swizzled e4m3 operand tiles, one item ahead), 11 issuer of P.V.
//
// Every wait is bounded; after a time-out the roles run their loops to the end without blocking, the status word
// says what gave up, and the CTA frees its TMEM.  Unwritten rows of a tile (pages past the sequence end) keep
// whatever cache rows the stage held before; their probabilities are exactly zero, and the V halves of the stages
// are zero-filled once at kernel start so that the first use cannot multiply a zero by a NaN pattern.  (The cache
// planes themselves are zero-initialised and the quantiser saturates, so a page never holds NaN codes.)
//
// Function of the reference's fp8 decode kernel (src/ops/kernel/gqa_attention_decode_fp8.cuh) with the split /
// merge contract of this repository (partials (m, l, o) per split, merged by paged_attn_merge_kernel).
#include <cuda_fp8.h>
#include <math_constants.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "attention.h"

namespace nfb {

namespace {

constexpr int D = 256;
constexpr int kTileKeys = 128;
constexpr int kBoxKeys = 64;
constexpr int kBoxBytes = kBoxKeys * 128;        // one TMA box: [64 keys][128 B]
constexpr int kHalfBytes = kTileKeys * 128;      // one d-half of a tile: [128 keys][128 B], two boxes
constexpr int kOperandBytes = 2 * kHalfBytes;    // K (or V) of one tile
constexpr int kStageBytes = 2 * kOperandBytes;   // 64 KB
constexpr int kStages = 3;
constexpr int kRows = 16;                        // MMA N: query rows of the group, zero padded
constexpr int kQPartBytes = 2 * kRows * 128;     // one e4m3 term of Q: two d-halves of [16 rows][128 B]
constexpr int kQBytes = 2 * kQPartBytes;         // hi + lo
constexpr int kPPartBytes = kTileKeys * kRows;   // one e4m3 term of P^T: [128 keys][16 rows]
constexpr int kPBytes = 2 * kPPartBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kQBytes + 2 * kPBytes + 1024;
constexpr int kSoftmaxWarps = 8;     // two threads per key: each owns half of the group's query rows
constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
constexpr int kWarpProducer = 8, kWarpS = 9, kWarpQ = 10, kWarpPV = 11;
constexpr int kThreads = 12 * 32;
constexpr int kTmemCols = 256;                   // S^T: 2 buffers x 4 partials x 16, O_hi and O_lo: 2 x 16 each
constexpr float kPScale = 1.f;      // p' = kPScale * p * v_scale / R <= 16 * 2
constexpr float kLoScale = 128.f;   // second term of P: 128 x the residual (<= half an e4m3 step of 32, i.e. <= 128)
constexpr float kFrameSlack = 4.f;  // log2 units a score may exceed its row's frame before the frame moves
constexpr int kMaxItems = 256;      // items one CTA may walk (their descriptors live in shared memory)
constexpr int kMaxBoxes = 512;      // 64-key boxes of those items (cache rows looked up once, in the prologue)
constexpr int kColO = 8 * kRows;    // first O^T column: [hi d0-127][hi d128-255][lo d0-127][lo d128-255]

enum : int { kStatusAttnWait = 6 };

// Optional event trace of CTA 0 (development aid): five roles x 1024 (code << 56 | globaltimer ns) entries.
constexpr int kTraceRoles = 5, kTraceLen = 1024;
__device__ unsigned long long g_attn_trace[kTraceRoles * kTraceLen];
bool g_attn_trace_on = false;
__device__ __forceinline__ void trace_event(int on, int role, int& n, int code) {
  if (on && blockIdx.x == 0 && n < kTraceLen) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_attn_trace[role * kTraceLen + n++] = (static_cast<unsigned long long>(code) << 56) | (t & 0x00ffffffffffffffull);
  }
}

struct TcParams {
  PagedAttnParams a;
  int G;
  int* status;
  int trace;
};

// A piece of work: tiles [k0, k_end) of one (query token, kv head) row, visible keys [k_begin, k_end), partial result
// slot `split` of that row.  Pieces are cut by the prologue so that every CTA gets the same number of 128-key tiles.
struct Item {
  int t, kvh, split, k_begin, k_end, k0, nt, box0;
};
struct ItemRec {
  int t, kvh_split, k_begin, k_end, k0, box0;
};
__device__ __forceinline__ Item get_item(const ItemRec* recs, int i) {
  const ItemRec r = recs[i];
  Item it;
  it.t = r.t;
  it.kvh = r.kvh_split >> 16;
  it.split = r.kvh_split & 0xffff;
  it.k_begin = r.k_begin;
  it.k_end = r.k_end;
  it.k0 = r.k0;
  it.nt = (r.k_end - r.k0 + kTileKeys - 1) / kTileKeys;
  it.box0 = r.box0;
  return it;
}
// tiles of a (token, head) row and where they start: a window drops the keys before kv_len - window
__device__ __forceinline__ int row_tiles(const PagedAttnParams& p, int t, int& k_lo, int& kv_len) {
  kv_len = p.q_kv_len[t];
  k_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
  if (p.q_seq[t] < 0 || kv_len <= k_lo) return 0;
  return (kv_len - (k_lo & ~(kTileKeys - 1)) + kTileKeys - 1) / kTileKeys;
}

// ---- descriptors ----
// MN-major operand, 128-byte swizzle, one swizzle row (128 elements of 8 bits) wide: rows of the atom are the eight
// consecutive contraction indices (keys), 1024 bytes between groups of eight.  Only the contraction-direction
// stride is exercised, so both offset fields carry it.
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1024 >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// MN-major operand without swizzle, 16 elements (one 16-byte chunk) wide: core matrices of [8 keys][16 B] packed
// back to back, 128 bytes between groups of eight keys (again the only stride that is exercised).
__device__ __forceinline__ uint64_t desc_mn_plain16(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 16;
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
constexpr uint32_t kIdescS = umma_idesc(128, kRows, 0, 0);                           // K-major A and B
constexpr uint32_t kIdescPV = umma_idesc(128, kRows, 0, 0) | (1u << 15) | (1u << 16);  // MN-major A and B

// ---- TMEM <-> registers, N columns of this thread's lane ----
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t* r) {
  if constexpr (N == 2) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr));
  } else if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
  } else if constexpr (N == 8) {
    tmem_ld_x8(taddr, r);
  } else {
    tmem_ld_x16(taddr, r);
  }
}
template <int N>
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t* r) {
  if constexpr (N == 2) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1,%2};" ::"r"(taddr), "r"(r[0]), "r"(r[1]) : "memory");
  } else if constexpr (N == 4) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
  } else {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
  }
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// barrier of the softmax threads that also ORs a predicate over all of them
__device__ __forceinline__ bool softmax_any(bool v) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 256, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r) : "r"(static_cast<uint32_t>(v)) : "memory");
  return r != 0;
}

// x ~ hi + lo, both e4m3; two values at a time.  Returns hi in the low 16 bits, lo in the high 16 bits.
__device__ __forceinline__ uint32_t split_e4m3x2(float a, float b) {
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
  const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hr));
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a - hf.x, b - hf.y), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(hi) | (static_cast<uint32_t>(lo) << 16);
}

// the same split with the second term scaled by kLoScale (P: separate accumulators for the two terms)
__device__ __forceinline__ uint32_t split_e4m3x2_scaled(float a, float b) {
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
  const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hr));
  const __nv_fp8x2_storage_t lo =
      __nv_cvt_float2_to_fp8x2(make_float2((a - hf.x) * kLoScale, (b - hf.y) * kLoScale), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(hi) | (static_cast<uint32_t>(lo) << 16);
}
// maximum over the warp in one instruction: floats mapped to integers of the same order
__device__ __forceinline__ float warp_max_fast(float v) {
  int i = __float_as_int(v);
  i = i >= 0 ? i : i ^ 0x7fffffff;
  i = __reduce_max_sync(0xffffffffu, i);
  return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

struct Bars {
  uint64_t full[kStages], empty[kStages];
  uint64_t s_full[2], p_full[2], pv_done[2];
  uint64_t q_full[2], q_empty[2];
};

// A position in this CTA's stream of tiles: local item, its descriptor, tile inside the item, ordinal of the item
// among the non-empty ones (selects the Q buffer).
struct Cursor {
  int li;
  Item it;
  int j;
  uint32_t qn;
  bool valid;
};
__device__ __forceinline__ void cursor_seek(Cursor& c, const ItemRec* recs, int n_local) {
  c.valid = c.li < n_local;
  if (c.valid) {
    c.it = get_item(recs, c.li);
    c.j = 0;
  }
}
__device__ __forceinline__ void cursor_next(Cursor& c, const ItemRec* recs, int n_local) {
  if (++c.j >= c.it.nt) {
    ++c.li;
    ++c.qn;
    cursor_seek(c, recs, n_local);
  }
}

template <int NR>   // query rows of the group, padded to 4 / 8 / 16
__global__ void __launch_bounds__(kThreads, 1) paged_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                    const __grid_constant__ CUtensorMap tmap_v,
                                                                    const TcParams tp) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) Bars bars;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float q_scale[2][kRows];
  __shared__ float red_m[2][kSoftmaxWarps][kRows / 2];
  __shared__ float red_v[2][kSoftmaxWarps];
  __shared__ float red_l[kSoftmaxWarps][kRows / 2];
  __shared__ ItemRec item_recs[kMaxItems];
  __shared__ int box_rows[kMaxBoxes];   // boxes of this CTA's pieces in order: first cache row of the box, or -1
  __shared__ int part_sh[4];            // prologue: total tiles, longest row, pieces, boxes

  const PagedAttnParams& p = tp.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = tp.G;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_base = smem_base + kStages * kStageBytes;
  const uint32_t p_base = q_base + 2 * kQBytes;
  uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abortp = &abort_flag;
  int tn = 0;   // this thread's trace cursor
  if (threadIdx.x == 0) trace_event(tp.trace, 2, tn, 0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 2);   // the S product and the P.V product each release their half
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars.s_full[b]), 1);
      mbar_init(smem_u32(&bars.p_full[b]), kSoftmaxThreads);
      mbar_init(smem_u32(&bars.pv_done[b]), 1);
      mbar_init(smem_u32(&bars.q_full[b]), 1);
      mbar_init(smem_u32(&bars.q_empty[b]), 1 + kSoftmaxThreads);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == kWarpS) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  // zero the V halves of the ring and the Q tiles once (see the header: a stale V row is multiplied by an exact
  // zero, so it must not hold a NaN pattern; stale K rows only produce scores that are masked; Q rows past the
  // group stay zero for the whole kernel)
  for (int i = threadIdx.x; i < kStages * (kOperandBytes / 16); i += kThreads) {
    const int st = i / (kOperandBytes / 16), o = i % (kOperandBytes / 16);
    reinterpret_cast<uint4*>(smem_gen + st * kStageBytes + kOperandBytes)[o] = make_uint4(0, 0, 0, 0);
  }
  for (int i = threadIdx.x; i < (2 * kQBytes + 2 * kPBytes) / 16; i += kThreads)   // Q and P^T tiles (adjacent)
    reinterpret_cast<uint4*>(smem_gen + kStages * kStageBytes)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x < 2 * kRows) (&q_scale[0][0])[threadIdx.x] = 1.f;   // rows past the group: a finite scale for their zero scores
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  pdl_launch_next();
  pdl_wait_prior();   // q, the new token's cache rows and the step's tables come from earlier kernels

  const int H = p.n_kv_heads, P = p.kv.page_size;
  // ---- partition: every CTA takes the same number of consecutive 128-key tiles of the flattened (row, tile) list;
  // a row cut by a CTA boundary yields one piece (and one partial-result slot) per CTA that touches it.  The tile
  // counts and their prefix sums live in the K half of stage 0 until the first TMA load overwrites it. ----
  const int R = p.Tq * H;
  int* sc = reinterpret_cast<int*>(smem_gen);            // [R + 1] tile counts, then exclusive prefix sums
  int* chunk_sum = sc + R + 1;                            // [kThreads]
  if (threadIdx.x < 4) part_sh[threadIdx.x] = 0;
  __syncthreads();
  {
    int longest = 0;
    for (int r = threadIdx.x; r < R; r += kThreads) {
      int k_lo, kv_len;
      const int nt = row_tiles(p, r / H, k_lo, kv_len);
      sc[r] = nt;
      longest = max(longest, nt);
    }
    longest = __reduce_max_sync(0xffffffffu, longest);
    if (lane == 0) atomicMax(&part_sh[1], longest);
  }
  __syncthreads();
  const int chunk = (R + kThreads - 1) / kThreads;
  {
    int sum = 0;
    for (int r = threadIdx.x * chunk; r < min(R, (threadIdx.x + 1) * chunk); ++r) sum += sc[r];
    chunk_sum[threadIdx.x] = sum;
  }
  __syncthreads();
  if (warp == 0) {   // exclusive scan of the kThreads chunk sums: 12 per lane, then across the warp
    constexpr int kPer = kThreads / 32;
    int loc[kPer], tot = 0;
#pragma unroll
    for (int i = 0; i < kPer; ++i) { loc[i] = tot; tot += chunk_sum[lane * kPer + i]; }
    int inc = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += v;
    }
    const int base = inc - tot;
#pragma unroll
    for (int i = 0; i < kPer; ++i) chunk_sum[lane * kPer + i] = base + loc[i];
    if (lane == 31) part_sh[0] = inc;
  }
  __syncthreads();
  {
    int run = chunk_sum[threadIdx.x];
    for (int r = threadIdx.x * chunk; r < min(R, (threadIdx.x + 1) * chunk); ++r) {
      const int nt = sc[r];
      sc[r] = run;
      run += nt;
    }
    if (threadIdx.x == 0) sc[R] = part_sh[0];
  }
  __syncthreads();
  const int total_tiles = part_sh[0];
  // tiles per CTA: an equal share, but never so small that the longest row would need more slots than it has
  const int share = max(1, max((total_tiles + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x),
                               (part_sh[1] + max(1, p.n_splits - 1) - 1) / max(1, p.n_splits - 1)));
  const int my_lo = min(total_tiles, static_cast<int>(blockIdx.x) * share);
  const int my_hi = min(total_tiles, my_lo + share);
  if (threadIdx.x == 0 && my_lo < my_hi) {
    // first row that reaches past my_lo (binary search over the prefix sums), then walk
    int lo = 0, hi = R;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (sc[mid + 1] <= my_lo) lo = mid + 1; else hi = mid;
    }
    int n = 0, boxes = 0, pos = my_lo;
    for (int r = lo; r < R && pos < my_hi; ++r) {
      const int nt = sc[r + 1] - sc[r];
      if (nt == 0) continue;
      const int a = pos - sc[r], b = min(nt, my_hi - sc[r]);
      if (n < kMaxItems && boxes + 2 * (b - a) <= kMaxBoxes) {
        int k_lo, kv_len;
        row_tiles(p, r / H, k_lo, kv_len);
        const int k0 = (k_lo & ~(kTileKeys - 1)) + a * kTileKeys;
        ItemRec rec;
        rec.t = r / H;
        rec.kvh_split = ((r % H) << 16) | (static_cast<int>(blockIdx.x) - sc[r] / share);
        rec.k_begin = max(k_lo, k0);
        rec.k_end = min(kv_len, k0 + (b - a) * kTileKeys);
        rec.k0 = k0;
        rec.box0 = boxes;
        item_recs[n++] = rec;
        boxes += 2 * (b - a);
      } else {
        abort_flag = 1;   // (the host bounds the share; a violation means an argument lied about the lengths)
        report_status(tp.status, kStatusBadArgument);
      }
      pos = sc[r] + b;
    }
    part_sh[2] = n;
    part_sh[3] = boxes;
  }
  // partial-result slots that no piece fills: the CTA that holds a row's first tile closes the row's unused slots;
  // rows without keys are closed round-robin
  for (int r = threadIdx.x; r < R; r += kThreads) {
    const int nt = sc[r + 1] - sc[r];
    int first_empty = -1;
    if (nt == 0) {
      if (r % static_cast<int>(gridDim.x) == static_cast<int>(blockIdx.x)) first_empty = 0;
    } else if (sc[r] / share == static_cast<int>(blockIdx.x)) {
      first_empty = (sc[r] + nt - 1) / share - static_cast<int>(blockIdx.x) + 1;
    }
    if (first_empty >= 0) {
      const long long row0 = (static_cast<long long>(r / H) * p.n_q_heads + (r % H) * G) * p.n_splits;
      for (int g2 = 0; g2 < G; ++g2)
        for (int sl = first_empty; sl < p.n_splits; ++sl) {
          float* ml = p.part_ml + (row0 + static_cast<long long>(g2) * p.n_splits + sl) * 2;
          ml[0] = -CUDART_INF_F;
          ml[1] = 0.f;
        }
    }
  }
  __syncthreads();
  const int n_local = part_sh[2];
  // the cache rows of the pieces' boxes, looked up once: no role chases a table afterwards
  for (int i = 0; i < n_local; ++i) {
    const ItemRec r = item_recs[i];
    const int nb = 2 * ((r.k_end - r.k0 + kTileKeys - 1) / kTileKeys);
    for (int b2 = threadIdx.x; b2 < nb; b2 += kThreads) {
      const int key0 = r.k0 + b2 * kBoxKeys;
      int row = -1;
      if (key0 < r.k_end && key0 + kBoxKeys > r.k_begin) {
        const int page = p.block_table[static_cast<long long>(p.q_seq[r.t]) * p.table_stride + key0 / P];
        if (page >= 0) row = (page * H + (r.kvh_split >> 16)) * P + key0 % P;
      }
      box_rows[r.box0 + b2] = row;
    }
  }
  fence_proxy_async_smem();   // the scratch words above lie where the first TMA load lands
  __syncthreads();
  if (threadIdx.x == 0) trace_event(tp.trace, 2, tn, 1);

  if (warp == kWarpProducer) {
    // =========================== TMA producer ===========================
    if (elect_one()) {
      const uint64_t pol = l2_policy_evict_first();
      uint32_t g = 0;
      for (int li = 0; li < n_local; ++li) {
        const Item it = get_item(item_recs, li);
        for (int j = 0; j < it.nt; ++j, ++g) {
          const int stage = g % kStages;
          trace_event(tp.trace, 0, tn, 10);
          if (g >= kStages)
            mbar_wait(smem_u32(&bars.empty[stage]), ((g / kStages) & 1) ^ 1, abortp, tp.status, kStatusEmptyWaitTimeout);
          if (*abortp) break;
          trace_event(tp.trace, 0, tn, 11);
          int rows[2];
          uint32_t bytes = 0;
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            rows[b] = box_rows[it.box0 + 2 * j + b];
            if (rows[b] >= 0) bytes += 4 * kBoxBytes;
          }
          const uint32_t full = smem_u32(&bars.full[stage]);
          const uint32_t dst = smem_base + stage * kStageBytes;
          mbar_expect_tx(full, bytes);
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            if (rows[b] < 0) continue;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              tma_load_2d(dst + h * kHalfBytes + b * kBoxBytes, &tmap_k, full, h * 128, rows[b], pol);
              tma_load_2d(dst + kOperandBytes + h * kHalfBytes + b * kBoxBytes, &tmap_v, full, h * 128, rows[b], pol);
            }
          }
        }
        if (*abortp) break;
      }
      if (*abortp) {
        // unwinding: let the copies that were issued land before the CTA leaves
        const uint32_t first = g > kStages ? g - kStages : 0;
        for (uint32_t j = first; j < g; ++j)
          for (uint32_t spin = 0; spin < (1u << 20); ++spin)
            if (mbar_try_wait(smem_u32(&bars.full[j % kStages]), (j / kStages) & 1)) break;
      }
    }
    __syncwarp();
  } else if (warp == kWarpS) {
    // =========================== issuer of S^T = K . Q^T ===========================
    // Sixteen k-steps (two e4m3 terms of Q x two d-halves x four 32-byte steps) go into FOUR partial accumulators,
    // one per step inside the swizzle atom, so that consecutive instructions never depend on each other; the
    // softmax threads add the four partials.  (Sixteen dependent N = 16 instructions would pay the tensor pipe's
    // full latency sixteen times.)
    if (elect_one()) {
      Cursor c{0, {}, 0, 0, false};
      cursor_seek(c, item_recs, n_local);
      for (uint32_t gs = 0; c.valid && !*abortp; ++gs) {
        const uint32_t qb = c.qn & 1;
        if (c.j == 0) mbar_wait(smem_u32(&bars.q_full[qb]), (c.qn >> 1) & 1, abortp, tp.status, kStatusAttnWait);
        // the S^T buffer of this parity was read by the softmax of two tiles ago (its P^T arrival says so)
        if (gs >= 2) mbar_wait(smem_u32(&bars.p_full[gs & 1]), ((gs >> 1) - 1) & 1, abortp, tp.status, kStatusAttnWait);
        trace_event(tp.trace, 1, tn, 20);
        mbar_wait(smem_u32(&bars.full[gs % kStages]), (gs / kStages) & 1, abortp, tp.status, kStatusTmaWaitTimeout);
        trace_event(tp.trace, 1, tn, 21);
        tc_fence_after();
        const uint32_t kaddr = smem_base + (gs % kStages) * kStageBytes;
        const uint32_t qaddr = q_base + qb * kQBytes;
        const uint32_t d = tmem_base + (gs & 1) * (4 * kRows);
#pragma unroll
        for (int part = 0; part < 2; ++part)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint64_t a = umma_desc_k_sw128(kaddr + h * kHalfBytes);
            const uint64_t b = umma_desc_k_sw128(qaddr + part * kQPartBytes + h * (kRows * 128));
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              tc_mma_f8f6f4(d + ks * kRows, a + 2 * ks, b + 2 * ks, kIdescS, (part | h) ? 1u : 0u);
          }
        tc_commit(smem_u32(&bars.s_full[gs & 1]));
        tc_commit(smem_u32(&bars.empty[gs % kStages]));
        if (c.j == c.it.nt - 1) tc_commit(smem_u32(&bars.q_empty[qb]));
        trace_event(tp.trace, 1, tn, 22);
        cursor_next(c, item_recs, n_local);
      }
    }
    __syncwarp();
  } else if (warp == kWarpPV) {
    // =========================== issuer of O^T += V^T . P^T ===========================
    if (elect_one()) {
      Cursor c{0, {}, 0, 0, false};
      cursor_seek(c, item_recs, n_local);
      for (uint32_t gp = 0; c.valid && !*abortp; ++gp) {
        trace_event(tp.trace, 4, tn, 23);
        mbar_wait(smem_u32(&bars.p_full[gp & 1]), (gp >> 1) & 1, abortp, tp.status, kStatusAttnWait);
        trace_event(tp.trace, 4, tn, 24);
        tc_fence_after();
        const uint32_t vaddr = smem_base + (gp % kStages) * kStageBytes + kOperandBytes;
        const uint32_t paddr = p_base + (gp & 1) * kPBytes;
        // four accumulators (two terms of P x two d-halves); the key steps are the outer loop, so that consecutive
        // instructions go to different accumulators
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)   // 32 keys per instruction: four 1024-byte groups of V, 512 bytes of P^T
#pragma unroll
          for (int part = 0; part < 2; ++part)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint64_t a = desc_mn_sw128(vaddr + h * kHalfBytes);
              const uint64_t b = desc_mn_plain16(paddr + part * kPPartBytes);
              tc_mma_f8f6f4(tmem_base + kColO + (2 * part + h) * kRows, a + ks * (4096 >> 4), b + ks * (512 >> 4),
                            kIdescPV, (c.j == 0 && ks == 0) ? 0u : 1u);
            }
        tc_commit(smem_u32(&bars.empty[gp % kStages]));
        tc_commit(smem_u32(&bars.pv_done[gp & 1]));
        trace_event(tp.trace, 4, tn, 25);
        cursor_next(c, item_recs, n_local);
      }
    }
    __syncwarp();
  } else if (warp == kWarpQ) {
    // =========================== query staging ===========================
    uint32_t qn = 0;
    for (int li = 0; li < n_local; ++li) {
      const Item it = get_item(item_recs, li);
      const uint32_t qb = qn & 1;
      // lane owns d = 8 * lane .. + 7 of every row; all rows are requested before the first one is used
      uint4 raw[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r)
        if (r < G)
          raw[r] = *reinterpret_cast<const uint4*>(
              p.q + (static_cast<long long>(it.t) * p.n_q_heads + it.kvh * G + r) * D + lane * 8);
      if (qn >= 2) mbar_wait(smem_u32(&bars.q_empty[qb]), ((qn >> 1) - 1) & 1, abortp, tp.status, kStatusAttnWait);
      const int half = lane >> 4, chunk = (lane & 15) >> 1, sub = (lane & 1) * 8;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        if (r >= G) continue;
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
        float f[8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          f[2 * i] = __bfloat162float(v2[i].x);
          f[2 * i + 1] = __bfloat162float(v2[i].y);
          amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
        }
        amax = warp_max_fast(amax);
        const float sc = amax > 0.f ? amax / 448.f : 1.f;
        const float inv = 1.f / sc;
        uint32_t hi[2], lo[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t w0 = split_e4m3x2(f[4 * i] * inv, f[4 * i + 1] * inv);
          const uint32_t w1 = split_e4m3x2(f[4 * i + 2] * inv, f[4 * i + 3] * inv);
          hi[i] = (w0 & 0xffff) | (w1 << 16);
          lo[i] = (w0 >> 16) | (w1 & 0xffff0000u);
        }
        // K-major tile with the 128-byte swizzle: 16-byte chunk index XOR row-in-atom
        const uint32_t off = half * (kRows * 128) + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4) + sub;
        uint8_t* qdst = smem_gen + kStages * kStageBytes + qb * kQBytes + off;
        *reinterpret_cast<uint2*>(qdst) = make_uint2(hi[0], hi[1]);
        *reinterpret_cast<uint2*>(qdst + kQPartBytes) = make_uint2(lo[0], lo[1]);
        if (lane == 0) q_scale[qb][r] = sc;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.q_full[qb]));
      if (lane == 0) trace_event(tp.trace, 3, tn, 40);
      ++qn;
    }
  } else {
    // =========================== softmax: two threads per key (= TMEM lane), half of the rows each ===========
    constexpr int NH = NR / 2;                 // rows of this thread
    const int tid = threadIdx.x;               // 0..255
    const int key_lane = tid & 127;            // key inside the tile = TMEM lane
    const int rh = warp >> 2;                  // which half of the rows
    const int row0 = rh * NH;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float c_log2e = p.sm_scale * 1.4426950408889634f;
    const __half* kscales = reinterpret_cast<const __half*>(p.kv.k_scales);
    const __half* vscales = reinterpret_cast<const __half*>(p.kv.v_scales);
    // the scales of this thread's key in a tile, fetched one tile ahead of its scores (also across items)
    auto fetch = [&](const Cursor& c, float& ks, float& vs, bool& ok) {
      ok = false; ks = 0.f; vs = 0.f;
      if (!c.valid) return;
      const int key = c.it.k0 + c.j * kTileKeys + key_lane;
      if (key >= c.it.k_begin && key < c.it.k_end) {
        const int box_row = box_rows[c.it.box0 + (key - c.it.k0) / kBoxKeys];
        if (box_row >= 0) {
          const long long row = box_row + key % kBoxKeys;
          ks = __half2float(kscales[row]);
          vs = __half2float(vscales[row]);
          if (p.tree_mask != nullptr) {
            const int tbase = p.tree_base[c.it.t];
            ok = key < tbase || ((p.tree_mask[c.it.t] >> (key - tbase)) & 1ull);
          } else {
            ok = true;
          }
        }
      }
    };
    Cursor c{0, {}, 0, 0, false};
    cursor_seek(c, item_recs, n_local);
    float ks_n, vs_n;
    bool ok_n;
    fetch(c, ks_n, vs_n, ok_n);
    float qs[NH], m_run[NH], l_part[NH];
    float r_run = 0.f;
    for (uint32_t g = 0; c.valid; ++g) {
      const uint32_t qb = c.qn & 1;
      if (c.j == 0) {
        mbar_wait(smem_u32(&bars.q_full[qb]), (c.qn >> 1) & 1, abortp, tp.status, kStatusAttnWait);
#pragma unroll
        for (int r = 0; r < NH; ++r) {
          qs[r] = q_scale[qb][row0 + r] * c_log2e;
          m_run[r] = -CUDART_INF_F;
          l_part[r] = 0.f;
        }
        r_run = 0.f;
        mbar_arrive(smem_u32(&bars.q_empty[qb]));
      }
      const Item it = c.it;
      const int j = c.j;
      const float ks = ks_n, vs = vs_n;
      const bool ok = ok_n;
      Cursor nx = c;
      cursor_next(nx, item_recs, n_local);
      fetch(nx, ks_n, vs_n, ok_n);
      const uint32_t sb = g & 1;
      if (tid == 0) trace_event(tp.trace, 2, tn, 30);
      mbar_wait(smem_u32(&bars.s_full[sb]), (g >> 1) & 1, abortp, tp.status, kStatusAccumWaitTimeout);
      if (tid == 0) trace_event(tp.trace, 2, tn, 31);
      tc_fence_after();
      uint32_t acc[4][NH];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) tmem_ld<NH>(tmem_base + lane_sel + (sb * 4 + q4) * kRows + row0, acc[q4]);
      tmem_ld_wait();
      float s[NH];
      bool exceed = ok && vs > 2.f * r_run;
#pragma unroll
      for (int r = 0; r < NH; ++r) {
        const float dot = (__uint_as_float(acc[0][r]) + __uint_as_float(acc[1][r])) +
                          (__uint_as_float(acc[2][r]) + __uint_as_float(acc[3][r]));
        s[r] = ok ? dot * qs[r] * ks : -CUDART_INF_F;
        exceed |= s[r] > m_run[r] + kFrameSlack;   // (always true for a visible key while the row has no frame yet)
      }
      // Frames: a row's softmax frame m and the V-scale frame R only move when some key leaves the slack above them.
      // One barrier-with-OR says whether any does; on most tiles none does and no maximum is computed at all.
      bool moved = false;
      float fcorr[NH];
      float rr = 1.f;
      if (softmax_any(exceed)) {
#pragma unroll
        for (int r = 0; r < NH; ++r) {
          const float wm = warp_max_fast(s[r]);
          if (lane == 0) red_m[sb][warp][r] = wm;
        }
        {
          const float wv = warp_max_fast(ok ? vs : 0.f);
          if (lane == 0) red_v[sb][warp] = wv;
        }
        softmax_bar();
        const int w0 = rh * 4;
#pragma unroll
        for (int r = 0; r < NH; ++r) {
          const float tm = fmaxf(fmaxf(red_m[sb][w0][r], red_m[sb][w0 + 1][r]), fmaxf(red_m[sb][w0 + 2][r], red_m[sb][w0 + 3][r]));
          fcorr[r] = 1.f;
          if (tm > m_run[r] + kFrameSlack || (m_run[r] == -CUDART_INF_F && tm > -CUDART_INF_F)) {
            fcorr[r] = m_run[r] == -CUDART_INF_F ? 0.f : exp2f(m_run[r] - tm);
            m_run[r] = tm;
            moved = true;
          }
        }
        const float tv = fmaxf(fmaxf(red_v[sb][w0], red_v[sb][w0 + 1]), fmaxf(red_v[sb][w0 + 2], red_v[sb][w0 + 3]));
        if (tv > 2.f * r_run) {
          rr = r_run / tv;   // (r_run == 0: nothing was accumulated in the old frame)
          r_run = tv;
          moved = true;
        }
      }
      if (tid == 0) trace_event(tp.trace, 2, tn, 32);
      // the P^T buffer of this parity was read by the product of two tiles ago
      if (g >= 2) mbar_wait(smem_u32(&bars.pv_done[sb]), ((g >> 1) - 1) & 1, abortp, tp.status, kStatusAttnWait);
      if (moved && j > 0) {
        // O^T holds sums in the old frames: wait for the previous product, rescale this thread's 4 x NH columns
        mbar_wait(smem_u32(&bars.pv_done[(g - 1) & 1]), ((g - 1) >> 1) & 1, abortp, tp.status, kStatusAttnWait);
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          uint32_t o[NH];
          const uint32_t oaddr = tmem_base + lane_sel + kColO + h * kRows + row0;
          tmem_ld<NH>(oaddr, o);
          tmem_ld_wait();
#pragma unroll
          for (int r = 0; r < NH; ++r) o[r] = __float_as_uint(__uint_as_float(o[r]) * fcorr[r] * rr);
          tmem_st<NH>(oaddr, o);
        }
        tmem_st_wait();
#pragma unroll
        for (int r = 0; r < NH; ++r) l_part[r] *= fcorr[r];
      }
      if (tid == 0) trace_event(tp.trace, 2, tn, 33 + (moved && j > 0 ? 1 : 0));
      const float vw = (ok && r_run > 0.f) ? vs / r_run * kPScale : 0.f;
      uint32_t hi[NH / 4 + 1] = {}, lo[NH / 4 + 1] = {};
#pragma unroll
      for (int r = 0; r < NH; r += 2) {
        const float p0 = ok ? exp2f(s[r] - m_run[r]) : 0.f;
        const float p1 = ok ? exp2f(s[r + 1] - m_run[r + 1]) : 0.f;
        l_part[r] += p0;
        l_part[r + 1] += p1;
        const uint32_t w = split_e4m3x2_scaled(p0 * vw, p1 * vw);
        hi[r >> 2] |= (w & 0xffff) << (8 * (r & 3));
        lo[r >> 2] |= (w >> 16) << (8 * (r & 3));
      }
      uint8_t* pdst = smem_gen + kStages * kStageBytes + 2 * kQBytes + sb * kPBytes + key_lane * kRows + row0;
      if constexpr (NH == 2) {
        *reinterpret_cast<uint16_t*>(pdst) = static_cast<uint16_t>(hi[0]);
        *reinterpret_cast<uint16_t*>(pdst + kPPartBytes) = static_cast<uint16_t>(lo[0]);
      } else if constexpr (NH == 4) {
        *reinterpret_cast<uint32_t*>(pdst) = hi[0];
        *reinterpret_cast<uint32_t*>(pdst + kPPartBytes) = lo[0];
      } else {
        *reinterpret_cast<uint2*>(pdst) = make_uint2(hi[0], hi[1]);
        *reinterpret_cast<uint2*>(pdst + kPPartBytes) = make_uint2(lo[0], lo[1]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&bars.p_full[sb]));
      if (tid == 0) trace_event(tp.trace, 2, tn, 35);

      if (j == it.nt - 1) {
        // ---- the item's partial result ----
        const long long part_row0 = (static_cast<long long>(it.t) * p.n_q_heads + it.kvh * G) * p.n_splits + it.split;
#pragma unroll
        for (int r = 0; r < NH; ++r) {
          const float ws = warp_sum(l_part[r]);
          if (lane == 0) red_l[warp][r] = ws;
        }
        mbar_wait(smem_u32(&bars.pv_done[sb]), (g >> 1) & 1, abortp, tp.status, kStatusAttnWait);
        tc_fence_after();
        const float oscale = r_run / kPScale;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t o[NH], ol[NH];
          tmem_ld<NH>(tmem_base + lane_sel + kColO + h * kRows + row0, o);
          tmem_ld<NH>(tmem_base + lane_sel + kColO + (2 + h) * kRows + row0, ol);
          tmem_ld_wait();
#pragma unroll
          for (int r = 0; r < NH; ++r)
            if (row0 + r < G)
              p.part_o[(part_row0 + static_cast<long long>(row0 + r) * p.n_splits) * D + h * 128 + key_lane] =
                  (__uint_as_float(o[r]) + __uint_as_float(ol[r]) * (1.f / kLoScale)) * oscale;
        }
        tc_fence_before();
        softmax_bar();
        // row r is written by lane (r % NH) of the first warp of the half that owns it
        if ((warp & 3) == 0 && lane < NH && row0 + lane < G) {
          float mine = -CUDART_INF_F;
#pragma unroll
          for (int r = 0; r < NH; ++r) mine = (r == lane) ? m_run[r] : mine;
          float* ml = p.part_ml + (part_row0 + static_cast<long long>(row0 + lane) * p.n_splits) * 2;
          ml[0] = mine;
          ml[1] = red_l[warp][lane] + red_l[warp + 1][lane] + red_l[warp + 2][lane] + red_l[warp + 3][lane];
        }
        softmax_bar();   // red_l is reused by the next item
        if (tid == 0) trace_event(tp.trace, 2, tn, 36);
      }
      c = nx;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kWarpS) tmem_dealloc(tmem_base, kTmemCols);
}

struct MapKey {
  const void* base; uint64_t rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const { return std::hash<const void*>()(k.base) ^ (std::hash<uint64_t>()(k.rows) << 1); }
};

bool plane_map(const void* base, uint64_t rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{base, rows};
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap m;
    if (!make_tmap_2d(&m, TmapDtype::U8, base, rows, D, D, kBoxKeys, 128, true)) return false;
    if (cache.size() > 4096) cache.clear();
    it = cache.emplace(key, m).first;
  }
  *out = it->second;
  return true;
}

template <int NR>
cudaError_t launch_tc(const CUtensorMap& tk, const CUtensorMap& tv, const TcParams& tp, int grid, cudaStream_t stream,
                      bool pdl) {
  auto kern = paged_attn_tc_kernel<NR>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tk, tv, tp);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace

// Development aid: switch the event trace of CTA 0 on / off and copy it out ([5 roles][1024] entries, 0 = unused).
void paged_attention_tc_trace(bool enable, unsigned long long* host_out) {
  if (host_out != nullptr) cudaMemcpyFromSymbol(host_out, g_attn_trace, sizeof(g_attn_trace));
  static const unsigned long long zeros[kTraceRoles * kTraceLen] = {};
  cudaMemcpyToSymbol(g_attn_trace, zeros, sizeof(zeros));
  g_attn_trace_on = enable;
}

// Returns cudaErrorNotSupported when the problem is outside this kernel (the caller falls back to the mma.sync one).
cudaError_t paged_attention_tc_split(const PagedAttnParams& p, cudaStream_t stream, bool pdl) {
  const int G = p.n_q_heads / p.n_kv_heads;
  const int P = p.kv.page_size;
  if (p.kv.format != kKvFp8Row || p.head_dim != D || G > kRows || p.kv_plane_rows <= 0) return cudaErrorNotSupported;
  if (P % kBoxKeys || p.split_keys % kTileKeys || p.sel_blocks != nullptr) return cudaErrorNotSupported;
  if (reinterpret_cast<uintptr_t>(p.kv.k_codes) % 16 || reinterpret_cast<uintptr_t>(p.kv.v_codes) % 16 ||
      reinterpret_cast<uintptr_t>(p.q) % 16)
    return cudaErrorNotSupported;
  CUtensorMap tk, tv;
  if (!plane_map(p.kv.k_codes, static_cast<uint64_t>(p.kv_plane_rows), &tk) ||
      !plane_map(p.kv.v_codes, static_cast<uint64_t>(p.kv_plane_rows), &tv))
    return cudaErrorNotSupported;
  TcParams tp;
  tp.a = p;
  tp.G = G;
  tp.status = p.status;
  tp.trace = g_attn_trace_on ? 1 : 0;
  // The kernel cuts the (token, kv head) rows into pieces itself (equal numbers of 128-key tiles per CTA); n_splits
  // is the number of partial-result slots a row has, split_keys only bounds the context (kv_len <= n_splits x
  // split_keys).  Rows are only cut when they have at least two slots.
  const long long rows = static_cast<long long>(p.Tq) * p.n_kv_heads;
  const long long row_tiles_max = (static_cast<long long>(p.n_splits) * p.split_keys + kTileKeys - 1) / kTileKeys;
  if (p.n_splits < 2 || p.n_splits > 0xffff || rows + 1 + kThreads > kOperandBytes / 4) return cudaErrorNotSupported;
  const long long work = rows * row_tiles_max;
  const int grid = static_cast<int>(work < sm_count() ? work : sm_count());
  // shared tables of one CTA: at most kMaxBoxes / 2 tiles and kMaxItems pieces (one piece has at least one tile)
  const long long share_max = std::max((work + grid - 1) / grid, (row_tiles_max + p.n_splits - 2) / (p.n_splits - 1));
  if (share_max > kMaxBoxes / 2 || share_max > kMaxItems) return cudaErrorNotSupported;
  if (G <= 4) return launch_tc<4>(tk, tv, tp, grid, stream, pdl);
  if (G <= 8) return launch_tc<8>(tk, tv, tp, grid, stream, pdl);
  return launch_tc<16>(tk, tv, tp, grid, stream, pdl);
}

}  // namespace nfb
