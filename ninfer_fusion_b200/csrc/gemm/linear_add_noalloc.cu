// See linear_add_noalloc.h.  The scratch array below is the only device memory this entry point uses
// beyond the caller's inputs and output.
#include "linear_add_noalloc.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../pointwise/pointwise.h"
#include "gemm.h"

namespace {

// fp32 split-K partials [splits][T][N].  In host code this name is only a handle for the runtime's symbol
// table, never a device address: the address is fetched per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[NFB200_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

int fail(char* err, int err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) std::snprintf(err, static_cast<size_t>(err_len), "%s", msg);
  return code;
}

// One-time set-up per device, with that device current (the caller's current device is used as is).
const char* scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  if (dev < 0 || dev >= kMaxDevices) return "device index out of range";
  std::lock_guard<std::mutex> g(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return nullptr;
}

}  // namespace

extern "C" int nfb200_linear_add_noalloc(const void* x, long long ldx, const void* w, long long ldw, void* resid,
                                         int T, int N, int K, int splits, void* stream, char* err, int err_len) {
  if (x == nullptr || w == nullptr || resid == nullptr) return fail(err, err_len, 1, "null pointer argument");
  if (T <= 0 || N <= 0 || K <= 0) return fail(err, err_len, 1, "T, N and K must be positive");
  if (T > 256) return fail(err, err_len, 2, "T must be <= 256 (decode / verify sized problems)");
  const int num_kb = (K + 63) / 64;
  if (splits == 0) {
    splits = nfb::gemm_pick_splits(T, N, K, nfb::kEpiPartial, 148);
    while (splits > 1 && static_cast<long long>(splits) * T * N > NFB200_NOALLOC_SCRATCH_FLOATS) --splits;
    while (splits > 1 && (num_kb + splits - 1) / splits * (splits - 1) >= num_kb) --splits;
  }
  if (splits < 1 || splits > 8) return fail(err, err_len, 1, "splits must be in 1..8");
  if (static_cast<long long>(splits) * T * N > NFB200_NOALLOC_SCRATCH_FLOATS) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "splits*T*N = %lld floats exceeds the built-in scratch of %d floats",
                  static_cast<long long>(splits) * T * N, NFB200_NOALLOC_SCRATCH_FLOATS);
    return fail(err, err_len, 2, msg);
  }
  float* scratch = nullptr;
  if (const char* m = scratch_for_current_device(&scratch)) return fail(err, err_len, 3, m);

  nfb::GemmArgs a;
  a.w = w; a.N = N; a.K = K; a.ldw = ldw;
  a.x = x; a.T = T; a.ldx = ldx;
  a.partial = scratch;
  a.splits = splits;
  a.epi = nfb::kEpiPartial;
  a.ldo = 2;
  a.stream = static_cast<cudaStream_t>(stream);
  if (const char* m = nfb::gemm_bf16(a)) return fail(err, err_len, 4, m);
  // resid = bf16(resid + sum_z partial[z])
  if (const char* m = nfb::add_rmsnorm(scratch, splits, nullptr, resid, resid, nullptr, nullptr, T, N, 0.f, 0,
                                       static_cast<cudaStream_t>(stream), false))
    return fail(err, err_len, 4, m);
  return 0;
}
