// See linear_add_noalloc.h.  The scratch array below is the only device memory this entry point uses
// beyond the caller's inputs and output.
#include "linear_add_noalloc.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <mutex>

#include "../pointwise/pointwise.h"
#include "gemm.h"

namespace {

// fp32 split-K partials [splits][T][N].  In host code this name is only a handle for the runtime's symbol
// table, never a device address: the address is fetched per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[NFB200_NOALLOC_SCRATCH_FLOATS];

// Status word of the bounded waits inside the two kernels (0 = fine).  Each call copies it into the host mirror
// below at the end of its stream work; the NEXT call on that device reads the mirror and reports a failure.
static __device__ int g_noalloc_status;

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
int* g_status_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
volatile int g_status_mirror[kMaxDevices] = {};   // page-locked at first use (registered, not allocated)
bool g_mirror_registered = false;
std::mutex g_setup_mutex;

int fail(char* err, int err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) std::snprintf(err, static_cast<size_t>(err_len), "%s", msg);
  return code;
}

// One-time set-up per device, with that device current (the caller's current device is used as is).
const char* scratch_for_current_device(float** out, int* dev_out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  if (dev < 0 || dev >= kMaxDevices) return "device index out of range";
  std::lock_guard<std::mutex> g(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    void* sp = nullptr;
    e = cudaGetSymbolAddress(&sp, g_noalloc_status);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sms <= 0) return "cannot read the multiprocessor count";
    if (!g_mirror_registered) {
      // page-lock the mirror so that the device-to-host copy at the end of a call is asynchronous
      e = cudaHostRegister(const_cast<int*>(g_status_mirror), sizeof(g_status_mirror), cudaHostRegisterDefault);
      if (e != cudaSuccess) return cudaGetErrorString(e);
      g_mirror_registered = true;
    }
    g_status_ptr[dev] = static_cast<int*>(sp);
    g_sm_count[dev] = sms;
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  *dev_out = dev;
  return nullptr;
}

}  // namespace

extern "C" int nfb200_linear_add_noalloc(const void* x, long long ldx, const void* w, long long ldw, void* resid,
                                         int T, int N, int K, int splits, void* stream, char* err, int err_len) {
  if (x == nullptr || w == nullptr || resid == nullptr) return fail(err, err_len, 1, "null pointer argument");
  if (T <= 0 || N <= 0 || K <= 0) return fail(err, err_len, 1, "T, N and K must be positive");
  if (T > 256) return fail(err, err_len, 2, "T must be <= 256 (decode / verify sized problems)");
  // limits of the second kernel (16-byte accesses to the residual, one CTA cluster per row block)
  if (N % 8) return fail(err, err_len, 1, "N must be a multiple of 8");
  if (N > 8192) return fail(err, err_len, 2, "N must be <= 8192");
  if (reinterpret_cast<uintptr_t>(resid) & 15) return fail(err, err_len, 1, "resid must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15)
    return fail(err, err_len, 1, "x and w must be 16-byte aligned");
  if ((K % 8) || (ldx % 8) || (ldw % 8)) return fail(err, err_len, 1, "K, ldx and ldw must be multiples of 8");
  float* scratch = nullptr;
  int dev = -1;
  if (const char* m = scratch_for_current_device(&scratch, &dev)) return fail(err, err_len, 3, m);
  if (g_status_mirror[dev] != 0) {
    // a bounded wait of an earlier call on this device ran out: that call's residual is not valid
    const int code = g_status_mirror[dev];
    g_status_mirror[dev] = 0;
    cudaMemsetAsync(g_status_ptr[dev], 0, sizeof(int), static_cast<cudaStream_t>(stream));
    char msg[160];
    std::snprintf(msg, sizeof(msg), "an earlier call on this device gave up a bounded wait (status %d); "
                                    "its output is not valid, nothing was launched now", code);
    return fail(err, err_len, 5, msg);
  }
  const int num_kb = (K + 63) / 64;
  if (splits == 0) {
    splits = nfb::gemm_pick_splits(T, N, K, nfb::kEpiPartial, g_sm_count[dev]);
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
  nfb::GemmArgs a;
  a.w = w; a.N = N; a.K = K; a.ldw = ldw;
  a.x = x; a.T = T; a.ldx = ldx;
  a.partial = scratch;
  a.splits = splits;
  a.epi = nfb::kEpiPartial;
  a.ldo = 2;
  a.status = g_status_ptr[dev];
  a.stream = static_cast<cudaStream_t>(stream);
  if (const char* m = nfb::gemm_bf16(a)) return fail(err, err_len, 4, m);
  // resid = bf16(resid + sum_z partial[z])
  if (const char* m = nfb::add_rmsnorm(scratch, splits, nullptr, resid, resid, nullptr, nullptr, T, N, 0.f, 0,
                                       static_cast<cudaStream_t>(stream), false))
    return fail(err, err_len, 4, m);
  // leave the status where the next call on this device will look (asynchronous: the mirror is page-locked)
  if (cudaMemcpyAsync(const_cast<int*>(&g_status_mirror[dev]), g_status_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost,
                      static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return fail(err, err_len, 4, "could not queue the status read-back");
  return 0;
}
