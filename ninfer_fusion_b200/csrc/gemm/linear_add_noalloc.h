// A C entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for hosts that embed the
// library where device allocation is off the table at call time: code running inside a captured or
// latency-critical region that owns all of the process's device memory up front, plugins that are handed
// raw device pointers by a foreign runtime (and therefore have no allocator of their own to ask), and
// processes whose memory pool is fully committed to another framework.  Such callers can still run the
// row-parallel "linear + residual add" of the decoder (o_proj / GDN out_proj / down_proj):
//
//     resid[t, n] += sum_k x[t, k] * w[n, k]            (bf16 in, fp32 accumulate, bf16 out)
//
// It is the split-K form of the tcgen05 GEMM: every K-split writes an fp32 partial tile and a second
// kernel sums the partials onto the residual.  The partials live in a file-scope `static __device__` array
// inside the library (16 MiB, present on every GPU that loads the library until the process exits), so the
// call itself performs no cudaMalloc / cudaFree and uses no allocating library routine.
//
// Rules for callers:
//   * splits * T * N must not exceed kNoAllocScratchFloats (4 Mi floats); larger problems are refused.
//   * T <= 256, N <= 8192 and N % 8 == 0; K, ldx and ldw multiples of 8; x, w and resid 16-byte aligned
//     (the second kernel updates the residual with 16-byte accesses).  Anything else is refused before a
//     kernel is launched, so a refused call leaves the scratch and the residual untouched.
//   * The kernels' internal waits are bounded.  Should one ever run out, the call that hit it cannot know
//     (it has returned already): the failure is recorded on the device, copied to the host at the end of that
//     call's stream work, and the NEXT call on that device returns code 5 without launching anything.
//   * The first call on a device looks up the scratch array's device address (cudaGetSymbolAddress with
//     that device current).  Make that first call outside any stream capture, and early: when the CUDA
//     runtime loads modules lazily, this look-up is also the moment the driver instantiates the library's
//     static array on that device (free device memory drops by 16 MiB once, there and never again).
//   * All calls share the one scratch array.  Nothing in it has to start at zero (each call overwrites
//     every partial it later reads), but two calls that overlap on the GPU (different streams, or
//     programmatic overlap) race on it: serialise them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define NFB200_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

// x: [T, K] bf16 (leading dimension ldx elements), w: [N, K] bf16 (ldw), resid: [T, N] bf16, contiguous,
// updated in place.  splits: K-splits (1..8; 0 = choose).  stream: a cudaStream_t (may be null).
// Returns 0 on success; otherwise a non-zero code and, when err != NULL, a message in err[0..err_len).
__attribute__((visibility("default")))
int nfb200_linear_add_noalloc(const void* x, long long ldx, const void* w, long long ldw, void* resid, int T,
                              int N, int K, int splits, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
