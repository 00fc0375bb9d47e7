// Host entry points of the row / pointwise kernels (plain C++ ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfb {

// resid_out = bf16(resid_in + delta + sum_z partial[z]);  normed = rmsnorm(resid_out) * w
// Any of partial / delta / resid_in / resid_out / normed may be null.
const char* add_rmsnorm(const float* partial, int splits, const void* delta, const void* resid_in,
                        void* resid_out, const void* norm_w, void* normed, int T, int N, float eps,
                        int unit_offset, cudaStream_t stream, bool pdl, uint8_t* q_codes = nullptr,
                        uint8_t* q_sf = nullptr);
// q_codes / q_sf (optional): an nvfp4 copy of `normed` (packed e2m1 [T, N/2] + 128x4-tiled e4m3 scale plane) for a
// block-scaled GEMM that consumes the normalised rows.

const char* embed_gather(const int* ids, const void* table, void* out, int T, int N, int vocab,
                         cudaStream_t stream, bool pdl);

// Strided per-head RMSNorm (one warp per row of D values).
const char* head_rmsnorm(const void* x, long long row_stride, const void* w, void* y, long long out_stride,
                         int rows, int D, float eps, int unit_offset, cudaStream_t stream);

}  // namespace nfb
