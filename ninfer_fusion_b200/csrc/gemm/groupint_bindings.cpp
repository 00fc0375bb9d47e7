// torch.ops.nfb200.{groupint_linear, groupint_linear_pair}: checked adapters over the encoded row-split object
// (base plane, high-bit plane and scale plane at their 256-byte aligned offsets, as the artifact stores them).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "gemm_groupint.h"
#include "../pointwise/hadamard.h"

namespace {

using at::Tensor;
using OptT = const std::optional<Tensor>&;

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// plane offsets of one encoded [N, K] object; returns the object's size
int64_t bind_planes(const Tensor& payload, int64_t fmt, int64_t N, int64_t K, nfb::GroupIntWeight& w) {
  TORCH_CHECK(payload.is_cuda() && payload.scalar_type() == at::kByte && payload.is_contiguous(),
              "groupint: payload must be a contiguous CUDA uint8 tensor");
  TORCH_CHECK(fmt >= 0 && fmt <= 3, "groupint: unknown format");
  const int64_t Kp = align_up(K, 128);
  const int64_t group = fmt == nfb::kW8G32 ? 32 : 64;
  const int64_t hb = fmt == nfb::kQ5G64 ? 1 : fmt == nfb::kQ6G64 ? 2 : 0;
  const int64_t base_bytes = fmt == nfb::kW8G32 ? N * Kp : N * Kp / 2;
  const int64_t high_bytes = N * Kp * hb / 8;
  const int64_t high_off = align_up(base_bytes, 256);
  const int64_t scale_off = high_off + align_up(high_bytes, 256);
  const int64_t total = scale_off + N * (Kp / group) * 2;
  TORCH_CHECK(payload.numel() >= total, "groupint: payload is shorter than its planes (", payload.numel(), " < ", total, ")");
  const uint8_t* b = static_cast<const uint8_t*>(payload.data_ptr());
  w.base = b;
  w.high = hb ? b + high_off : nullptr;
  w.scale = reinterpret_cast<const __half*>(b + scale_off);
  w.N = static_cast<int>(N);
  return total;
}

// optional device status word (int32[1]) that a bounded wait which ran out is recorded in
int* status_ptr(OptT status) {
  if (!status.has_value() || !status->defined()) return nullptr;
  TORCH_CHECK(status->is_cuda() && status->scalar_type() == at::kInt && status->numel() >= 1, "groupint: status must be a CUDA int32 tensor");
  return static_cast<int*>(status->data_ptr());
}

void check_act(const Tensor& x, int64_t K) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && x.size(1) == K,
              "groupint: x must be a row-major bf16 [T, K] matrix");
}
void check_out(const Tensor& o, int64_t T, int64_t N, const char* name) {
  TORCH_CHECK(o.is_cuda() && o.scalar_type() == at::kBFloat16 && o.dim() == 2 && o.stride(1) == 1 && o.size(0) == T &&
              o.size(1) == N, "groupint: ", name, " must be a row-major bf16 [T, N] matrix");
}

void run_chunks(nfb::GroupIntLinearParams p, const Tensor& x, const Tensor* resid) {
  const int64_t T = x.size(0);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
  const __nv_bfloat16* x0 = static_cast<const __nv_bfloat16*>(x.data_ptr());
  __nv_bfloat16* o0 = p.w[0].out;
  __nv_bfloat16* o1 = p.w[1].out;
  const __nv_bfloat16* r0 = resid ? static_cast<const __nv_bfloat16*>(resid->data_ptr()) : nullptr;
  for (int64_t t0 = 0; t0 < T; t0 += 32) {   // weights are re-streamed per 32 tokens: meant for decode-sized T
    p.T = static_cast<int>(std::min<int64_t>(32, T - t0));
    p.x = x0 + t0 * p.ldx;
    p.w[0].out = o0 + t0 * p.w[0].ldo;
    if (p.n_weights == 2) p.w[1].out = o1 + t0 * p.w[1].ldo;
    p.resid = r0 ? r0 + t0 * p.ldr : nullptr;
    const char* err = nfb::groupint_linear(p, stream);
    TORCH_CHECK(err == nullptr, err ? err : "");
  }
}

void groupint_linear(const Tensor& x, const Tensor& payload, int64_t fmt, int64_t N, int64_t K, const Tensor& out, OptT resid,
                     OptT status) {
  check_act(x, K);
  check_out(out, x.size(0), N, "out");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::GroupIntLinearParams p = {};
  p.K = static_cast<int>(K); p.Kp = static_cast<int>(align_up(K, 128)); p.fmt = static_cast<int>(fmt); p.n_weights = 1;
  bind_planes(payload, fmt, N, K, p.w[0]);
  p.w[0].out = static_cast<__nv_bfloat16*>(out.data_ptr()); p.w[0].ldo = out.stride(0);
  p.ldx = x.stride(0);
  p.status = status_ptr(status);
  const Tensor* r = nullptr;
  if (resid.has_value() && resid->defined()) {
    check_out(*resid, x.size(0), N, "resid");
    r = &*resid; p.ldr = resid->stride(0);
  }
  if (x.size(0) > 0) run_chunks(p, x, r);
}

void groupint_linear_pair(const Tensor& x, const Tensor& payload0, int64_t N0, const Tensor& payload1, int64_t N1, int64_t fmt,
                          int64_t K, const Tensor& out0, const Tensor& out1, OptT status) {
  check_act(x, K);
  check_out(out0, x.size(0), N0, "out0");
  check_out(out1, x.size(0), N1, "out1");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::GroupIntLinearParams p = {};
  p.K = static_cast<int>(K); p.Kp = static_cast<int>(align_up(K, 128)); p.fmt = static_cast<int>(fmt); p.n_weights = 2;
  bind_planes(payload0, fmt, N0, K, p.w[0]);
  bind_planes(payload1, fmt, N1, K, p.w[1]);
  p.w[0].out = static_cast<__nv_bfloat16*>(out0.data_ptr()); p.w[0].ldo = out0.stride(0);
  p.w[1].out = static_cast<__nv_bfloat16*>(out1.data_ptr()); p.w[1].ldo = out1.stride(0);
  p.ldx = x.stride(0);
  p.status = status_ptr(status);
  if (x.size(0) > 0) run_chunks(p, x, nullptr);
}

void hadamard_blocks(const Tensor& x, const Tensor& out, int64_t block) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "hadamard_blocks: x must be row-major bf16");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.stride(1) == 1 &&
              out.sizes() == x.sizes(), "hadamard_blocks: out must match x");
  c10::cuda::CUDAGuard guard(x.device());
  const char* err = nfb::hadamard_blocks(static_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0),
                                         static_cast<__nv_bfloat16*>(out.data_ptr()), out.stride(0),
                                         static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), static_cast<int>(block),
                                         at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(err == nullptr, err ? err : "");
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(nfb200, m) {
  m.def("hadamard_blocks(Tensor x, Tensor out, int block) -> ()", &hadamard_blocks);
  m.def("groupint_linear(Tensor x, Tensor payload, int fmt, int N, int K, Tensor out, Tensor? resid, Tensor? status=None) -> ()", &groupint_linear);
  m.def("groupint_linear_pair(Tensor x, Tensor payload0, int N0, Tensor payload1, int N1, int fmt, int K, Tensor out0, "
        "Tensor out1, Tensor? status=None) -> ()", &groupint_linear_pair);
}
