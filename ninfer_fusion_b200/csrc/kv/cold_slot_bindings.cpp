// torch.ops.nfb200.{cold_slot_pack_int8, cold_slot_restore_int8, cold_slot_restore_bf16}
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <tuple>

#include "cold_slot.h"

namespace {

using at::Tensor;

Tensor cold_slot_pack_int8(const Tensor& codes, const Tensor& scales, int64_t rows_per_slot) {
  TORCH_CHECK(codes.is_cuda() && codes.scalar_type() == at::kChar && codes.dim() == 2 && codes.is_contiguous(),
              "cold_slot_pack_int8: codes must be a contiguous CUDA int8 [rows, dim] tensor");
  const int64_t R = codes.size(0), D = codes.size(1);
  TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kHalf && scales.is_contiguous() && scales.numel() == R * (D / 64),
              "cold_slot_pack_int8: scales must be fp16 [rows, dim / 64]");
  TORCH_CHECK(rows_per_slot > 0 && R % rows_per_slot == 0, "cold_slot_pack_int8: rows must be a multiple of rows_per_slot");
  c10::cuda::CUDAGuard guard(codes.device());
  const int64_t n = R / rows_per_slot;
  Tensor slots = at::empty({n, nfb::cold_slot_bytes(static_cast<int>(rows_per_slot), static_cast<int>(D))},
                           codes.options().dtype(at::kByte));
  const char* err = nfb::cold_slot_pack_int8(static_cast<const int8_t*>(codes.data_ptr()), scales.data_ptr(), static_cast<int>(n),
                                             static_cast<int>(rows_per_slot), static_cast<int>(D),
                                             static_cast<uint8_t*>(slots.data_ptr()), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(err == nullptr, err ? err : "");
  return slots;
}

void check_slots(const Tensor& slots, int64_t rows, int64_t dim) {
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kByte && slots.dim() == 2 && slots.is_contiguous() && rows > 0 &&
              dim > 0 && slots.size(1) == nfb::cold_slot_bytes(static_cast<int>(rows), static_cast<int>(dim)),
              "cold slot: slots must be a contiguous CUDA uint8 [n, slot_bytes(rows, dim)] tensor");
}

std::tuple<Tensor, Tensor> cold_slot_restore_int8(const Tensor& slots, int64_t rows, int64_t dim) {
  check_slots(slots, rows, dim);
  c10::cuda::CUDAGuard guard(slots.device());
  const int64_t n = slots.size(0);
  Tensor codes = at::empty({n * rows, dim}, slots.options().dtype(at::kChar));
  Tensor scales = at::empty({n * rows, dim / 64}, slots.options().dtype(at::kHalf));
  const char* err = nfb::cold_slot_restore_int8(static_cast<const uint8_t*>(slots.data_ptr()), static_cast<int>(n),
                                                static_cast<int>(rows), static_cast<int>(dim),
                                                static_cast<int8_t*>(codes.data_ptr()), scales.data_ptr(),
                                                at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(err == nullptr, err ? err : "");
  return {codes, scales};
}

Tensor cold_slot_restore_bf16(const Tensor& slots, int64_t rows, int64_t dim) {
  check_slots(slots, rows, dim);
  c10::cuda::CUDAGuard guard(slots.device());
  const int64_t n = slots.size(0);
  Tensor out = at::empty({n * rows, dim}, slots.options().dtype(at::kBFloat16));
  const char* err = nfb::cold_slot_restore_bf16(static_cast<const uint8_t*>(slots.data_ptr()), static_cast<int>(n),
                                                static_cast<int>(rows), static_cast<int>(dim), out.data_ptr(),
                                                at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(err == nullptr, err ? err : "");
  return out;
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(nfb200, m) {
  m.def("cold_slot_pack_int8(Tensor codes, Tensor scales, int rows_per_slot) -> Tensor", &cold_slot_pack_int8);
  m.def("cold_slot_restore_int8(Tensor slots, int rows, int dim) -> (Tensor, Tensor)", &cold_slot_restore_int8);
  m.def("cold_slot_restore_bf16(Tensor slots, int rows, int dim) -> Tensor", &cold_slot_restore_bf16);
}
