// torch.ops.nfb200.{gemm_quant, quant_act_*}: checked adapters to the quantised-weight GEMM launchers.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstddef>

#include "../comm/comm.h"
#include "gemm_quant.h"

namespace {

inline size_t nfb_tp_call_idx_offset() { return offsetof(nfb::TpState, call_idx); }

using at::Tensor;
using OptT = const std::optional<Tensor>&;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void chk(const char* err) { TORCH_CHECK(err == nullptr, err ? err : ""); }
inline void need(const Tensor& t, at::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
}

void quant_act_fp8(const Tensor& x, const Tensor& codes, const Tensor& scale, bool pdl) {
  need(x, at::kBFloat16, "x"); need(codes, at::kByte, "codes"); need(scale, at::kFloat, "scale");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && codes.is_contiguous() && codes.numel() >= x.numel() &&
              scale.numel() >= x.size(0), "quant_act_fp8: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  chk(nfb::quant_act_fp8(static_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0), x.size(0), x.size(1),
                         static_cast<uint8_t*>(codes.data_ptr()), static_cast<float*>(scale.data_ptr()), cur_stream(), pdl));
}

void quant_act_nvfp4(const Tensor& x, const Tensor& codes, const Tensor& sf_plane, bool pdl) {
  need(x, at::kBFloat16, "x"); need(codes, at::kByte, "codes"); need(sf_plane, at::kByte, "sf_plane");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && codes.is_contiguous() && codes.numel() >= x.numel() / 2 &&
              sf_plane.numel() >= nfb::nvfp4_act_scale_bytes(x.size(0), x.size(1)), "quant_act_nvfp4: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  chk(nfb::quant_act_nvfp4(static_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0), x.size(0), x.size(1),
                           static_cast<uint8_t*>(codes.data_ptr()), static_cast<uint8_t*>(sf_plane.data_ptr()),
                           cur_stream(), pdl));
}

// x_codes: [T, K] (fp8) or [T, K/2] (nvfp4) bytes; w_codes likewise with N rows.
void gemm_quant(int64_t qtype, const Tensor& x_codes, const Tensor& x_scale, const Tensor& w_codes, const Tensor& w_scale,
                double w_divisor, const Tensor& out, int64_t epi, OptT resid, int64_t splits, OptT status, bool pdl,
                OptT next_codes, OptT next_sf) {
  need(x_codes, at::kByte, "x_codes"); need(w_codes, at::kByte, "w_codes"); need(out, at::kBFloat16, "out");
  TORCH_CHECK(x_codes.dim() == 2 && w_codes.dim() == 2 && x_codes.stride(1) == 1 && w_codes.stride(1) == 1 &&
              x_codes.size(1) == w_codes.size(1), "gemm_quant: code shapes");
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.size(0) == x_codes.size(0), "gemm_quant: out shape");
  c10::cuda::CUDAGuard guard(x_codes.device());
  nfb::QGemmArgs a;
  a.qtype = static_cast<int>(qtype);
  const bool bs = qtype == nfb::kQNvfp4;
  a.N = w_codes.size(0); a.T = x_codes.size(0); a.K = bs ? w_codes.size(1) * 2 : w_codes.size(1);
  a.w = w_codes.data_ptr(); a.ldw = w_codes.stride(0);
  a.x = x_codes.data_ptr(); a.ldx = x_codes.stride(0);
  if (bs) {
    need(x_scale, at::kByte, "x_scale"); need(w_scale, at::kByte, "w_scale");
    TORCH_CHECK(x_scale.numel() >= nfb::nvfp4_act_scale_bytes(a.T, a.K), "gemm_quant: activation scale plane too small");
    TORCH_CHECK(w_scale.numel() >= ((a.N + 127) / 128) * (a.K / 64) * 512, "gemm_quant: weight scale plane too small");
  } else {
    need(x_scale, at::kFloat, "x_scale"); need(w_scale, at::kFloat, "w_scale");
    TORCH_CHECK(x_scale.numel() >= a.T && w_scale.numel() >= a.N, "gemm_quant: scale vectors too small");
  }
  a.x_scale = x_scale.data_ptr(); a.w_scale = w_scale.data_ptr();
  a.w_divisor = static_cast<float>(w_divisor);
  TORCH_CHECK(out.size(1) == (epi == nfb::kEpiSwiglu ? a.N / 2 : a.N), "gemm_quant: out width");
  a.out = out.data_ptr(); a.ldo = out.stride(0);
  if (resid.has_value() && resid->defined()) {
    need(*resid, at::kBFloat16, "resid");
    a.resid = resid->data_ptr(); a.ldr = resid->stride(0);
  }
  a.epi = static_cast<int>(epi); a.splits = static_cast<int>(splits);
  a.status = status.has_value() && status->defined() ? static_cast<int*>(status->data_ptr()) : nullptr;
  if (next_codes.has_value() && next_codes->defined()) {
    TORCH_CHECK(next_sf.has_value() && next_sf->defined(), "gemm_quant: next_sf required with next_codes");
    need(*next_codes, at::kByte, "next_codes"); need(*next_sf, at::kByte, "next_sf");
    TORCH_CHECK(next_codes->numel() >= a.T * (a.N / 4) && next_sf->numel() >= nfb::nvfp4_act_scale_bytes(a.T, a.N / 2),
                "gemm_quant: buffers of the fused activation quantiser are too small");
    a.next_codes = next_codes->data_ptr(); a.next_sf = next_sf->data_ptr();
  }
  a.stream = cur_stream(); a.pdl = pdl;
  chk(nfb::gemm_quant(a));
}

// Row-parallel GEMM whose epilogue pushes the scaled fp32 tile into peer memory.  all = true: one-shot all-reduce
// (every rank's [parity][src][T_cap][N] buffer, call counter from `state`); all = false: reduce-scatter into the owner.
void gemm_quant_push(int64_t qtype, const Tensor& x_codes, const Tensor& x_scale, const Tensor& w_codes,
                     const Tensor& w_scale, double w_divisor, bool all, int64_t splits, int64_t world, int64_t rank,
                     at::IntArrayRef peer_bases, int64_t recv_off, int64_t flag_off, int64_t T_cap, const Tensor& state,
                     OptT status, bool pdl) {
  need(x_codes, at::kByte, "x_codes"); need(w_codes, at::kByte, "w_codes"); need(state, at::kByte, "state");
  TORCH_CHECK(x_codes.dim() == 2 && w_codes.dim() == 2 && x_codes.size(1) == w_codes.size(1), "gemm_quant_push: code shapes");
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMaxRanks, "peer_bases size");
  c10::cuda::CUDAGuard guard(x_codes.device());
  nfb::QGemmArgs a;
  a.qtype = static_cast<int>(qtype);
  const bool bs = qtype == nfb::kQNvfp4;
  a.N = w_codes.size(0); a.T = x_codes.size(0); a.K = bs ? w_codes.size(1) * 2 : w_codes.size(1);
  a.w = w_codes.data_ptr(); a.ldw = w_codes.stride(0);
  a.x = x_codes.data_ptr(); a.ldx = x_codes.stride(0);
  a.x_scale = x_scale.data_ptr(); a.w_scale = w_scale.data_ptr();
  a.w_divisor = static_cast<float>(w_divisor);
  a.ldo = 2;
  a.epi = all ? nfb::kEpiPushAll : nfb::kEpiPushPartial;
  a.splits = static_cast<int>(splits);
  a.world = static_cast<int>(world); a.rank = static_cast<int>(rank); a.T_cap = static_cast<int>(T_cap);
  // the call counter is the field `call_idx` of the tensor-parallel state block (comm/comm.h: TpState)
  a.call_idx = reinterpret_cast<const unsigned int*>(static_cast<const char*>(state.data_ptr()) + nfb_tp_call_idx_offset());
  for (int r = 0; r < world; ++r) {
    a.peer_recv[r] = reinterpret_cast<float*>(peer_bases[r] + recv_off);
    a.peer_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + flag_off);
  }
  a.status = status.has_value() && status->defined() ? static_cast<int*>(status->data_ptr()) : nullptr;
  a.stream = cur_stream(); a.pdl = pdl;
  chk(nfb::gemm_quant(a));
}

int64_t nvfp4_act_scale_bytes(int64_t T, int64_t K) { return nfb::nvfp4_act_scale_bytes(T, K); }

}  // namespace

TORCH_LIBRARY_FRAGMENT(nfb200, m) {
  m.def("quant_act_fp8(Tensor x, Tensor codes, Tensor scale, bool pdl=False) -> ()", &quant_act_fp8);
  m.def("quant_act_nvfp4(Tensor x, Tensor codes, Tensor sf_plane, bool pdl=False) -> ()", &quant_act_nvfp4);
  m.def("gemm_quant(int qtype, Tensor x_codes, Tensor x_scale, Tensor w_codes, Tensor w_scale, float w_divisor, Tensor out, int epi, Tensor? resid, int splits, Tensor? status, bool pdl, Tensor? next_codes=None, Tensor? next_sf=None) -> ()", &gemm_quant);
  m.def("nvfp4_act_scale_bytes(int T, int K) -> int", &nvfp4_act_scale_bytes);
  m.def("gemm_quant_push(int qtype, Tensor x_codes, Tensor x_scale, Tensor w_codes, Tensor w_scale, float w_divisor, bool all, int splits, int world, int rank, int[] peer_bases, int recv_off, int flag_off, int T_cap, Tensor state, Tensor? status, bool pdl) -> ()", &gemm_quant_push);
}
