// torch.ops.nfb200.moe_* : checked adapters from torch tensors to the mixture-of-experts launchers.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "moe.h"

namespace {

using at::Tensor;
using OptT = const std::optional<Tensor>&;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void chk(const char* err) { TORCH_CHECK(err == nullptr, err ? err : ""); }
inline void need(const Tensor& t, at::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
  TORCH_CHECK(t.is_contiguous() || (t.dim() == 2 && t.stride(1) == 1), name, " must have unit inner stride");
}
template <typename T>
inline T* ptr_or_null(OptT t) {
  return t.has_value() && t->defined() ? static_cast<T*>(t->data_ptr()) : nullptr;
}
inline nfb::MoeState* state_ptr(const Tensor& state) {
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == at::kByte &&
                  state.numel() >= static_cast<int64_t>(sizeof(nfb::MoeState)), "bad MoE state tensor");
  return reinterpret_cast<nfb::MoeState*>(state.data_ptr());
}

void moe_route(const Tensor& logits, int64_t E, int64_t k, bool norm_topk, bool has_shared_gate, const Tensor& hist,
               const Tensor& ids, const Tensor& weights, const Tensor& pos, OptT shared_gate) {
  need(logits, at::kBFloat16, "logits"); need(hist, at::kInt, "hist"); need(ids, at::kInt, "ids");
  need(weights, at::kFloat, "weights"); need(pos, at::kInt, "pos");
  TORCH_CHECK(logits.dim() == 2 && logits.size(1) >= E + (has_shared_gate ? 1 : 0), "logits too narrow");
  const int64_t T = logits.size(0);
  TORCH_CHECK(hist.numel() >= E && ids.numel() >= T * k && weights.numel() >= T * k && pos.numel() >= T * k);
  TORCH_CHECK(ids.is_contiguous() && weights.is_contiguous() && pos.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  nfb::MoeRouteParams p = {};
  p.T = static_cast<int>(T); p.E = static_cast<int>(E); p.k = static_cast<int>(k); p.norm_topk = norm_topk ? 1 : 0;
  p.logits = static_cast<const __nv_bfloat16*>(logits.data_ptr()); p.ld = logits.stride(0);
  p.has_shared_gate = has_shared_gate ? 1 : 0;
  p.hist = static_cast<int*>(hist.data_ptr()); p.ids = static_cast<int*>(ids.data_ptr());
  p.weights = static_cast<float*>(weights.data_ptr()); p.pos = static_cast<int*>(pos.data_ptr());
  if (shared_gate.has_value() && shared_gate->defined()) {
    need(*shared_gate, at::kFloat, "shared_gate");
    TORCH_CHECK(shared_gate->numel() >= T);
    p.shared_gate = static_cast<float*>(shared_gate->data_ptr());
  }
  chk(nfb::moe_route(p, cur_stream()));
}

// tiles: int32 [3, max_tiles] = (local expert, first row, valid rows) per token tile
void moe_plan(int64_t world, int64_t rank, int64_t E, int64_t tile_tokens, int64_t cap, const Tensor& hist,
              at::IntArrayRef peer_bases, int64_t counts_off, int64_t count_flag_off, const Tensor& send_base,
              const Tensor& tiles, const Tensor& state, OptT status) {
  need(hist, at::kInt, "hist"); need(send_base, at::kInt, "send_base"); need(tiles, at::kInt, "tiles");
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMoeMaxRanks, "peer_bases size");
  TORCH_CHECK(tiles.dim() == 2 && tiles.size(0) == 3 && tiles.is_contiguous(), "tiles must be int32 [3, max_tiles]");
  TORCH_CHECK(hist.numel() >= E && send_base.numel() >= E);
  c10::cuda::CUDAGuard guard(hist.device());
  nfb::MoePlanParams p = {};
  p.world = static_cast<int>(world); p.rank = static_cast<int>(rank); p.E = static_cast<int>(E);
  p.tile_tokens = static_cast<int>(tile_tokens); p.cap = static_cast<int>(cap);
  p.max_tiles = static_cast<int>(tiles.size(1));
  p.hist = static_cast<int*>(hist.data_ptr());
  for (int r = 0; r < world; ++r) {
    p.peer_counts[r] = reinterpret_cast<int*>(peer_bases[r] + counts_off);
    p.peer_count_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + count_flag_off);
  }
  p.my_counts = p.peer_counts[rank];
  p.my_count_flag = p.peer_count_flag[rank];
  p.send_base = static_cast<int*>(send_base.data_ptr());
  int* t = static_cast<int*>(tiles.data_ptr());
  p.tile_expert = t; p.tile_row0 = t + p.max_tiles; p.tile_rows = t + 2 * p.max_tiles;
  p.state = state_ptr(state);
  p.status = ptr_or_null<int>(status);
  chk(nfb::moe_plan(p, cur_stream()));
}

void moe_push(int64_t world, int64_t rank, int64_t E, int64_t cap, const Tensor& x, const Tensor& ids,
              const Tensor& pos, const Tensor& send_base, at::IntArrayRef peer_bases, int64_t recv_x_off,
              int64_t recv_meta_off, int64_t arrive_flag_off, const Tensor& state, OptT status) {
  need(x, at::kBFloat16, "x"); need(ids, at::kInt, "ids"); need(pos, at::kInt, "pos"); need(send_base, at::kInt, "send_base");
  TORCH_CHECK(x.dim() == 2 && ids.dim() == 2 && ids.size(0) == x.size(0) && ids.is_contiguous() && pos.is_contiguous());
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMoeMaxRanks, "peer_bases size");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::MoePushParams p = {};
  p.world = static_cast<int>(world); p.rank = static_cast<int>(rank);
  p.T = static_cast<int>(x.size(0)); p.k = static_cast<int>(ids.size(1)); p.H = static_cast<int>(x.size(1));
  p.E = static_cast<int>(E); p.cap = static_cast<int>(cap);
  p.x = static_cast<const __nv_bfloat16*>(x.data_ptr()); p.ldx = x.stride(0);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(p.x) % 16 == 0, "x must be 16-byte aligned");
  p.ids = static_cast<const int*>(ids.data_ptr()); p.pos = static_cast<const int*>(pos.data_ptr());
  p.send_base = static_cast<const int*>(send_base.data_ptr());
  for (int r = 0; r < world; ++r) {
    p.peer_recv_x[r] = reinterpret_cast<__nv_bfloat16*>(peer_bases[r] + recv_x_off);
    p.peer_recv_meta[r] = reinterpret_cast<int*>(peer_bases[r] + recv_meta_off);
    p.peer_arrive_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + arrive_flag_off);
  }
  p.my_arrive_flag = p.peer_arrive_flag[rank];
  p.state = state_ptr(state);
  p.status = ptr_or_null<int>(status);
  chk(nfb::moe_push(p, cur_stream()));
}

// x: [cap, K] expert-sorted rows; w: [local experts, rows per expert, K].
void moe_gemm(const Tensor& x, const Tensor& w, int64_t epi, int64_t tile_tokens, int64_t max_tiles, const Tensor& tiles,
              const Tensor& state, OptT out, int64_t world, OptT recv_meta, at::IntArrayRef peer_bases, int64_t ret_off,
              int64_t ret_flag_off, OptT status) {
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w"); need(tiles, at::kInt, "tiles");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && w.is_contiguous() && x.size(1) == w.size(2), "moe_gemm: shapes");
  TORCH_CHECK(tiles.dim() == 2 && tiles.size(0) == 3 && tiles.is_contiguous() && max_tiles <= tiles.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  nfb::MoeGemmArgs a;
  a.w = w.data_ptr(); a.n_local_experts = static_cast<int>(w.size(0)); a.rows_per_expert = w.size(1);
  a.K = w.size(2); a.ldw = w.size(2);
  a.x = x.data_ptr(); a.cap = x.size(0); a.ldx = x.stride(0);
  a.tile_tokens = static_cast<int>(tile_tokens); a.max_tiles = static_cast<int>(max_tiles);
  const int* t = static_cast<const int*>(tiles.data_ptr());
  const int64_t stride = tiles.size(1);
  a.tile_expert = t; a.tile_row0 = t + stride; a.tile_rows = t + 2 * stride;
  a.state = state_ptr(state);
  a.epi = static_cast<int>(epi);
  if (epi == nfb::kMoeEpiSwiglu) {
    TORCH_CHECK(out.has_value() && out->defined(), "moe_gemm: out required");
    need(*out, at::kBFloat16, "out");
    TORCH_CHECK(out->dim() == 2 && out->size(0) >= x.size(0) && out->size(1) == w.size(1) / 2, "moe_gemm: out shape");
    a.out = out->data_ptr(); a.ldo = out->stride(0);
  } else {
    TORCH_CHECK(recv_meta.has_value() && recv_meta->defined(), "moe_gemm: recv_meta required");
    need(*recv_meta, at::kInt, "recv_meta");
    TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMoeMaxRanks, "peer_bases size");
    a.world = static_cast<int>(world);
    a.recv_meta = static_cast<const int*>(recv_meta->data_ptr());
    for (int r = 0; r < world; ++r) {
      a.peer_ret[r] = reinterpret_cast<__nv_bfloat16*>(peer_bases[r] + ret_off);
      a.peer_ret_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + ret_flag_off);
    }
  }
  a.status = ptr_or_null<int>(status);
  a.stream = cur_stream();
  chk(nfb::moe_gemm(a));
}

// fp8 block-scaled variant: x [cap, K] and w [experts, rows, K] are uint8 e4m3 codes.
void moe_gemm_fp8(const Tensor& x, const Tensor& x_scale, const Tensor& w, const Tensor& w_scale, int64_t epi,
                  int64_t tile_tokens, int64_t max_tiles, const Tensor& tiles, const Tensor& state, OptT out, int64_t world,
                  OptT recv_meta, at::IntArrayRef peer_bases, int64_t ret_off, int64_t ret_flag_off, OptT status) {
  need(x, at::kByte, "x"); need(w, at::kByte, "w"); need(tiles, at::kInt, "tiles");
  need(x_scale, at::kFloat, "x_scale"); need(w_scale, at::kFloat, "w_scale");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && w.is_contiguous() && x.size(1) == w.size(2), "moe_gemm_fp8: shapes");
  TORCH_CHECK(tiles.dim() == 2 && tiles.size(0) == 3 && tiles.is_contiguous() && max_tiles <= tiles.size(1));
  const int64_t nkb = w.size(2) / 128;
  TORCH_CHECK(w_scale.is_contiguous() && w_scale.numel() == w.size(0) * (w.size(1) / 128) * nkb, "moe_gemm_fp8: w_scale shape");
  TORCH_CHECK(x_scale.is_contiguous() && x_scale.numel() >= x.size(0) * nkb, "moe_gemm_fp8: x_scale shape");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::MoeGemmArgs a;
  a.w = w.data_ptr(); a.n_local_experts = static_cast<int>(w.size(0)); a.rows_per_expert = w.size(1);
  a.K = w.size(2); a.ldw = w.size(2);
  a.x = x.data_ptr(); a.cap = x.size(0); a.ldx = x.stride(0);
  a.w_scale = static_cast<const float*>(w_scale.data_ptr()); a.x_scale = static_cast<const float*>(x_scale.data_ptr());
  a.tile_tokens = static_cast<int>(tile_tokens); a.max_tiles = static_cast<int>(max_tiles);
  const int* t = static_cast<const int*>(tiles.data_ptr());
  const int64_t stride = tiles.size(1);
  a.tile_expert = t; a.tile_row0 = t + stride; a.tile_rows = t + 2 * stride;
  a.state = state_ptr(state);
  a.epi = static_cast<int>(epi);
  if (epi == nfb::kMoeEpiSwiglu) {
    TORCH_CHECK(out.has_value() && out->defined(), "moe_gemm_fp8: out required");
    need(*out, at::kBFloat16, "out");
    TORCH_CHECK(out->dim() == 2 && out->size(0) >= x.size(0) && out->size(1) == w.size(1) / 2, "moe_gemm_fp8: out shape");
    a.out = out->data_ptr(); a.ldo = out->stride(0);
  } else {
    TORCH_CHECK(recv_meta.has_value() && recv_meta->defined(), "moe_gemm_fp8: recv_meta required");
    need(*recv_meta, at::kInt, "recv_meta");
    TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMoeMaxRanks, "peer_bases size");
    a.world = static_cast<int>(world);
    a.recv_meta = static_cast<const int*>(recv_meta->data_ptr());
    for (int r = 0; r < world; ++r) {
      a.peer_ret[r] = reinterpret_cast<__nv_bfloat16*>(peer_bases[r] + ret_off);
      a.peer_ret_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + ret_flag_off);
    }
  }
  a.status = ptr_or_null<int>(status);
  a.stream = cur_stream();
  chk(nfb::moe_gemm_fp8(a));
}

void moe_quant_rows_block128(const Tensor& x, const Tensor& codes, const Tensor& scales, OptT state) {
  need(x, at::kBFloat16, "x"); need(codes, at::kByte, "codes"); need(scales, at::kFloat, "scales");
  TORCH_CHECK(x.dim() == 2 && codes.is_contiguous() && codes.numel() >= x.numel() && scales.is_contiguous() &&
              scales.numel() >= x.size(0) * (x.size(1) / 128), "moe_quant_rows_block128: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  const nfb::MoeState* st = state.has_value() && state->defined() ? state_ptr(*state) : nullptr;
  chk(nfb::moe_quant_rows_block128(static_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0), static_cast<int>(x.size(0)),
                                   static_cast<int>(x.size(1)), st, static_cast<uint8_t*>(codes.data_ptr()),
                                   static_cast<float*>(scales.data_ptr()), cur_stream()));
}

void moe_combine(const Tensor& x, const Tensor& weights, const Tensor& ret, int64_t my_base, int64_t ret_flag_off,
                 OptT shared, OptT shared_gate, OptT norm_w, OptT normed, double eps, const Tensor& state, OptT status) {
  need(x, at::kBFloat16, "x"); need(weights, at::kFloat, "weights"); need(ret, at::kBFloat16, "ret");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && weights.dim() == 2 && weights.is_contiguous());
  const int64_t T = x.size(0), H = x.size(1), k = weights.size(1);
  TORCH_CHECK(weights.size(0) >= T && ret.numel() >= T * k * H && ret.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  nfb::MoeCombineParams p = {};
  p.T = static_cast<int>(T); p.k = static_cast<int>(k); p.H = static_cast<int>(H);
  p.arrivals_this_call = static_cast<unsigned int>(T * k * (H / 128));
  p.x = static_cast<__nv_bfloat16*>(x.data_ptr());
  p.weights = static_cast<const float*>(weights.data_ptr());
  p.ret = static_cast<const __nv_bfloat16*>(ret.data_ptr());
  p.ret_flag = reinterpret_cast<const unsigned int*>(my_base + ret_flag_off);
  if (shared.has_value() && shared->defined()) {
    need(*shared, at::kBFloat16, "shared");
    TORCH_CHECK(shared->is_contiguous() && shared->numel() >= T * H && shared_gate.has_value() && shared_gate->defined());
    need(*shared_gate, at::kFloat, "shared_gate");
    p.shared = static_cast<const __nv_bfloat16*>(shared->data_ptr());
    p.shared_gate = static_cast<const float*>(shared_gate->data_ptr());
  }
  if (norm_w.has_value() && norm_w->defined() && normed.has_value() && normed->defined()) {
    need(*norm_w, at::kBFloat16, "norm_w"); need(*normed, at::kBFloat16, "normed");
    TORCH_CHECK(norm_w->numel() == H && normed->is_contiguous() && normed->numel() >= T * H);
    p.norm_w = static_cast<const __nv_bfloat16*>(norm_w->data_ptr());
    p.normed = static_cast<__nv_bfloat16*>(normed->data_ptr());
  }
  p.eps = static_cast<float>(eps);
  p.state = state_ptr(state);
  p.status = ptr_or_null<int>(status);
  chk(nfb::moe_combine(p, cur_stream()));
}

int64_t moe_state_bytes() { return static_cast<int64_t>(sizeof(nfb::MoeState)); }
int64_t moe_tile_tokens(double rows_per_expert) { return nfb::moe_tile_tokens(rows_per_expert); }
int64_t moe_push_ctas() { return nfb::kMoePushCtas; }

}  // namespace

TORCH_LIBRARY_FRAGMENT(nfb200, m) {
  m.def("moe_route(Tensor logits, int E, int k, bool norm_topk, bool has_shared_gate, Tensor hist, Tensor ids, Tensor weights, Tensor pos, Tensor? shared_gate) -> ()", &moe_route);
  m.def("moe_plan(int world, int rank, int E, int tile_tokens, int cap, Tensor hist, int[] peer_bases, int counts_off, int count_flag_off, Tensor send_base, Tensor tiles, Tensor state, Tensor? status) -> ()", &moe_plan);
  m.def("moe_push(int world, int rank, int E, int cap, Tensor x, Tensor ids, Tensor pos, Tensor send_base, int[] peer_bases, int recv_x_off, int recv_meta_off, int arrive_flag_off, Tensor state, Tensor? status) -> ()", &moe_push);
  m.def("moe_gemm(Tensor x, Tensor w, int epi, int tile_tokens, int max_tiles, Tensor tiles, Tensor state, Tensor? out, int world, Tensor? recv_meta, int[] peer_bases, int ret_off, int ret_flag_off, Tensor? status) -> ()", &moe_gemm);
  m.def("moe_gemm_fp8(Tensor x, Tensor x_scale, Tensor w, Tensor w_scale, int epi, int tile_tokens, int max_tiles, Tensor tiles, Tensor state, Tensor? out, int world, Tensor? recv_meta, int[] peer_bases, int ret_off, int ret_flag_off, Tensor? status) -> ()", &moe_gemm_fp8);
  m.def("moe_quant_rows_block128(Tensor x, Tensor codes, Tensor scales, Tensor? state) -> ()", &moe_quant_rows_block128);
  m.def("moe_combine(Tensor x, Tensor weights, Tensor ret, int my_base, int ret_flag_off, Tensor? shared, Tensor? shared_gate, Tensor? norm_w, Tensor? normed, float eps, Tensor state, Tensor? status) -> ()", &moe_combine);
  m.def("moe_state_bytes() -> int", &moe_state_bytes);
  m.def("moe_tile_tokens(float rows_per_expert) -> int", &moe_tile_tokens);
  m.def("moe_push_ctas() -> int", &moe_push_ctas);
}
