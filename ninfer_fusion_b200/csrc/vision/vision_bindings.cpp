// torch.ops.nfb200.{layer_norm, vision_pos_embed_add, vision_rope, packed_attention}: checked adapters.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "vision.h"

namespace {

using at::Tensor;
using OptT = const std::optional<Tensor>&;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void chk(const char* err) { TORCH_CHECK(err == nullptr, err ? err : ""); }
inline void need(const Tensor& t, at::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
}
inline const __nv_bfloat16* bf(const Tensor& t) { return static_cast<const __nv_bfloat16*>(t.data_ptr()); }
inline __nv_bfloat16* bf_mut(const Tensor& t) { return static_cast<__nv_bfloat16*>(t.data_ptr()); }

void layer_norm(const Tensor& x, const Tensor& w, OptT b, const Tensor& out, double eps) {
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w"); need(out, at::kBFloat16, "out");
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1, "layer_norm: row-major matrices");
  TORCH_CHECK(out.size(0) == x.size(0) && out.size(1) == x.size(1) && w.numel() == x.size(1) && w.is_contiguous(),
              "layer_norm: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::LayerNormParams p = {};
  p.T = static_cast<int>(x.size(0)); p.D = static_cast<int>(x.size(1));
  p.x = bf(x); p.ldx = x.stride(0); p.w = bf(w); p.out = bf_mut(out); p.ldo = out.stride(0);
  if (b.has_value() && b->defined()) {
    need(*b, at::kBFloat16, "b");
    TORCH_CHECK(b->numel() == x.size(1) && b->is_contiguous(), "layer_norm: bias shape");
    p.b = bf(*b);
  }
  p.eps = static_cast<float>(eps);
  chk(nfb::layer_norm(p, cur_stream()));
}

void vision_pos_embed_add(const Tensor& x, const Tensor& table, const Tensor& pos_yx, const Tensor& grid_hw, int64_t side) {
  need(x, at::kBFloat16, "x"); need(table, at::kBFloat16, "table"); need(pos_yx, at::kInt, "pos_yx"); need(grid_hw, at::kInt, "grid_hw");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && table.is_contiguous() && table.dim() == 2 && table.size(0) == side * side &&
              table.size(1) == x.size(1), "vision_pos_embed_add: table shape");
  TORCH_CHECK(pos_yx.is_contiguous() && grid_hw.is_contiguous() && pos_yx.numel() == 2 * x.size(0) &&
              grid_hw.numel() == 2 * x.size(0), "vision_pos_embed_add: position shapes");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::VisionPosEmbedParams p = {};
  p.P = static_cast<int>(x.size(0)); p.D = static_cast<int>(x.size(1)); p.side = static_cast<int>(side);
  p.x = bf_mut(x); p.table = bf(table);
  p.pos_yx = static_cast<const int*>(pos_yx.data_ptr()); p.grid_hw = static_cast<const int*>(grid_hw.data_ptr());
  chk(nfb::vision_pos_embed_add(p, cur_stream()));
}

void vision_rope(const Tensor& qkv, const Tensor& pos_yx, int64_t heads, int64_t head_dim, double theta) {
  need(qkv, at::kBFloat16, "qkv"); need(pos_yx, at::kInt, "pos_yx");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == 3 * heads * head_dim, "vision_rope: qkv shape");
  TORCH_CHECK(pos_yx.is_contiguous() && pos_yx.numel() == 2 * qkv.size(0), "vision_rope: position shape");
  c10::cuda::CUDAGuard guard(qkv.device());
  nfb::VisionRopeParams p = {};
  p.P = static_cast<int>(qkv.size(0)); p.H = static_cast<int>(heads); p.D = static_cast<int>(head_dim);
  p.qkv = bf_mut(qkv); p.ld = qkv.stride(0); p.pos_yx = static_cast<const int*>(pos_yx.data_ptr());
  p.theta = static_cast<float>(theta);
  chk(nfb::vision_rope(p, cur_stream()));
}

void packed_attention(const Tensor& qkv, const Tensor& out, const Tensor& tiles, int64_t heads, double scale) {
  need(qkv, at::kBFloat16, "qkv"); need(out, at::kBFloat16, "out"); need(tiles, at::kInt, "tiles");
  const int64_t hd = heads * nfb::kPackedAttnHeadDim;
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == 3 * hd, "packed_attention: qkv must be [P, 3 * heads * 72]");
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.size(0) == qkv.size(0) && out.size(1) == hd, "packed_attention: out shape");
  TORCH_CHECK(tiles.is_contiguous() && tiles.dim() == 2 && tiles.size(1) == 3, "packed_attention: tiles must be [n, 3]");
  c10::cuda::CUDAGuard guard(qkv.device());
  nfb::PackedAttnParams p = {};
  p.H = static_cast<int>(heads); p.qkv = bf(qkv); p.ld = qkv.stride(0); p.out = bf_mut(out); p.ldo = out.stride(0);
  p.tiles = static_cast<const int*>(tiles.data_ptr()); p.n_tiles = static_cast<int>(tiles.size(0));
  p.scale = static_cast<float>(scale);
  chk(nfb::packed_attention(p, cur_stream()));
}

int64_t packed_attention_tile() { return nfb::kPackedAttnTile; }

}  // namespace

TORCH_LIBRARY_FRAGMENT(nfb200, m) {
  m.def("layer_norm(Tensor x, Tensor w, Tensor? b, Tensor out, float eps) -> ()", &layer_norm);
  m.def("vision_pos_embed_add(Tensor x, Tensor table, Tensor pos_yx, Tensor grid_hw, int side) -> ()", &vision_pos_embed_add);
  m.def("vision_rope(Tensor qkv, Tensor pos_yx, int heads, int head_dim, float theta) -> ()", &vision_rope);
  m.def("packed_attention(Tensor qkv, Tensor out, Tensor tiles, int heads, float scale) -> ()", &packed_attention);
  m.def("packed_attention_tile() -> int", &packed_attention_tile);
}
