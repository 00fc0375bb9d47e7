// torch.ops.nfb200.* : thin, checked adapters from torch tensors to the plain
// C++ launchers.  No kernel code lives here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <ATen/ATen.h>

#include "attention/attention.h"
#include "comm/comm.h"
#include "gdn/gdn.h"
#include "gemm/gemm.h"
#include "pointwise/pointwise.h"
#include "sampling/sampling.h"

namespace {

using at::Tensor;
using OptT = const std::optional<Tensor>&;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void chk(const char* err) { TORCH_CHECK(err == nullptr, err ? err : ""); }

inline void need_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}
inline void need(const Tensor& t, at::ScalarType dt, const char* name) {
  need_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
}
inline void need_rows(const Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with unit inner stride");
}
template <typename T>
inline T* ptr_or_null(OptT t) {
  return t.has_value() && t->defined() ? static_cast<T*>(t->data_ptr()) : nullptr;
}

int64_t sm_count() {
  static int n = 0;
  if (n == 0) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

// Optional L2 prefetch hint: a (contiguous) tensor the next kernel will stream; at most the first 32 MB are asked for.
void fill_prefetch(nfb::GemmArgs& a, OptT next) {
  if (!(next.has_value() && next->defined() && next->is_cuda() && next->is_contiguous())) return;
  a.prefetch = next->data_ptr();
  const int64_t bytes = next->numel() * next->element_size();
  a.prefetch_bytes = bytes < (32 << 20) ? bytes : (32 << 20);
}

// Optional decode conv epilogue (nfb::GemmConv): all four tensors or none.
void fill_conv(nfb::GemmArgs& a, OptT conv_w, OptT conv_state, OptT conv_slot, OptT conv_out) {
  if (!(conv_state.has_value() && conv_state->defined())) return;
  TORCH_CHECK(conv_w.has_value() && conv_slot.has_value() && conv_out.has_value(), "conv epilogue: all four tensors");
  need(*conv_w, at::kBFloat16, "conv_w"); need(*conv_state, at::kBFloat16, "conv_state");
  need(*conv_slot, at::kInt, "conv_slot"); need(*conv_out, at::kBFloat16, "conv_out");
  TORCH_CHECK(conv_w->dim() == 2 && conv_w->size(1) == 4 && conv_w->is_contiguous(), "conv_w must be [C, 4]");
  const int64_t C = conv_w->size(0);
  TORCH_CHECK(conv_state->dim() == 3 && conv_state->size(1) == 3 && conv_state->size(2) == C && conv_state->is_contiguous(),
              "conv_state must be [slots, 3, C]");
  TORCH_CHECK(conv_out->dim() == 2 && conv_out->size(0) == a.T && conv_out->size(1) == C && conv_out->is_contiguous(),
              "conv_out must be [T, C]");
  TORCH_CHECK(conv_slot->numel() >= a.T && conv_slot->is_contiguous(), "conv_slot must hold one slot per token");
  a.conv.w = conv_w->data_ptr(); a.conv.state = conv_state->data_ptr();
  a.conv.slot = static_cast<const int*>(conv_slot->data_ptr()); a.conv.out = conv_out->data_ptr();
  a.conv.C = static_cast<int>(C);
}

// out = epilogue(x @ w^T).  epi: 0 store(+bias), 1 residual add, 2 swiglu, 3 split-K partials.
void gemm_bf16(const Tensor& x, const Tensor& w, OptT out, int64_t epi, OptT resid, OptT bias, OptT partial,
               int64_t splits, OptT status, bool pdl, int64_t act, OptT conv_w, OptT conv_state, OptT conv_slot,
               OptT conv_out, OptT prefetch) {
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w");
  need_rows(x, "x"); need_rows(w, "w");
  TORCH_CHECK(x.size(1) == w.size(1), "gemm_bf16: K mismatch");
  TORCH_CHECK(act >= 0 && act <= 2 && (act == 0 || epi == nfb::kEpiStore), "gemm_bf16: activation needs the store epilogue");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::GemmArgs a;
  a.w = w.data_ptr(); a.N = w.size(0); a.K = w.size(1); a.ldw = w.stride(0);
  a.x = x.data_ptr(); a.T = x.size(0); a.ldx = x.stride(0);
  const int64_t out_cols = epi == nfb::kEpiSwiglu ? a.N / 2 : a.N;
  if (epi != nfb::kEpiPartial) {
    TORCH_CHECK(out.has_value(), "gemm_bf16: out required");
    need(*out, at::kBFloat16, "out"); need_rows(*out, "out");
    TORCH_CHECK(out->size(0) == a.T && out->size(1) == out_cols, "gemm_bf16: out shape");
    a.out = out->data_ptr(); a.ldo = out->stride(0);
  }
  if (epi == nfb::kEpiResidual) {
    TORCH_CHECK(resid.has_value(), "gemm_bf16: resid required");
    need(*resid, at::kBFloat16, "resid"); need_rows(*resid, "resid");
    TORCH_CHECK(resid->size(0) == a.T && resid->size(1) == a.N, "gemm_bf16: resid shape");
    a.resid = resid->data_ptr(); a.ldr = resid->stride(0);
  }
  if (bias.has_value() && bias->defined()) {
    need(*bias, at::kFloat, "bias");
    TORCH_CHECK(bias->numel() == a.N && bias->is_contiguous(), "gemm_bf16: bias shape");
    a.bias = static_cast<const float*>(bias->data_ptr());
  }
  if (epi == nfb::kEpiPartial) {
    TORCH_CHECK(partial.has_value(), "gemm_bf16: partial workspace required");
    need(*partial, at::kFloat, "partial");
    TORCH_CHECK(partial->is_contiguous() && partial->numel() >= splits * a.T * a.N, "gemm_bf16: workspace too small");
    a.partial = static_cast<float*>(partial->data_ptr());
  }
  a.splits = static_cast<int>(splits); a.epi = static_cast<int>(epi); a.act = static_cast<int>(act);
  a.status = ptr_or_null<int>(status);
  a.stream = cur_stream(); a.pdl = pdl;
  fill_conv(a, conv_w, conv_state, conv_slot, conv_out);
  fill_prefetch(a, prefetch);
  chk(nfb::gemm_bf16(a));
}

Tensor gemm_trace(bool enable, int64_t n_ctas) {
  nfb::gemm_trace_enable(enable);
  Tensor out = at::zeros({n_ctas, 12}, at::TensorOptions().dtype(at::kLong));
  if (n_ctas > 0) nfb::gemm_trace_read(reinterpret_cast<unsigned long long*>(out.data_ptr()), static_cast<int>(n_ctas));
  return out;
}

// mode 1: start a multi-launch timeline; mode 0: stop and return (launches seen, stamps [64, 256, 12] int64 ns)
std::tuple<int64_t, Tensor> gemm_timeline(int64_t mode) {
  if (mode == 1) {
    nfb::gemm_timeline_begin();
    return {0, at::zeros({0}, at::TensorOptions().dtype(at::kLong))};
  }
  Tensor out = at::zeros({64, 256, 12}, at::TensorOptions().dtype(at::kLong));
  int slots = 0, ctas = 0;
  const int used = nfb::gemm_timeline_end(reinterpret_cast<unsigned long long*>(out.data_ptr()), &slots, &ctas);
  TORCH_CHECK(slots == 64 && ctas == 256, "timeline geometry changed");
  return {used, out};
}

int64_t gemm_pick_splits(int64_t T, int64_t N, int64_t K, int64_t epi) {
  return nfb::gemm_pick_splits(static_cast<int>(T), static_cast<int>(N), static_cast<int>(K), static_cast<int>(epi),
                               static_cast<int>(sm_count()));
}

void add_rmsnorm(OptT partial, int64_t splits, OptT delta, OptT resid_in, OptT resid_out, OptT norm_w, OptT normed,
                 int64_t T, int64_t N, double eps, bool unit_offset, bool pdl, OptT q_codes, OptT q_sf) {
  auto dev_of = [&]() -> const Tensor& {
    if (resid_in.has_value() && resid_in->defined()) return *resid_in;
    if (delta.has_value() && delta->defined()) return *delta;
    TORCH_CHECK(partial.has_value() && partial->defined(), "add_rmsnorm: no input");
    return *partial;
  };
  c10::cuda::CUDAGuard guard(dev_of().device());
  for (OptT t : {delta, resid_in, resid_out, normed}) {
    if (t.has_value() && t->defined()) {
      need(*t, at::kBFloat16, "add_rmsnorm tensor");
      TORCH_CHECK(t->is_contiguous() && t->numel() == T * N, "add_rmsnorm: tensors must be contiguous [T, N]");
    }
  }
  if (partial.has_value() && partial->defined()) {
    need(*partial, at::kFloat, "partial");
    TORCH_CHECK(partial->is_contiguous() && partial->numel() >= splits * T * N, "add_rmsnorm: partial too small");
  }
  if (norm_w.has_value() && norm_w->defined()) {
    need(*norm_w, at::kBFloat16, "norm_w");
    TORCH_CHECK(norm_w->numel() == N, "add_rmsnorm: norm_w shape");
  }
  if (q_codes.has_value() && q_codes->defined()) {
    TORCH_CHECK(q_sf.has_value() && q_sf->defined(), "add_rmsnorm: q_codes without q_sf");
    need(*q_codes, at::kByte, "q_codes"); need(*q_sf, at::kByte, "q_sf");
    TORCH_CHECK(q_codes->is_contiguous() && q_codes->numel() >= T * N / 2, "add_rmsnorm: q_codes too small");
    TORCH_CHECK(q_sf->numel() >= ((T + 255) / 256) * 2 * (N / 64) * 512, "add_rmsnorm: q_sf too small");
  }
  chk(nfb::add_rmsnorm(ptr_or_null<float>(partial), static_cast<int>(splits), ptr_or_null<void>(delta),
                       ptr_or_null<void>(resid_in), ptr_or_null<void>(resid_out), ptr_or_null<void>(norm_w),
                       ptr_or_null<void>(normed), static_cast<int>(T), static_cast<int>(N), static_cast<float>(eps),
                       unit_offset ? 1 : 0, cur_stream(), pdl, ptr_or_null<uint8_t>(q_codes), ptr_or_null<uint8_t>(q_sf)));
}

Tensor gdn_prefill_trace(bool enable) {
  Tensor t = at::zeros({5}, at::kLong);
  c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, at::cuda::current_device()));
  nfb::gdn_prefill_trace(enable, reinterpret_cast<long long*>(t.data_ptr<int64_t>()));
  return t;
}

void embed_gather(const Tensor& ids, const Tensor& table, const Tensor& out, bool pdl) {
  need(ids, at::kInt, "ids"); need(table, at::kBFloat16, "table"); need(out, at::kBFloat16, "out");
  TORCH_CHECK(table.is_contiguous() && out.is_contiguous() && ids.is_contiguous());
  TORCH_CHECK(out.size(0) == ids.numel() && out.size(1) == table.size(1));
  c10::cuda::CUDAGuard guard(ids.device());
  chk(nfb::embed_gather(static_cast<const int*>(ids.data_ptr()), table.data_ptr(), out.data_ptr(),
                        static_cast<int>(ids.numel()), static_cast<int>(table.size(1)),
                        static_cast<int>(table.size(0)), cur_stream(), pdl));
}

// `tiers` (mixed layers, format 4): CPU int64 tensor of 13 device addresses
// [cell_map, then per tier 0..2: k_codes, v_codes, k_scales, v_scales] (0 = none); the caller keeps the tensors alive.
nfb::KvLayer make_kv(const Tensor& k_codes, const Tensor& v_codes, OptT k_scales, OptT v_scales, int64_t page_size,
                     int64_t n_kv_heads, int64_t head_dim, int64_t format, int64_t group, OptT tiers = std::nullopt) {
  need(k_codes, at::kByte, "k_codes"); need(v_codes, at::kByte, "v_codes");
  TORCH_CHECK(k_codes.is_contiguous() && v_codes.is_contiguous());
  nfb::KvLayer kv;
  if (format == nfb::kKvMixed) {
    TORCH_CHECK(tiers.has_value() && tiers->defined() && !tiers->is_cuda() && tiers->scalar_type() == at::kLong &&
                tiers->numel() == 1 + 4 * nfb::kKvTiers && tiers->is_contiguous(), "mixed KV layer needs its tier descriptor");
    const int64_t* d = tiers->data_ptr<int64_t>();
    TORCH_CHECK(d[0] != 0, "mixed KV layer without a cell map");
    kv.cell_map = reinterpret_cast<const int*>(d[0]);
    for (int t = 0; t < nfb::kKvTiers; ++t) {
      kv.tier_k_codes[t] = reinterpret_cast<uint8_t*>(d[1 + 4 * t]);
      kv.tier_v_codes[t] = reinterpret_cast<uint8_t*>(d[2 + 4 * t]);
      kv.tier_k_scales[t] = reinterpret_cast<uint8_t*>(d[3 + 4 * t]);
      kv.tier_v_scales[t] = reinterpret_cast<uint8_t*>(d[4 + 4 * t]);
      TORCH_CHECK(kv.tier_k_codes[t] != nullptr && kv.tier_v_codes[t] != nullptr, "mixed KV layer: a tier has no planes");
    }
    TORCH_CHECK(kv.tier_k_scales[1] && kv.tier_v_scales[1] && kv.tier_k_scales[2] && kv.tier_v_scales[2],
                "mixed KV layer: the fp8 and nvfp4 tiers need scale planes");
    TORCH_CHECK(head_dim == 256, "mixed KV layers need head_dim 256");
    kv.k_codes = static_cast<uint8_t*>(k_codes.data_ptr());
    kv.v_codes = static_cast<uint8_t*>(v_codes.data_ptr());
    kv.k_scales = kv.v_scales = nullptr;
    kv.page_size = static_cast<int>(page_size);
    kv.n_kv_heads = static_cast<int>(n_kv_heads);
    kv.head_dim = static_cast<int>(head_dim);
    kv.format = nfb::kKvMixed;
    kv.group = static_cast<int>(head_dim);
    return kv;
  }
  kv.k_codes = static_cast<uint8_t*>(k_codes.data_ptr());
  kv.v_codes = static_cast<uint8_t*>(v_codes.data_ptr());
  kv.k_scales = ptr_or_null<uint8_t>(k_scales);
  kv.v_scales = ptr_or_null<uint8_t>(v_scales);
  kv.page_size = static_cast<int>(page_size);
  kv.n_kv_heads = static_cast<int>(n_kv_heads);
  kv.head_dim = static_cast<int>(head_dim);
  kv.format = static_cast<int>(format);
  kv.group = static_cast<int>(group);
  const int64_t rb = nfb::kv_row_bytes(kv.format, kv.head_dim);
  TORCH_CHECK(k_codes.numel() % (n_kv_heads * page_size * rb) == 0, "kv codes size is not a whole number of pages");
  if (nfb::kv_scale_bytes(kv.format, kv.head_dim, kv.group) > 0)
    TORCH_CHECK(kv.k_scales != nullptr && kv.v_scales != nullptr, "this KV format needs scale planes");
  return kv;
}

// Moves K/V rows of each sequence from cache positions src_pos[b, m] to dst_pos[b, m] (in order m = 0.., -1 = skip).
void kv_move_rows(const Tensor& block_table, const Tensor& table_row, const Tensor& src_pos, const Tensor& dst_pos,
                  const Tensor& k_codes, const Tensor& v_codes, OptT k_scales, OptT v_scales, int64_t page_size,
                  int64_t n_kv_heads, int64_t head_dim, int64_t format, int64_t group) {
  need(block_table, at::kInt, "block_table"); need(table_row, at::kInt, "table_row");
  need(src_pos, at::kInt, "src_pos"); need(dst_pos, at::kInt, "dst_pos");
  TORCH_CHECK(src_pos.dim() == 2 && src_pos.is_contiguous() && dst_pos.is_contiguous() && src_pos.sizes() == dst_pos.sizes() &&
              src_pos.size(0) == table_row.numel() && block_table.dim() == 2 && block_table.is_contiguous(), "kv_move_rows: shapes");
  c10::cuda::CUDAGuard guard(k_codes.device());
  nfb::KvLayer kv = make_kv(k_codes, v_codes, k_scales, v_scales, page_size, n_kv_heads, head_dim, format, group);
  chk(nfb::kv_move_rows(kv, static_cast<const int*>(block_table.data_ptr()), static_cast<int>(block_table.size(1)),
                        static_cast<const int*>(table_row.data_ptr()), static_cast<const int*>(src_pos.data_ptr()),
                        static_cast<const int*>(dst_pos.data_ptr()), static_cast<int>(src_pos.size(0)),
                        static_cast<int>(src_pos.size(1)), cur_stream()));
}

// Re-encodes cells of a mixed-precision KV layer into another tier.  `anchor`: any device tensor of the layer (device
// guard); `src_cell` / `dst_cell`: int32 device arrays of tier << 28 | slot.
void kv_requant(const Tensor& tiers, const Tensor& anchor, const Tensor& src_cell, const Tensor& dst_cell,
                int64_t page_size, int64_t n_kv_heads, int64_t head_dim) {
  need(anchor, at::kByte, "anchor"); need(src_cell, at::kInt, "src_cell"); need(dst_cell, at::kInt, "dst_cell");
  TORCH_CHECK(src_cell.is_contiguous() && dst_cell.is_contiguous() && src_cell.numel() == dst_cell.numel(), "cell lists");
  c10::cuda::CUDAGuard guard(anchor.device());
  nfb::KvRequantParams p = {};
  p.kv = make_kv(anchor, anchor, std::nullopt, std::nullopt, page_size, n_kv_heads, head_dim, nfb::kKvMixed, head_dim, tiers);
  p.src_cell = static_cast<const int*>(src_cell.data_ptr());
  p.dst_cell = static_cast<const int*>(dst_cell.data_ptr());
  p.n_cells = static_cast<int>(src_cell.numel());
  chk(nfb::kv_requant(p, cur_stream()));
}

void attn_prep(const Tensor& proj, int64_t q_off, int64_t k_off, int64_t v_off, int64_t n_q_heads,
               int64_t n_kv_heads, int64_t head_dim, OptT q_norm_w, OptT k_norm_w, double eps, bool unit_offset,
               int64_t rot_dim, const Tensor& inv_freq, double attn_factor, const Tensor& rope_pos,
               const Tensor& token_seq, const Tensor& cache_pos, const Tensor& block_table, const Tensor& q_out,
               const Tensor& k_codes, const Tensor& v_codes, OptT k_scales, OptT v_scales, int64_t page_size,
               int64_t format, int64_t group, bool pdl, bool k_hadamard, OptT k_row_scale, OptT tiers) {
  need(proj, at::kBFloat16, "proj"); need_rows(proj, "proj");
  need(inv_freq, at::kFloat, "inv_freq"); need(rope_pos, at::kInt, "rope_pos");
  need(token_seq, at::kInt, "token_seq"); need(cache_pos, at::kInt, "cache_pos");
  need(block_table, at::kInt, "block_table"); need(q_out, at::kBFloat16, "q_out");
  TORCH_CHECK(block_table.dim() == 2 && block_table.is_contiguous() && q_out.is_contiguous() && rope_pos.is_contiguous());
  c10::cuda::CUDAGuard guard(proj.device());
  nfb::AttnPrepParams p = {};
  p.proj = static_cast<const __nv_bfloat16*>(proj.data_ptr());
  p.ld_proj = proj.stride(0);
  p.q_off = static_cast<int>(q_off); p.k_off = static_cast<int>(k_off); p.v_off = static_cast<int>(v_off);
  p.T = static_cast<int>(proj.size(0));
  p.n_q_heads = static_cast<int>(n_q_heads); p.n_kv_heads = static_cast<int>(n_kv_heads);
  p.head_dim = static_cast<int>(head_dim);
  p.q_norm_w = ptr_or_null<const __nv_bfloat16>(q_norm_w);
  p.k_norm_w = ptr_or_null<const __nv_bfloat16>(k_norm_w);
  p.eps = static_cast<float>(eps); p.unit_offset = unit_offset ? 1 : 0;
  p.rot_dim = static_cast<int>(rot_dim);
  TORCH_CHECK(inv_freq.numel() >= rot_dim / 2, "inv_freq too short");
  p.inv_freq = static_cast<const float*>(inv_freq.data_ptr());
  p.rope_attn_factor = static_cast<float>(attn_factor);
  p.rope_pos = static_cast<const int*>(rope_pos.data_ptr());
  p.pos_axes = rope_pos.dim() == 2 ? static_cast<int>(rope_pos.size(1)) : 1;
  TORCH_CHECK(p.pos_axes == 1 || p.pos_axes == 3, "rope_pos must be [T] or [T, 3]");
  TORCH_CHECK(rope_pos.numel() == static_cast<int64_t>(p.T) * p.pos_axes && token_seq.numel() == p.T &&
              cache_pos.numel() == p.T, "per-token arrays must have T entries");
  p.token_seq = static_cast<const int*>(token_seq.data_ptr());
  p.cache_pos = static_cast<const int*>(cache_pos.data_ptr());
  p.block_table = static_cast<const int*>(block_table.data_ptr());
  p.table_stride = static_cast<int>(block_table.size(1));
  TORCH_CHECK(q_out.numel() == static_cast<int64_t>(p.T) * n_q_heads * head_dim, "q_out shape");
  p.q_out = static_cast<__nv_bfloat16*>(q_out.data_ptr());
  p.kv = make_kv(k_codes, v_codes, k_scales, v_scales, page_size, n_kv_heads, head_dim, format, group, tiers);
  p.k_hadamard = k_hadamard ? 1 : 0;
  if (k_row_scale.has_value() && k_row_scale->defined()) {
    need(*k_row_scale, at::kBFloat16, "k_row_scale");
    TORCH_CHECK(k_row_scale->is_contiguous() && k_row_scale->numel() == n_kv_heads * head_dim,
                "k_row_scale must be a contiguous [n_kv_heads, head_dim] table");
    p.k_row_scale = static_cast<const __nv_bfloat16*>(k_row_scale->data_ptr());
  }
  chk(nfb::attn_prep(p, cur_stream(), pdl));
}

void paged_attention(const Tensor& q, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim, const Tensor& q_seq,
                     const Tensor& q_kv_len, const Tensor& block_table, const Tensor& k_codes, const Tensor& v_codes,
                     OptT k_scales, OptT v_scales, int64_t page_size, int64_t format, int64_t group, double sm_scale,
                     int64_t split_keys, int64_t n_splits, const Tensor& part_o, const Tensor& part_ml, OptT gate,
                     const Tensor& out, OptT tree_mask, OptT tree_base, int64_t impl, bool pdl, int64_t window,
                     OptT sel_blocks, OptT sel_count, OptT tiers, OptT q_codes, OptT q_sf) {
  need(q, at::kBFloat16, "q"); need(q_seq, at::kInt, "q_seq"); need(q_kv_len, at::kInt, "q_kv_len");
  need(block_table, at::kInt, "block_table"); need(part_o, at::kFloat, "part_o"); need(part_ml, at::kFloat, "part_ml");
  need(out, at::kBFloat16, "out");
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous() && block_table.dim() == 2 && block_table.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  nfb::PagedAttnParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q.data_ptr());
  p.Tq = static_cast<int>(q.numel() / (n_q_heads * head_dim));
  p.n_q_heads = static_cast<int>(n_q_heads); p.n_kv_heads = static_cast<int>(n_kv_heads);
  p.head_dim = static_cast<int>(head_dim);
  TORCH_CHECK(q_seq.numel() == p.Tq && q_kv_len.numel() == p.Tq, "per-query arrays must have Tq entries");
  p.q_seq = static_cast<const int*>(q_seq.data_ptr());
  p.q_kv_len = static_cast<const int*>(q_kv_len.data_ptr());
  p.block_table = static_cast<const int*>(block_table.data_ptr());
  p.table_stride = static_cast<int>(block_table.size(1));
  p.kv = make_kv(k_codes, v_codes, k_scales, v_scales, page_size, n_kv_heads, head_dim, format, group, tiers);
  p.sm_scale = static_cast<float>(sm_scale);
  p.split_keys = static_cast<int>(split_keys); p.n_splits = static_cast<int>(n_splits);
  TORCH_CHECK(part_o.numel() >= static_cast<int64_t>(p.Tq) * n_q_heads * n_splits * head_dim, "part_o too small");
  TORCH_CHECK(part_ml.numel() >= static_cast<int64_t>(p.Tq) * n_q_heads * n_splits * 2, "part_ml too small");
  p.part_o = static_cast<float*>(part_o.data_ptr());
  p.part_ml = static_cast<float*>(part_ml.data_ptr());
  if (gate.has_value() && gate->defined()) {
    need(*gate, at::kBFloat16, "gate"); need_rows(*gate, "gate");
    p.gate = static_cast<const __nv_bfloat16*>(gate->data_ptr());
    p.ld_gate = gate->stride(0);
  }
  TORCH_CHECK(out.numel() == static_cast<int64_t>(p.Tq) * n_q_heads * head_dim, "out shape");
  p.out = static_cast<__nv_bfloat16*>(out.data_ptr());
  if (tree_mask.has_value() && tree_mask->defined()) {
    need(*tree_mask, at::kLong, "tree_mask");
    TORCH_CHECK(tree_base.has_value(), "tree_base required with tree_mask");
    need(*tree_base, at::kInt, "tree_base");
    p.tree_mask = static_cast<const unsigned long long*>(tree_mask->data_ptr());
    p.tree_base = static_cast<const int*>(tree_base->data_ptr());
  }
  p.impl = static_cast<int>(impl);
  if (format == nfb::kKvFp8Row) p.kv_plane_rows = k_codes.numel() / head_dim;
  TORCH_CHECK(window >= 0, "window must be >= 0");
  p.window = static_cast<int>(window);
  if (sel_blocks.has_value() && sel_blocks->defined()) {
    TORCH_CHECK(sel_count.has_value() && sel_count->defined(), "sel_count required with sel_blocks");
    need(*sel_blocks, at::kInt, "sel_blocks"); need(*sel_count, at::kInt, "sel_count");
    TORCH_CHECK(sel_blocks->dim() == 2 && sel_blocks->is_contiguous() && sel_blocks->size(0) == p.Tq &&
                sel_count->numel() == p.Tq, "selection: sel_blocks [Tq, max_blocks], sel_count [Tq]");
    p.sel_blocks = static_cast<const int*>(sel_blocks->data_ptr());
    p.sel_count = static_cast<const int*>(sel_count->data_ptr());
    p.sel_stride = static_cast<int>(sel_blocks->size(1));
  }
  if (q_codes.has_value() && q_codes->defined()) {
    TORCH_CHECK(q_sf.has_value() && q_sf->defined(), "q_sf required with q_codes");
    need(*q_codes, at::kByte, "q_codes"); need(*q_sf, at::kByte, "q_sf");
    TORCH_CHECK(q_codes->numel() >= static_cast<int64_t>(p.Tq) * n_q_heads * head_dim / 2 && head_dim % 16 == 0,
                "q_codes too small");
    p.q_codes = static_cast<uint8_t*>(q_codes->data_ptr());
    p.q_sf = static_cast<uint8_t*>(q_sf->data_ptr());
  }
  chk(nfb::paged_attention(p, cur_stream(), pdl));
}

// Development aid: returns the event trace of CTA 0 of the tcgen05 attention kernel and switches tracing on / off.
Tensor attn_tc_trace(bool enable) {
  Tensor out = at::zeros({5, 1024}, at::TensorOptions().dtype(at::kLong));
  nfb::paged_attention_tc_trace(enable, reinterpret_cast<unsigned long long*>(out.data_ptr()));
  return out;
}

void paged_attention_prefill(const Tensor& q, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim,
                             const Tensor& q_seq, const Tensor& q_kv_len, const Tensor& blk_start,
                             const Tensor& blk_count, const Tensor& block_table, const Tensor& k_codes,
                             const Tensor& v_codes, OptT k_scales, OptT v_scales, int64_t page_size, int64_t format,
                             int64_t group, double sm_scale, OptT gate, const Tensor& out, bool pdl, int64_t window,
                             OptT tiers) {
  need(q, at::kBFloat16, "q"); need(q_seq, at::kInt, "q_seq"); need(q_kv_len, at::kInt, "q_kv_len");
  need(blk_start, at::kInt, "blk_start"); need(blk_count, at::kInt, "blk_count");
  need(block_table, at::kInt, "block_table"); need(out, at::kBFloat16, "out");
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous() && block_table.dim() == 2 && block_table.is_contiguous());
  TORCH_CHECK(blk_start.numel() == blk_count.numel(), "block descriptor sizes");
  c10::cuda::CUDAGuard guard(q.device());
  nfb::PrefillAttnParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q.data_ptr());
  p.n_q_heads = static_cast<int>(n_q_heads); p.n_kv_heads = static_cast<int>(n_kv_heads);
  p.head_dim = static_cast<int>(head_dim);
  const int64_t T = q.numel() / (n_q_heads * head_dim);
  TORCH_CHECK(q_seq.numel() == T && q_kv_len.numel() == T && out.numel() == q.numel(), "per-token array sizes");
  p.q_seq = static_cast<const int*>(q_seq.data_ptr());
  p.q_kv_len = static_cast<const int*>(q_kv_len.data_ptr());
  p.blk_start = static_cast<const int*>(blk_start.data_ptr());
  p.blk_count = static_cast<const int*>(blk_count.data_ptr());
  p.n_blocks = static_cast<int>(blk_start.numel());
  p.block_table = static_cast<const int*>(block_table.data_ptr());
  p.table_stride = static_cast<int>(block_table.size(1));
  p.kv = make_kv(k_codes, v_codes, k_scales, v_scales, page_size, n_kv_heads, head_dim, format, group, tiers);
  p.sm_scale = static_cast<float>(sm_scale);
  if (gate.has_value() && gate->defined()) {
    need(*gate, at::kBFloat16, "gate"); need_rows(*gate, "gate");
    p.gate = static_cast<const __nv_bfloat16*>(gate->data_ptr());
    p.ld_gate = gate->stride(0);
  }
  p.out = static_cast<__nv_bfloat16*>(out.data_ptr());
  TORCH_CHECK(window >= 0, "window must be >= 0");
  p.window = static_cast<int>(window);
  chk(nfb::paged_attention_prefill(p, cur_stream(), pdl));
}

int64_t prefill_attn_block_tokens(int64_t n_q_heads, int64_t n_kv_heads) {
  return nfb::prefill_attn_block_tokens(static_cast<int>(n_q_heads), static_cast<int>(n_kv_heads));
}

void causal_conv1d_silu(const Tensor& x, int64_t c_off, int64_t C, const Tensor& w, const Tensor& cu_seqlens,
                        const Tensor& token_seq, const Tensor& state_slot, const Tensor& conv_state,
                        const Tensor& out, bool update_state, bool one_token_per_seq, bool pdl, OptT seq_end,
                        bool state_only, OptT parent, OptT last_token) {
  need(x, at::kBFloat16, "x"); need_rows(x, "x"); need(w, at::kBFloat16, "w");
  need(cu_seqlens, at::kInt, "cu_seqlens"); need(token_seq, at::kInt, "token_seq");
  need(state_slot, at::kInt, "state_slot"); need(conv_state, at::kBFloat16, "conv_state");
  need(out, at::kBFloat16, "out");
  TORCH_CHECK(w.is_contiguous() && w.numel() == C * 4 && conv_state.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(conv_state.dim() == 3 && conv_state.size(1) == 3 && conv_state.size(2) == C, "conv_state [slots,3,C]");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::ConvParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x.data_ptr()); p.ld_x = x.stride(0);
  p.c_off = static_cast<int>(c_off); p.C = static_cast<int>(C); p.T = static_cast<int>(x.size(0));
  p.n_seq = static_cast<int>(state_slot.numel());
  TORCH_CHECK(cu_seqlens.numel() == p.n_seq + 1 && token_seq.numel() == p.T);
  TORCH_CHECK(out.numel() == static_cast<int64_t>(p.T) * C, "conv out shape");
  p.w = static_cast<const __nv_bfloat16*>(w.data_ptr());
  p.cu_seqlens = static_cast<const int*>(cu_seqlens.data_ptr());
  p.token_seq = static_cast<const int*>(token_seq.data_ptr());
  p.state_slot = static_cast<const int*>(state_slot.data_ptr());
  p.conv_state = static_cast<__nv_bfloat16*>(conv_state.data_ptr());
  p.out = static_cast<__nv_bfloat16*>(out.data_ptr());
  p.update_state = update_state ? 1 : 0;
  p.one_token_per_seq = one_token_per_seq ? 1 : 0;
  if (seq_end.has_value() && seq_end->defined()) {
    need(*seq_end, at::kInt, "seq_end");
    TORCH_CHECK(seq_end->numel() == p.n_seq && !one_token_per_seq, "seq_end [n_seq], not with the decode fast path");
    p.seq_end = static_cast<const int*>(seq_end->data_ptr());
  }
  p.state_only = state_only ? 1 : 0;
  if (parent.has_value() && parent->defined()) {
    need(*parent, at::kInt, "parent");
    TORCH_CHECK(parent->numel() == p.T && !one_token_per_seq, "parent [T], not with the decode fast path");
    p.parent = static_cast<const int*>(parent->data_ptr());
  }
  if (last_token.has_value() && last_token->defined()) {
    need(*last_token, at::kInt, "last_token");
    TORCH_CHECK(last_token->numel() == p.n_seq, "last_token [n_seq]");
    p.last_token = static_cast<const int*>(last_token->data_ptr());
  }
  chk(nfb::causal_conv1d_silu(p, cur_stream(), pdl));
}

void gdn_recurrent(const Tensor& qkv, int64_t q_off, int64_t k_off, int64_t v_off, const Tensor& proj, int64_t z_off,
                   int64_t a_off, int64_t b_off, int64_t n_qk_heads, int64_t n_v_heads, const Tensor& A_log,
                   const Tensor& dt_bias, const Tensor& norm_w, double eps, const Tensor& cu_seqlens,
                   const Tensor& state_slot, const Tensor& state, bool write_state, const Tensor& out, bool pdl,
                   OptT seq_end, OptT commit, OptT chunk_ws, OptT conv_w, OptT conv_state, OptT q_codes, OptT q_sf) {
  need(qkv, at::kBFloat16, "qkv"); need_rows(qkv, "qkv"); need(proj, at::kBFloat16, "proj"); need_rows(proj, "proj");
  need(A_log, at::kFloat, "A_log"); need(dt_bias, at::kFloat, "dt_bias"); need(norm_w, at::kBFloat16, "norm_w");
  need(cu_seqlens, at::kInt, "cu_seqlens"); need(state_slot, at::kInt, "state_slot");
  need(state, at::kFloat, "state"); need(out, at::kBFloat16, "out");
  TORCH_CHECK(state.is_contiguous() && state.dim() == 4 && state.size(1) == n_v_heads && state.size(2) == 128 &&
              state.size(3) == 128, "state must be [slots, Hv, 128, 128]");
  TORCH_CHECK(out.is_contiguous() && out.numel() == qkv.size(0) * n_v_heads * 128, "gdn out shape");
  TORCH_CHECK(A_log.numel() == n_v_heads && dt_bias.numel() == n_v_heads && norm_w.numel() == 128);
  c10::cuda::CUDAGuard guard(qkv.device());
  nfb::GdnParams p = {};
  p.qkv = static_cast<const __nv_bfloat16*>(qkv.data_ptr()); p.ld_qkv = qkv.stride(0);
  p.q_off = static_cast<int>(q_off); p.k_off = static_cast<int>(k_off); p.v_off = static_cast<int>(v_off);
  p.proj = static_cast<const __nv_bfloat16*>(proj.data_ptr()); p.ld_proj = proj.stride(0);
  p.z_off = static_cast<int>(z_off); p.a_off = static_cast<int>(a_off); p.b_off = static_cast<int>(b_off);
  p.T = static_cast<int>(qkv.size(0)); p.n_seq = static_cast<int>(state_slot.numel());
  TORCH_CHECK(cu_seqlens.numel() == p.n_seq + 1);
  p.n_qk_heads = static_cast<int>(n_qk_heads); p.n_v_heads = static_cast<int>(n_v_heads);
  p.A_log = static_cast<const float*>(A_log.data_ptr()); p.dt_bias = static_cast<const float*>(dt_bias.data_ptr());
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w.data_ptr()); p.eps = static_cast<float>(eps);
  p.cu_seqlens = static_cast<const int*>(cu_seqlens.data_ptr());
  p.state_slot = static_cast<const int*>(state_slot.data_ptr());
  p.state = static_cast<float*>(state.data_ptr());
  p.write_state = write_state ? 1 : 0;
  p.out = static_cast<__nv_bfloat16*>(out.data_ptr());
  if (seq_end.has_value() && seq_end->defined()) {
    need(*seq_end, at::kInt, "seq_end");
    TORCH_CHECK(seq_end->numel() == p.n_seq, "seq_end [n_seq]");
    p.seq_end = static_cast<const int*>(seq_end->data_ptr());
  }
  if (commit.has_value() && commit->defined()) {
    need(*commit, at::kByte, "commit");
    TORCH_CHECK(commit->numel() == p.T, "commit [T]");
    p.commit = static_cast<const unsigned char*>(commit->data_ptr());
  }
  if (conv_w.has_value() && conv_w->defined()) {
    // decode with the causal convolution fused in: `qkv` is the raw projection, channel c at column c
    TORCH_CHECK(conv_state.has_value() && conv_state->defined(), "conv_state required with conv_w");
    need(*conv_w, at::kBFloat16, "conv_w"); need(*conv_state, at::kBFloat16, "conv_state");
    TORCH_CHECK(conv_w->is_contiguous() && conv_w->dim() == 2 && conv_w->size(1) == 4, "conv_w must be [C, 4]");
    TORCH_CHECK(conv_state->is_contiguous() && conv_state->dim() == 3 && conv_state->size(1) == 3 &&
                conv_state->size(2) == conv_w->size(0), "conv_state must be [slots, 3, C]");
    TORCH_CHECK(conv_w->size(0) <= qkv.size(1) && reinterpret_cast<uintptr_t>(conv_w->data_ptr()) % 8 == 0, "conv_w layout");
    p.conv_w = static_cast<const __nv_bfloat16*>(conv_w->data_ptr());
    p.conv_state = static_cast<__nv_bfloat16*>(conv_state->data_ptr());
    p.conv_C = static_cast<int>(conv_w->size(0));
  }
  if (q_codes.has_value() && q_codes->defined()) {
    TORCH_CHECK(q_sf.has_value() && q_sf->defined(), "q_sf required with q_codes");
    need(*q_codes, at::kByte, "q_codes"); need(*q_sf, at::kByte, "q_sf");
    TORCH_CHECK(q_codes->numel() >= static_cast<int64_t>(p.T) * n_v_heads * 64, "q_codes too small");
    TORCH_CHECK(p.T == p.n_seq, "the fused output quantiser is for decode steps (one token per sequence)");
    p.q_codes = static_cast<uint8_t*>(q_codes->data_ptr());
    p.q_sf = static_cast<uint8_t*>(q_sf->data_ptr());
  }
  if (chunk_ws.has_value() && chunk_ws->defined()) {
    // chunked tensor-core formulation (long prefill chunks)
    need(*chunk_ws, at::kByte, "chunk_ws");
    TORCH_CHECK(chunk_ws->is_contiguous(), "chunk_ws must be contiguous");
    chk(nfb::gdn_chunked(p, chunk_ws->data_ptr(), static_cast<size_t>(chunk_ws->numel()), cur_stream()));
    return;
  }
  chk(nfb::gdn_recurrent(p, cur_stream(), pdl));
}

int64_t gdn_chunked_workspace_bytes(int64_t T, int64_t n_seq, int64_t n_v_heads) {
  return static_cast<int64_t>(nfb::gdn_chunked_workspace_bytes(
      nfb::gdn_chunked_max_chunks(static_cast<int>(T), static_cast<int>(n_seq)), static_cast<int>(n_v_heads)));
}

void argmax_rows(const Tensor& logits, const Tensor& out, bool pdl) {
  need(logits, at::kBFloat16, "logits"); need_rows(logits, "logits"); need(out, at::kInt, "out");
  TORCH_CHECK(out.numel() == logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  chk(nfb::argmax_rows(logits.data_ptr(), logits.stride(0), static_cast<int>(logits.size(0)),
                       static_cast<int>(logits.size(1)), static_cast<int*>(out.data_ptr()), cur_stream(), pdl));
}

void sample_rows(const Tensor& logits, OptT temperature, OptT top_k, OptT top_p, OptT min_p, OptT presence,
                 OptT frequency, OptT token_counts, OptT seeds, OptT positions, int64_t purpose, const Tensor& out,
                 OptT out_prob, OptT draft_ids, OptT accepted, OptT draft_dist_ids, OptT draft_dist_probs,
                 OptT out_dist_ids, OptT out_dist_probs) {
  need(logits, at::kBFloat16, "logits"); need_rows(logits, "logits"); need(out, at::kInt, "out");
  c10::cuda::CUDAGuard guard(logits.device());
  nfb::SampleParams p = {};
  p.logits = static_cast<const __nv_bfloat16*>(logits.data_ptr()); p.ld = logits.stride(0);
  p.T = static_cast<int>(logits.size(0)); p.V = static_cast<int>(logits.size(1));
  p.temperature = ptr_or_null<const float>(temperature); p.top_k = ptr_or_null<const int>(top_k);
  p.top_p = ptr_or_null<const float>(top_p); p.min_p = ptr_or_null<const float>(min_p);
  p.presence = ptr_or_null<const float>(presence); p.frequency = ptr_or_null<const float>(frequency);
  p.token_counts = ptr_or_null<const int>(token_counts);
  p.seeds = ptr_or_null<const unsigned long long>(seeds); p.positions = ptr_or_null<const int>(positions);
  p.purpose = static_cast<unsigned int>(purpose);
  p.out = static_cast<int*>(out.data_ptr()); p.out_prob = ptr_or_null<float>(out_prob);
  if (draft_ids.has_value() && draft_ids->defined()) {
    need(*draft_ids, at::kInt, "draft_ids");
    TORCH_CHECK(draft_ids->numel() >= p.T, "draft_ids: one entry per row");
    p.draft_ids = static_cast<const int*>(draft_ids->data_ptr());
  }
  if (accepted.has_value() && accepted->defined()) {
    need(*accepted, at::kInt, "accepted");
    TORCH_CHECK(accepted->numel() >= p.T, "accepted: one entry per row");
    p.accepted = static_cast<int*>(accepted->data_ptr());
  }
  if (draft_dist_ids.has_value() && draft_dist_ids->defined()) {
    TORCH_CHECK(draft_dist_probs.has_value() && draft_dist_probs->defined() && p.draft_ids != nullptr,
                "draft distribution needs ids, probabilities and draft_ids");
    need(*draft_dist_ids, at::kInt, "draft_dist_ids"); need(*draft_dist_probs, at::kFloat, "draft_dist_probs");
    TORCH_CHECK(draft_dist_ids->is_contiguous() && draft_dist_probs->is_contiguous() && draft_dist_ids->dim() == 2 &&
                draft_dist_ids->size(0) >= p.T && draft_dist_probs->sizes() == draft_dist_ids->sizes(), "draft distribution shapes");
    p.draft_dist_ids = static_cast<const int*>(draft_dist_ids->data_ptr());
    p.draft_dist_probs = static_cast<const float*>(draft_dist_probs->data_ptr());
    p.dist_k = static_cast<int>(draft_dist_ids->size(1));
  }
  if (out_dist_ids.has_value() && out_dist_ids->defined()) {
    TORCH_CHECK(out_dist_probs.has_value() && out_dist_probs->defined(), "out_dist needs ids and probabilities");
    need(*out_dist_ids, at::kInt, "out_dist_ids"); need(*out_dist_probs, at::kFloat, "out_dist_probs");
    TORCH_CHECK(out_dist_ids->is_contiguous() && out_dist_probs->is_contiguous() && out_dist_ids->dim() == 2 &&
                out_dist_ids->size(0) >= p.T && out_dist_probs->sizes() == out_dist_ids->sizes(), "out distribution shapes");
    p.out_dist_ids = static_cast<int*>(out_dist_ids->data_ptr());
    p.out_dist_probs = static_cast<float*>(out_dist_probs->data_ptr());
    p.dist_out_k = static_cast<int>(out_dist_ids->size(1));
  }
  chk(nfb::sample_rows(p, cur_stream()));
}

void accept_greedy_chain(const Tensor& target_ids, const Tensor& draft_ids, const Tensor& n_accepted,
                         const Tensor& out_tokens) {
  need(target_ids, at::kInt, "target_ids"); need(draft_ids, at::kInt, "draft_ids");
  need(n_accepted, at::kInt, "n_accepted"); need(out_tokens, at::kInt, "out_tokens");
  const int B = static_cast<int>(draft_ids.size(0)), K = static_cast<int>(draft_ids.size(1));
  TORCH_CHECK(target_ids.is_contiguous() && draft_ids.is_contiguous() && target_ids.numel() == B * (K + 1) &&
              out_tokens.numel() == B * (K + 1) && n_accepted.numel() == B);
  c10::cuda::CUDAGuard guard(target_ids.device());
  chk(nfb::accept_greedy_chain(static_cast<const int*>(target_ids.data_ptr()),
                               static_cast<const int*>(draft_ids.data_ptr()), B, K,
                               static_cast<int*>(n_accepted.data_ptr()), static_cast<int*>(out_tokens.data_ptr()),
                               cur_stream()));
}

void accept_greedy_tree(const Tensor& target_ids, const Tensor& node_tok, const Tensor& parent, int64_t max_depth,
                        const Tensor& n_accepted, const Tensor& out_tokens, const Tensor& out_nodes) {
  need(target_ids, at::kInt, "target_ids"); need(node_tok, at::kInt, "node_tok"); need(parent, at::kInt, "parent");
  need(n_accepted, at::kInt, "n_accepted"); need(out_tokens, at::kInt, "out_tokens"); need(out_nodes, at::kInt, "out_nodes");
  const int B = static_cast<int>(node_tok.size(0)), N = static_cast<int>(node_tok.size(1));
  TORCH_CHECK(target_ids.numel() == B * N && parent.numel() == B * N && n_accepted.numel() == B &&
              out_tokens.numel() == B * (max_depth + 1) && out_nodes.numel() == B * (max_depth + 1));
  c10::cuda::CUDAGuard guard(target_ids.device());
  chk(nfb::accept_greedy_tree(static_cast<const int*>(target_ids.data_ptr()),
                              static_cast<const int*>(node_tok.data_ptr()), static_cast<const int*>(parent.data_ptr()),
                              B, N, static_cast<int>(max_depth), static_cast<int*>(n_accepted.data_ptr()),
                              static_cast<int*>(out_tokens.data_ptr()), static_cast<int*>(out_nodes.data_ptr()),
                              cur_stream()));
}

// ---------------------------------------------------------------- tensor parallel
// One symmetric allocation per rank; `peer_bases[r]` is rank r's allocation as mapped here.
std::tuple<Tensor, Tensor> symm_alloc(int64_t bytes) {
  void* ptr = nullptr;
  Tensor handle = at::empty({64}, at::TensorOptions().dtype(at::kByte));
  chk(nfb::symm_alloc(static_cast<size_t>(bytes), &ptr, handle.data_ptr<uint8_t>()));
  int dev = 0;
  cudaGetDevice(&dev);
  Tensor view = at::from_blob(ptr, {bytes}, [](void*) {}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev));
  return {view, handle};
}

int64_t symm_open(const Tensor& handle) {
  TORCH_CHECK(!handle.is_cuda() && handle.scalar_type() == at::kByte && handle.numel() == 64, "handle must be 64 CPU bytes");
  void* ptr = nullptr;
  chk(nfb::symm_open(handle.data_ptr<uint8_t>(), &ptr));
  return reinterpret_cast<int64_t>(ptr);
}

void gemm_bf16_push(const Tensor& x, const Tensor& w, int64_t splits, int64_t world, int64_t rank,
                    at::IntArrayRef peer_bases, int64_t recv_off, int64_t flag_off, OptT status, bool pdl) {
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w"); need_rows(x, "x"); need_rows(w, "w");
  TORCH_CHECK(x.size(1) == w.size(1), "gemm_bf16_push: K mismatch");
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMaxRanks, "peer_bases size");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::GemmArgs a;
  a.w = w.data_ptr(); a.N = w.size(0); a.K = w.size(1); a.ldw = w.stride(0);
  a.x = x.data_ptr(); a.T = x.size(0); a.ldx = x.stride(0);
  a.splits = static_cast<int>(splits); a.epi = nfb::kEpiPushPartial;
  a.world = static_cast<int>(world); a.rank = static_cast<int>(rank);
  for (int r = 0; r < world; ++r) {
    a.peer_recv[r] = reinterpret_cast<float*>(peer_bases[r] + recv_off);
    a.peer_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + flag_off);
  }
  a.ldo = 2;
  a.status = ptr_or_null<int>(status); a.stream = cur_stream(); a.pdl = pdl;
  chk(nfb::gemm_bf16(a));
}

void tp_reduce_ag_norm(int64_t world, int64_t rank, int64_t T, int64_t T_cap, int64_t N, int64_t splits,
                       int64_t arrivals, at::IntArrayRef peer_bases, int64_t recv_off, int64_t flag_off,
                       int64_t x_off, int64_t ss_off, int64_t row_flag_off, OptT norm_w, OptT normed, double eps,
                       bool unit_offset, const Tensor& state, OptT status, bool pdl, int64_t phases) {
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMaxTpRanks, "peer_bases size");
  need(state, at::kByte, "state");
  TORCH_CHECK(state.numel() >= static_cast<int64_t>(sizeof(nfb::TpState)), "state too small");
  TORCH_CHECK(phases >= 1 && phases <= 3, "phases must be 1, 2 or 3");
  c10::cuda::CUDAGuard guard(state.device());
  nfb::TpReduceParams p = {};
  p.phases = static_cast<int>(phases);
  p.world = static_cast<int>(world); p.rank = static_cast<int>(rank); p.T = static_cast<int>(T);
  p.T_cap = static_cast<int>(T_cap); p.N = static_cast<int>(N); p.splits = static_cast<int>(splits);
  p.arrivals_this_call = static_cast<unsigned int>(arrivals);
  const int64_t me = peer_bases[rank];
  p.my_recv = reinterpret_cast<const float*>(me + recv_off);
  p.my_arrival_flag = reinterpret_cast<const unsigned int*>(me + flag_off);
  p.my_x = reinterpret_cast<__nv_bfloat16*>(me + x_off);
  p.my_ss = reinterpret_cast<float*>(me + ss_off);
  p.my_row_flag = reinterpret_cast<unsigned int*>(me + row_flag_off);
  for (int r = 0; r < world; ++r) {
    p.peer_x[r] = reinterpret_cast<__nv_bfloat16*>(peer_bases[r] + x_off);
    p.peer_ss[r] = reinterpret_cast<float*>(peer_bases[r] + ss_off);
    p.peer_row_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + row_flag_off);
  }
  if (norm_w.has_value() && norm_w->defined()) {
    need(*norm_w, at::kBFloat16, "norm_w");
    TORCH_CHECK(norm_w->numel() == N);
    p.norm_w = static_cast<const __nv_bfloat16*>(norm_w->data_ptr());
  }
  if (normed.has_value() && normed->defined()) {
    need(*normed, at::kBFloat16, "normed");
    TORCH_CHECK(normed->is_contiguous() && normed->numel() == T * N && p.norm_w != nullptr);
    p.normed = static_cast<__nv_bfloat16*>(normed->data_ptr());
  }
  p.eps = static_cast<float>(eps); p.unit_offset = unit_offset ? 1 : 0;
  p.state = reinterpret_cast<nfb::TpState*>(state.data_ptr());
  p.status = ptr_or_null<int>(status);
  chk(nfb::tp_reduce_ag_norm(p, cur_stream(), pdl));
}

void tp_argmax(int64_t world, int64_t rank, int64_t T_cap, const Tensor& logits, at::IntArrayRef peer_bases,
               int64_t cand_off, int64_t flag_off, const Tensor& out, const Tensor& state, OptT status, bool pdl,
               int64_t phases) {
  TORCH_CHECK(phases >= 1 && phases <= 3, "phases must be 1, 2 or 3");
  need(logits, at::kBFloat16, "logits"); need_rows(logits, "logits"); need(out, at::kInt, "out");
  need(state, at::kByte, "state");
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMaxTpRanks, "peer_bases size");
  TORCH_CHECK(out.numel() >= logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  nfb::TpArgmaxParams p = {};
  p.world = static_cast<int>(world); p.rank = static_cast<int>(rank); p.T = static_cast<int>(logits.size(0));
  p.T_cap = static_cast<int>(T_cap); p.V_local = static_cast<int>(logits.size(1));
  p.logits = static_cast<const __nv_bfloat16*>(logits.data_ptr()); p.ld = logits.stride(0);
  const int64_t me = peer_bases[rank];
  p.my_cand = reinterpret_cast<float2*>(me + cand_off);
  p.my_flag = reinterpret_cast<unsigned int*>(me + flag_off);
  for (int r = 0; r < world; ++r) {
    p.peer_cand[r] = reinterpret_cast<float2*>(peer_bases[r] + cand_off);
    p.peer_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + flag_off);
  }
  p.out = static_cast<int*>(out.data_ptr());
  p.state = reinterpret_cast<nfb::TpState*>(state.data_ptr());
  p.status = ptr_or_null<int>(status);
  p.phases = static_cast<int>(phases);
  chk(nfb::tp_argmax(p, cur_stream(), pdl));
}

void gemm_bf16_push_all(const Tensor& x, const Tensor& w, int64_t splits, int64_t world, int64_t rank,
                        at::IntArrayRef peer_bases, int64_t recv_off, int64_t flag_off, int64_t T_cap,
                        const Tensor& state, OptT status, bool pdl) {
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w"); need_rows(x, "x"); need_rows(w, "w");
  need(state, at::kByte, "state");
  TORCH_CHECK(x.size(1) == w.size(1), "gemm_bf16_push_all: K mismatch");
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMaxRanks, "peer_bases size");
  TORCH_CHECK(state.numel() >= static_cast<int64_t>(sizeof(nfb::TpState)), "state too small");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::GemmArgs a;
  a.w = w.data_ptr(); a.N = w.size(0); a.K = w.size(1); a.ldw = w.stride(0);
  a.x = x.data_ptr(); a.T = x.size(0); a.ldx = x.stride(0);
  a.splits = static_cast<int>(splits); a.epi = nfb::kEpiPushAll;
  a.world = static_cast<int>(world); a.rank = static_cast<int>(rank);
  a.T_cap = static_cast<int>(T_cap);
  a.call_idx = &reinterpret_cast<const nfb::TpState*>(state.data_ptr())->call_idx;
  for (int r = 0; r < world; ++r) {
    a.peer_recv[r] = reinterpret_cast<float*>(peer_bases[r] + recv_off);
    a.peer_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + flag_off);
  }
  a.ldo = 2;
  a.status = ptr_or_null<int>(status); a.stream = cur_stream(); a.pdl = pdl;
  chk(nfb::gemm_bf16(a));
}

void tp_sum_norm(int64_t world, int64_t T_cap, int64_t arrivals, int64_t my_base, int64_t recv_off, int64_t flag_off,
                 const Tensor& x, OptT norm_w, OptT normed, double eps, bool unit_offset, const Tensor& state,
                 OptT status, bool pdl) {
  need(x, at::kBFloat16, "x"); need(state, at::kByte, "state");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous(), "x must be contiguous [T, N]");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::TpSumNormParams p = {};
  p.world = static_cast<int>(world); p.T = static_cast<int>(x.size(0)); p.T_cap = static_cast<int>(T_cap);
  p.N = static_cast<int>(x.size(1));
  p.arrivals_this_call = static_cast<unsigned int>(arrivals);
  p.my_recv = reinterpret_cast<const float*>(my_base + recv_off);
  p.my_flag = reinterpret_cast<const unsigned int*>(my_base + flag_off);
  p.x = static_cast<__nv_bfloat16*>(x.data_ptr());
  if (norm_w.has_value() && norm_w->defined()) {
    need(*norm_w, at::kBFloat16, "norm_w");
    TORCH_CHECK(norm_w->numel() == p.N);
    p.norm_w = static_cast<const __nv_bfloat16*>(norm_w->data_ptr());
  }
  if (normed.has_value() && normed->defined()) {
    need(*normed, at::kBFloat16, "normed");
    TORCH_CHECK(normed->is_contiguous() && normed->numel() == x.numel());
    p.normed = static_cast<__nv_bfloat16*>(normed->data_ptr());
  }
  p.eps = static_cast<float>(eps); p.unit_offset = unit_offset ? 1 : 0;
  p.state = reinterpret_cast<nfb::TpState*>(state.data_ptr());
  p.status = ptr_or_null<int>(status);
  chk(nfb::tp_sum_norm(p, cur_stream(), pdl));
}

// Row-parallel GEMM whose epilogue reduce-scatters into the owner rank, reduces there and all-gathers the new
// residual tile (gemm kEpiRsAg).  All buffers are offsets into the ranks' symmetric allocations.
void gemm_bf16_rs_ag(const Tensor& x, const Tensor& w, int64_t splits, int64_t world, int64_t rank,
                     at::IntArrayRef peer_bases, int64_t recv_off, int64_t flag_off, int64_t x_off, int64_t ss_off,
                     int64_t xflag_off, int64_t T_cap, int64_t ld_resid, const Tensor& state, int64_t phase,
                     OptT status, bool pdl, OptT prefetch) {
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w"); need_rows(x, "x"); need_rows(w, "w");
  need(state, at::kByte, "state");
  TORCH_CHECK(x.size(1) == w.size(1), "gemm_bf16_rs_ag: K mismatch");
  TORCH_CHECK(static_cast<int64_t>(peer_bases.size()) == world && world <= nfb::kMaxRanks, "peer_bases size");
  TORCH_CHECK(state.numel() >= static_cast<int64_t>(sizeof(nfb::RsState)), "state too small");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::GemmArgs a;
  a.w = w.data_ptr(); a.N = w.size(0); a.K = w.size(1); a.ldw = w.stride(0);
  a.x = x.data_ptr(); a.T = x.size(0); a.ldx = x.stride(0);
  a.splits = static_cast<int>(splits); a.epi = nfb::kEpiRsAg;
  a.world = static_cast<int>(world); a.rank = static_cast<int>(rank);
  a.T_cap = static_cast<int>(T_cap); a.ld_resid = ld_resid;
  a.rs_state = reinterpret_cast<nfb::RsState*>(state.data_ptr());
  a.rs_phase = static_cast<int>(phase);
  for (int r = 0; r < world; ++r) {
    a.peer_recv[r] = reinterpret_cast<float*>(peer_bases[r] + recv_off);
    a.peer_flag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + flag_off);
    a.peer_x[r] = reinterpret_cast<void*>(peer_bases[r] + x_off);
    a.peer_ss[r] = reinterpret_cast<float*>(peer_bases[r] + ss_off);
    a.peer_xflag[r] = reinterpret_cast<unsigned int*>(peer_bases[r] + xflag_off);
  }
  a.ldo = 2;
  a.status = ptr_or_null<int>(status); a.stream = cur_stream(); a.pdl = pdl;
  fill_prefetch(a, prefetch);
  chk(nfb::gemm_bf16(a));
}

// Column-parallel GEMM (store or SwiGLU epilogue) that waits for the all-gathered residual stream by itself and
// applies the RMS norm as a row scale (see nfb::GemmGather).
void gemm_bf16_gathered(const Tensor& x, const Tensor& w, const Tensor& out, int64_t epi, int64_t splits,
                        int64_t my_base, int64_t ss_off, int64_t xflag_off, int64_t n_features, double eps,
                        const Tensor& state, OptT status, bool pdl, OptT conv_w, OptT conv_state, OptT conv_slot,
                        OptT conv_out, OptT prefetch) {
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w"); need(out, at::kBFloat16, "out");
  need_rows(x, "x"); need_rows(w, "w"); need_rows(out, "out");
  need(state, at::kByte, "state");
  TORCH_CHECK(x.size(1) == w.size(1), "gemm_bf16_gathered: K mismatch");
  TORCH_CHECK(epi == nfb::kEpiStore || epi == nfb::kEpiSwiglu, "gemm_bf16_gathered: store or SwiGLU epilogue");
  TORCH_CHECK(state.numel() >= static_cast<int64_t>(sizeof(nfb::RsState)), "state too small");
  TORCH_CHECK(n_features == x.size(1) && n_features % 128 == 0, "gemm_bf16_gathered: the GEMM's K must be the normalised width");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::GemmArgs a;
  a.w = w.data_ptr(); a.N = w.size(0); a.K = w.size(1); a.ldw = w.stride(0);
  a.x = x.data_ptr(); a.T = x.size(0); a.ldx = x.stride(0);
  const int64_t out_cols = epi == nfb::kEpiSwiglu ? a.N / 2 : a.N;
  TORCH_CHECK(out.size(0) == a.T && out.size(1) == out_cols, "gemm_bf16_gathered: out shape");
  a.out = out.data_ptr(); a.ldo = out.stride(0);
  a.splits = static_cast<int>(splits); a.epi = static_cast<int>(epi);
  a.gather.flag = reinterpret_cast<const unsigned int*>(my_base + xflag_off);
  a.gather.target = &reinterpret_cast<const nfb::RsState*>(state.data_ptr())->x_expected;
  a.gather.ss = reinterpret_cast<const float*>(my_base + ss_off);
  a.gather.ss_tiles = static_cast<int>(n_features / 128);
  a.gather.n_features = static_cast<int>(n_features);
  a.gather.eps = static_cast<float>(eps);
  a.status = ptr_or_null<int>(status); a.stream = cur_stream(); a.pdl = pdl;
  fill_conv(a, conv_w, conv_state, conv_slot, conv_out);
  fill_prefetch(a, prefetch);
  chk(nfb::gemm_bf16(a));
}

void tp_gather_norm(const Tensor& x, const Tensor& norm_w, const Tensor& normed, int64_t my_base, int64_t xflag_off,
                    double eps, bool unit_offset, const Tensor& state, OptT status, bool pdl) {
  need(x, at::kBFloat16, "x"); need(norm_w, at::kBFloat16, "norm_w"); need(normed, at::kBFloat16, "normed");
  need_rows(x, "x"); need(state, at::kByte, "state");
  TORCH_CHECK(normed.is_contiguous() && normed.dim() == 2 && normed.size(0) == x.size(0) && normed.size(1) == x.size(1),
              "tp_gather_norm: normed shape");
  TORCH_CHECK(norm_w.numel() == x.size(1) && norm_w.is_contiguous(), "tp_gather_norm: norm weight shape");
  TORCH_CHECK(state.numel() >= static_cast<int64_t>(sizeof(nfb::RsState)), "state too small");
  c10::cuda::CUDAGuard guard(x.device());
  nfb::TpGatherNormParams p = {};
  p.T = static_cast<int>(x.size(0)); p.N = static_cast<int>(x.size(1));
  p.flag = reinterpret_cast<const unsigned int*>(my_base + xflag_off);
  p.target = &reinterpret_cast<const nfb::RsState*>(state.data_ptr())->x_expected;
  p.x = static_cast<const __nv_bfloat16*>(x.data_ptr()); p.ldx = x.stride(0);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w.data_ptr());
  p.normed = static_cast<__nv_bfloat16*>(normed.data_ptr());
  p.eps = static_cast<float>(eps); p.unit_offset = unit_offset ? 1 : 0;
  p.status = ptr_or_null<int>(status);
  chk(nfb::tp_gather_norm(p, cur_stream(), pdl));
}

int64_t rs_state_bytes() { return static_cast<int64_t>(sizeof(nfb::RsState)); }

int64_t tp_state_bytes() { return static_cast<int64_t>(sizeof(nfb::TpState)); }

}  // namespace

TORCH_LIBRARY(nfb200, m) {
  m.def("symm_alloc(int bytes) -> (Tensor, Tensor)", &symm_alloc);
  m.def("symm_open(Tensor handle) -> int", &symm_open);
  m.def("gemm_bf16_push(Tensor x, Tensor w, int splits, int world, int rank, int[] peer_bases, int recv_off, int flag_off, Tensor? status, bool pdl) -> ()", &gemm_bf16_push);
  m.def("tp_reduce_ag_norm(int world, int rank, int T, int T_cap, int N, int splits, int arrivals, int[] peer_bases, int recv_off, int flag_off, int x_off, int ss_off, int row_flag_off, Tensor? norm_w, Tensor? normed, float eps, bool unit_offset, Tensor state, Tensor? status, bool pdl, int phases=3) -> ()", &tp_reduce_ag_norm);
  m.def("tp_argmax(int world, int rank, int T_cap, Tensor logits, int[] peer_bases, int cand_off, int flag_off, Tensor out, Tensor state, Tensor? status, bool pdl, int phases=3) -> ()", &tp_argmax);
  m.def("tp_state_bytes() -> int", &tp_state_bytes);
  m.def("rs_state_bytes() -> int", &rs_state_bytes);
  m.def("gemm_bf16_rs_ag(Tensor x, Tensor w, int splits, int world, int rank, int[] peer_bases, int recv_off, int flag_off, int x_off, int ss_off, int xflag_off, int T_cap, int ld_resid, Tensor state, int phase, Tensor? status, bool pdl, Tensor? prefetch=None) -> ()", &gemm_bf16_rs_ag);
  m.def("gemm_bf16_gathered(Tensor x, Tensor w, Tensor out, int epi, int splits, int my_base, int ss_off, int xflag_off, int n_features, float eps, Tensor state, Tensor? status, bool pdl, Tensor? conv_w=None, Tensor? conv_state=None, Tensor? conv_slot=None, Tensor? conv_out=None, Tensor? prefetch=None) -> ()", &gemm_bf16_gathered);
  m.def("tp_gather_norm(Tensor x, Tensor norm_w, Tensor normed, int my_base, int xflag_off, float eps, bool unit_offset, Tensor state, Tensor? status, bool pdl) -> ()", &tp_gather_norm);
  m.def("gemm_bf16_push_all(Tensor x, Tensor w, int splits, int world, int rank, int[] peer_bases, int recv_off, int flag_off, int T_cap, Tensor state, Tensor? status, bool pdl) -> ()", &gemm_bf16_push_all);
  m.def("tp_sum_norm(int world, int T_cap, int arrivals, int my_base, int recv_off, int flag_off, Tensor x, Tensor? norm_w, Tensor? normed, float eps, bool unit_offset, Tensor state, Tensor? status, bool pdl) -> ()", &tp_sum_norm);
  m.def("gemm_bf16(Tensor x, Tensor w, Tensor? out, int epi, Tensor? resid, Tensor? bias, Tensor? partial, int splits, Tensor? status, bool pdl, int act=0, Tensor? conv_w=None, Tensor? conv_state=None, Tensor? conv_slot=None, Tensor? conv_out=None, Tensor? prefetch=None) -> ()", &gemm_bf16);
  m.def("gemm_trace(bool enable, int n_ctas) -> Tensor", &gemm_trace);
  m.def("gemm_timeline(int mode) -> (int, Tensor)", &gemm_timeline);
  m.def("attn_tc_trace(bool enable) -> Tensor", &attn_tc_trace);
  m.def("gemm_pick_splits(int T, int N, int K, int epi) -> int", &gemm_pick_splits);
  m.def("add_rmsnorm(Tensor? partial, int splits, Tensor? delta, Tensor? resid_in, Tensor? resid_out, Tensor? norm_w, Tensor? normed, int T, int N, float eps, bool unit_offset, bool pdl, Tensor? q_codes=None, Tensor? q_sf=None) -> ()", &add_rmsnorm);
  m.def("embed_gather(Tensor ids, Tensor table, Tensor out, bool pdl) -> ()", &embed_gather);
  m.def("attn_prep(Tensor proj, int q_off, int k_off, int v_off, int n_q_heads, int n_kv_heads, int head_dim, Tensor? q_norm_w, Tensor? k_norm_w, float eps, bool unit_offset, int rot_dim, Tensor inv_freq, float attn_factor, Tensor rope_pos, Tensor token_seq, Tensor cache_pos, Tensor block_table, Tensor q_out, Tensor k_codes, Tensor v_codes, Tensor? k_scales, Tensor? v_scales, int page_size, int format, int group, bool pdl, bool k_hadamard=False, Tensor? k_row_scale=None, Tensor? tiers=None) -> ()", &attn_prep);
  m.def("paged_attention(Tensor q, int n_q_heads, int n_kv_heads, int head_dim, Tensor q_seq, Tensor q_kv_len, Tensor block_table, Tensor k_codes, Tensor v_codes, Tensor? k_scales, Tensor? v_scales, int page_size, int format, int group, float sm_scale, int split_keys, int n_splits, Tensor part_o, Tensor part_ml, Tensor? gate, Tensor out, Tensor? tree_mask, Tensor? tree_base, int impl, bool pdl, int window=0, Tensor? sel_blocks=None, Tensor? sel_count=None, Tensor? tiers=None, Tensor? q_codes=None, Tensor? q_sf=None) -> ()", &paged_attention);
  m.def("paged_attention_prefill(Tensor q, int n_q_heads, int n_kv_heads, int head_dim, Tensor q_seq, Tensor q_kv_len, Tensor blk_start, Tensor blk_count, Tensor block_table, Tensor k_codes, Tensor v_codes, Tensor? k_scales, Tensor? v_scales, int page_size, int format, int group, float sm_scale, Tensor? gate, Tensor out, bool pdl, int window=0, Tensor? tiers=None) -> ()", &paged_attention_prefill);
  m.def("kv_requant(Tensor tiers, Tensor anchor, Tensor src_cell, Tensor dst_cell, int page_size, int n_kv_heads, int head_dim) -> ()", &kv_requant);
  m.def("prefill_attn_block_tokens(int n_q_heads, int n_kv_heads) -> int", &prefill_attn_block_tokens);
  m.def("causal_conv1d_silu(Tensor x, int c_off, int C, Tensor w, Tensor cu_seqlens, Tensor token_seq, Tensor state_slot, Tensor conv_state, Tensor out, bool update_state, bool one_token_per_seq, bool pdl, Tensor? seq_end=None, bool state_only=False, Tensor? parent=None, Tensor? last_token=None) -> ()", &causal_conv1d_silu);
  m.def("gdn_recurrent(Tensor qkv, int q_off, int k_off, int v_off, Tensor proj, int z_off, int a_off, int b_off, int n_qk_heads, int n_v_heads, Tensor A_log, Tensor dt_bias, Tensor norm_w, float eps, Tensor cu_seqlens, Tensor state_slot, Tensor state, bool write_state, Tensor out, bool pdl, Tensor? seq_end=None, Tensor? commit=None, Tensor? chunk_ws=None, Tensor? conv_w=None, Tensor? conv_state=None, Tensor? q_codes=None, Tensor? q_sf=None) -> ()", &gdn_recurrent);
  m.def("gdn_chunked_workspace_bytes(int T, int n_seq, int n_v_heads) -> int", &gdn_chunked_workspace_bytes);
  m.def("gdn_prefill_trace(bool enable) -> Tensor", &gdn_prefill_trace);
  m.def("kv_move_rows(Tensor block_table, Tensor table_row, Tensor src_pos, Tensor dst_pos, Tensor k_codes, Tensor v_codes, Tensor? k_scales, Tensor? v_scales, int page_size, int n_kv_heads, int head_dim, int format, int group) -> ()", &kv_move_rows);
  m.def("argmax_rows(Tensor logits, Tensor out, bool pdl) -> ()", &argmax_rows);
  m.def("sample_rows(Tensor logits, Tensor? temperature, Tensor? top_k, Tensor? top_p, Tensor? min_p, Tensor? presence, Tensor? frequency, Tensor? token_counts, Tensor? seeds, Tensor? positions, int purpose, Tensor out, Tensor? out_prob, Tensor? draft_ids=None, Tensor? accepted=None, Tensor? draft_dist_ids=None, Tensor? draft_dist_probs=None, Tensor? out_dist_ids=None, Tensor? out_dist_probs=None) -> ()", &sample_rows);
  m.def("accept_greedy_chain(Tensor target_ids, Tensor draft_ids, Tensor n_accepted, Tensor out_tokens) -> ()", &accept_greedy_chain);
  m.def("accept_greedy_tree(Tensor target_ids, Tensor node_tok, Tensor parent, int max_depth, Tensor n_accepted, Tensor out_tokens, Tensor out_nodes) -> ()", &accept_greedy_tree);
}
