// Host entry points of the vision-tower kernels (plain C++ ABI).
//
// The tower's GEMMs run on the tcgen05 GEMM with bias / GELU / residual epilogues; what is left are the
// row operations and the attention:
//
//   layer_norm            (x - mean) * rsqrt(var + eps) * w + b per row
//   vision_pos_embed_add  x[p] += bilinear interpolation of a learned side x side table at the patch's
//                         grid position (the four corners and weights are computed in the kernel)
//   vision_rope           2-D rotary embedding of q and k in place inside the packed qkv rows
//   packed_attention      bidirectional attention over packed segments (one image or video frame each):
//                         flash-attention-2 layout on mma.sync bf16 tiles, K/V streamed by cp.async
//
// Reference: include/ninfer/ops/vision_pos_embed.h, include/ninfer/ops/rope.h:63-95 (vision 2-D table),
// include/ninfer/ops/softmax_attention.h:111-144 (packed), src/targets/qwen3_6/impl/runtime/vision_context_impl.h:300-387.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfb {

struct LayerNormParams {
  int T, D;
  const __nv_bfloat16* x;
  long long ldx;
  const __nv_bfloat16* w;  // [D]
  const __nv_bfloat16* b;  // [D], may be null
  __nv_bfloat16* out;
  long long ldo;
  float eps;
};
const char* layer_norm(const LayerNormParams& p, cudaStream_t stream);

struct VisionPosEmbedParams {
  int P, D, side;
  __nv_bfloat16* x;            // [P, D], updated in place
  const __nv_bfloat16* table;  // [side * side, D]
  const int* pos_yx;           // [P, 2] patch row / column inside its grid
  const int* grid_hw;          // [P, 2] height / width of the patch's grid
};
const char* vision_pos_embed_add(const VisionPosEmbedParams& p, cudaStream_t stream);

struct VisionRopeParams {
  int P, H, D;            // D = head_dim = rotary_dim, D / 2 pairs; the first D / 4 pairs turn with y, the rest with x
  __nv_bfloat16* qkv;     // [P, 3 * H * D]: q plane, k plane, v plane
  long long ld;
  const int* pos_yx;      // [P, 2]
  float theta;
};
const char* vision_rope(const VisionRopeParams& p, cudaStream_t stream);

constexpr int kPackedAttnHeadDim = 72;
constexpr int kPackedAttnTile = 64;   // queries per CTA and keys per tile

struct PackedAttnParams {
  int H;                       // heads (q heads = kv heads)
  const __nv_bfloat16* qkv;    // [P, 3 * H * 72]
  long long ld;
  __nv_bfloat16* out;          // [P, H * 72]
  long long ldo;
  const int* tiles;            // [n_tiles, 3]: first query row, segment begin, segment end
  int n_tiles;
  float scale;
};
const char* packed_attention(const PackedAttnParams& p, cudaStream_t stream);

}  // namespace nfb
