#include "tensor_map.h"

#include <mutex>

namespace nfb {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn get_encoder() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(p);
    }
  });
  return fn;
}
}  // namespace

bool make_tmap_2d(CUtensorMap* out, TmapDtype dt, const void* base, uint64_t rows, uint64_t cols,
                  uint64_t ld, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeFn enc = get_encoder();
  if (enc == nullptr) return false;
  CUtensorMapDataType cdt;
  uint64_t esz;
  switch (dt) {
    case TmapDtype::BF16: cdt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; esz = 2; break;
    case TmapDtype::U8: cdt = CU_TENSOR_MAP_DATA_TYPE_UINT8; esz = 1; break;
    default: cdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; esz = 4; break;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tmp;
  CUresult r = enc(&tmp, cdt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  *out = tmp;
  return true;
}

}  // namespace nfb
