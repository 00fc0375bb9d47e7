// Host-side construction of TMA tensor maps without linking libcuda: the
// encoder is fetched from the driver through the runtime's entry-point query.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfb {

enum class TmapDtype { BF16, U8, F32 };

// 2-D row-major tensor [rows, cols] with leading dimension `ld` (elements),
// copied in boxes of [box_rows, box_cols].  `swizzle128` selects the 128-byte
// shared-memory swizzle (box_cols * elem_size must then be exactly 128 bytes).
// Returns false (and leaves *out untouched) when the driver refuses the map.
bool make_tmap_2d(CUtensorMap* out, TmapDtype dt, const void* base, uint64_t rows, uint64_t cols,
                  uint64_t ld, uint32_t box_rows, uint32_t box_cols, bool swizzle128);

}  // namespace nfb
