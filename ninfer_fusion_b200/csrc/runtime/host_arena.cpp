// Variable-extent allocator over one startup-fixed host buffer (plain C ABI, used through ctypes by
// runtime/host_arena.py).  The buffer itself (pinned host memory holding cold KV replicas and state images) is owned
// by the caller; this file only does the bookkeeping: first-fit over an address-ordered free list, 256-byte
// granules, coalescing on free, generation-checked handles so that a stale handle is refused instead of freeing
// somebody else's extent.
//
// Reference: src/core/host_kv_arena.{h,cpp} (startup-fixed pinned variable-extent allocator for host replicas).
#include <cstdint>
#include <map>
#include <unordered_map>

namespace {

constexpr int64_t kGranule = 256;

struct Extent {
  int64_t offset;
  int64_t bytes;
  uint32_t generation;
};

struct Arena {
  int64_t capacity = 0;
  int64_t used = 0;
  int64_t peak = 0;
  uint32_t next_generation = 1;
  std::map<int64_t, int64_t> free_by_offset;           // offset -> bytes
  std::unordered_map<int64_t, Extent> live;            // offset -> extent
};

inline int64_t round_up(int64_t n) { return (n + kGranule - 1) / kGranule * kGranule; }

}  // namespace

extern "C" {

#define NFB_API __attribute__((visibility("default")))

NFB_API void* nfb200_arena_create(int64_t capacity_bytes) {
  Arena* a = new Arena();
  a->capacity = capacity_bytes / kGranule * kGranule;
  if (a->capacity > 0) a->free_by_offset[0] = a->capacity;
  return a;
}

NFB_API void nfb200_arena_destroy(void* h) { delete static_cast<Arena*>(h); }

// Returns the extent's offset (>= 0) and writes its generation, or -1 when no free run is large enough.
NFB_API int64_t nfb200_arena_alloc(void* h, int64_t bytes, uint32_t* generation) {
  Arena* a = static_cast<Arena*>(h);
  if (bytes <= 0) return -1;
  const int64_t need = round_up(bytes);
  for (auto it = a->free_by_offset.begin(); it != a->free_by_offset.end(); ++it) {
    if (it->second < need) continue;
    const int64_t off = it->first, run = it->second;
    a->free_by_offset.erase(it);
    if (run > need) a->free_by_offset[off + need] = run - need;
    const uint32_t gen = a->next_generation++;
    a->live[off] = Extent{off, need, gen};
    a->used += need;
    if (a->used > a->peak) a->peak = a->used;
    if (generation != nullptr) *generation = gen;
    return off;
  }
  return -1;
}

// 0 on success, -1 if (offset, generation) does not name a live extent.
NFB_API int32_t nfb200_arena_free(void* h, int64_t offset, uint32_t generation) {
  Arena* a = static_cast<Arena*>(h);
  auto it = a->live.find(offset);
  if (it == a->live.end() || it->second.generation != generation) return -1;
  int64_t off = offset, run = it->second.bytes;
  a->used -= run;
  a->live.erase(it);
  auto next = a->free_by_offset.lower_bound(off);
  if (next != a->free_by_offset.end() && next->first == off + run) {   // merge with the run after
    run += next->second;
    next = a->free_by_offset.erase(next);
  }
  if (next != a->free_by_offset.begin()) {                             // merge with the run before
    auto prev = std::prev(next);
    if (prev->first + prev->second == off) {
      off = prev->first;
      run += prev->second;
      a->free_by_offset.erase(prev);
    }
  }
  a->free_by_offset[off] = run;
  return 0;
}

NFB_API int64_t nfb200_arena_used(void* h) { return static_cast<Arena*>(h)->used; }
NFB_API int64_t nfb200_arena_peak(void* h) { return static_cast<Arena*>(h)->peak; }
NFB_API int64_t nfb200_arena_capacity(void* h) { return static_cast<Arena*>(h)->capacity; }
NFB_API int64_t nfb200_arena_largest_free(void* h) {
  int64_t best = 0;
  for (const auto& kv : static_cast<Arena*>(h)->free_by_offset) best = kv.second > best ? kv.second : best;
  return best;
}
NFB_API int32_t nfb200_arena_live_extents(void* h) { return static_cast<int32_t>(static_cast<Arena*>(h)->live.size()); }

}  // extern "C"
