// Reference-counted page allocator and block-table bookkeeping of the paged KV cache (plain C ABI, used through
// ctypes by runtime/kv_cache.py).  Pages are shared between block-table rows and detached page lists (session
// checkpoints) by reference count; a page returns to the free list when its last reference is released.  The free
// list is LIFO so that recently used pages (still in L2) are handed out first.
//
// Reference: src/core/paged_kv_cache.{h,cpp} (page-group leases, free-run allocator, block-table matrix).
#include <cstdint>
#include <vector>

namespace {

struct Pool {
  std::vector<int32_t> free_list;
  std::vector<int32_t> refcount;
};

}  // namespace

extern "C" {

#define NFB_API __attribute__((visibility("default")))

NFB_API void* nfb200_pool_create(int32_t n_pages) {
  Pool* p = new Pool();
  p->refcount.assign(static_cast<size_t>(n_pages), 0);
  p->free_list.reserve(static_cast<size_t>(n_pages));
  for (int32_t i = n_pages - 1; i >= 0; --i) p->free_list.push_back(i);
  return p;
}

NFB_API void nfb200_pool_destroy(void* h) { delete static_cast<Pool*>(h); }

NFB_API int32_t nfb200_pool_free_pages(void* h) { return static_cast<int32_t>(static_cast<Pool*>(h)->free_list.size()); }

// Returns the page id, or -1 when the pool is exhausted.
NFB_API int32_t nfb200_pool_alloc(void* h) {
  Pool* p = static_cast<Pool*>(h);
  if (p->free_list.empty()) return -1;
  const int32_t page = p->free_list.back();
  p->free_list.pop_back();
  p->refcount[static_cast<size_t>(page)] = 1;
  return page;
}

// Allocates n pages into out[]; all or nothing.  Returns 0 on success, -1 if fewer than n pages are free.
NFB_API int32_t nfb200_pool_alloc_many(void* h, int32_t n, int32_t* out) {
  Pool* p = static_cast<Pool*>(h);
  if (static_cast<int32_t>(p->free_list.size()) < n) return -1;
  for (int32_t i = 0; i < n; ++i) {
    out[i] = p->free_list.back();
    p->free_list.pop_back();
    p->refcount[static_cast<size_t>(out[i])] = 1;
  }
  return 0;
}

// Returns the new reference count, or -1 for a page that is not allocated.
NFB_API int32_t nfb200_pool_retain(void* h, int32_t page) {
  Pool* p = static_cast<Pool*>(h);
  if (page < 0 || page >= static_cast<int32_t>(p->refcount.size()) || p->refcount[static_cast<size_t>(page)] <= 0) return -1;
  return ++p->refcount[static_cast<size_t>(page)];
}

// Returns the new reference count (0 = the page went back to the free list), or -1 on a double release.
NFB_API int32_t nfb200_pool_release(void* h, int32_t page) {
  Pool* p = static_cast<Pool*>(h);
  if (page < 0 || page >= static_cast<int32_t>(p->refcount.size()) || p->refcount[static_cast<size_t>(page)] <= 0) return -1;
  const int32_t c = --p->refcount[static_cast<size_t>(page)];
  if (c == 0) p->free_list.push_back(page);
  return c;
}

NFB_API int32_t nfb200_pool_refcount(void* h, int32_t page) {
  Pool* p = static_cast<Pool*>(h);
  if (page < 0 || page >= static_cast<int32_t>(p->refcount.size())) return -1;
  return p->refcount[static_cast<size_t>(page)];
}

}  // extern "C"
