// Byte-level BPE merge core (plain C ABI, loaded with ctypes by frontend/tokenizer.py).
//
// The Python side owns the pre-tokeniser (a Unicode regex) and the byte -> symbol alphabet; this file owns the
// hot loop: given one pre-token as a sequence of initial symbol ids, repeatedly merge the adjacent pair with
// the lowest merge rank until no ranked pair is left.  Pairs live in a hash map (left id, right id) -> (rank,
// merged id); each pre-token is handled with a doubly linked list and a min-heap of candidate pairs, so the
// cost is O(n log n) per pre-token instead of the quadratic rescan.
//
// Reference: src/targets/qwen3_6/impl/frontend/tokenizer.cpp (BPE with added tokens and a frame-class column).
#include <cstdint>
#include <queue>
#include <unordered_map>
#include <vector>

namespace {

struct Merge { int32_t rank; int32_t id; };

struct Bpe {
  std::unordered_map<uint64_t, Merge> pairs;
};

inline uint64_t key(int32_t a, int32_t b) {
  return (static_cast<uint64_t>(static_cast<uint32_t>(a)) << 32) | static_cast<uint32_t>(b);
}

struct Cand {
  int32_t rank; int32_t pos; int32_t left, right;  // symbols at the time of insertion (stale entries are skipped)
  bool operator>(const Cand& o) const { return rank != o.rank ? rank > o.rank : pos > o.pos; }
};

}  // namespace

extern "C" {

__attribute__((visibility("default"))) void* nfb200_bpe_create(const int32_t* left, const int32_t* right,
                                                               const int32_t* merged, int32_t n_merges) {
  Bpe* b = new Bpe();
  b->pairs.reserve(static_cast<size_t>(n_merges) * 2);
  for (int32_t i = 0; i < n_merges; ++i) {
    const uint64_t k = key(left[i], right[i]);
    if (b->pairs.find(k) == b->pairs.end()) b->pairs.emplace(k, Merge{i, merged[i]});
  }
  return b;
}

__attribute__((visibility("default"))) void nfb200_bpe_destroy(void* h) { delete static_cast<Bpe*>(h); }

// symbols[n] in, merged ids out (out has room for n); returns the output length.
__attribute__((visibility("default"))) int32_t nfb200_bpe_encode(void* h, const int32_t* symbols, int32_t n,
                                                                 int32_t* out) {
  const Bpe* b = static_cast<const Bpe*>(h);
  if (n <= 0) return 0;
  std::vector<int32_t> sym(symbols, symbols + n), prev(n), next(n);
  for (int32_t i = 0; i < n; ++i) { prev[i] = i - 1; next[i] = i + 1 < n ? i + 1 : -1; }
  std::priority_queue<Cand, std::vector<Cand>, std::greater<Cand>> heap;
  auto push = [&](int32_t i) {
    const int32_t j = next[i];
    if (j < 0) return;
    auto it = b->pairs.find(key(sym[i], sym[j]));
    if (it != b->pairs.end()) heap.push(Cand{it->second.rank, i, sym[i], sym[j]});
  };
  for (int32_t i = 0; i + 1 < n; ++i) push(i);
  std::vector<char> dead(n, 0);
  while (!heap.empty()) {
    const Cand c = heap.top();
    heap.pop();
    const int32_t i = c.pos;
    if (dead[i]) continue;
    const int32_t j = next[i];
    if (j < 0 || dead[j] || sym[i] != c.left || sym[j] != c.right) continue;  // stale
    sym[i] = b->pairs.find(key(c.left, c.right))->second.id;
    dead[j] = 1;
    next[i] = next[j];
    if (next[j] >= 0) prev[next[j]] = i;
    if (prev[i] >= 0) push(prev[i]);
    push(i);
  }
  int32_t m = 0;
  for (int32_t i = 0; i >= 0; i = next[i]) out[m++] = sym[i];
  return m;
}

}  // extern "C"
