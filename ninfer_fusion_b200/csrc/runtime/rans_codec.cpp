// Range-ANS entropy coder for cold KV slots (host side): 4-bit symbols for packed E2M1 / int4 code planes, 8-bit
// symbols for everything else.  A slot is coded with its own static frequency table (12-bit probabilities), so slots
// decode independently; the caller gives a byte budget and keeps the raw slot when the coded form does not fit.
//
// Counterpart in the reference: the rANS slot encoder / decoder with budgeted streams behind
// include/ninfer/ops/entropy_nvfp4_slot.h (device kernels there; here the coder runs on the host, where cold slots
// live, so that no SM time is spent on a tier that is off the decode path).
//
// Stream: 'R' | bits (4 or 8) | u32 n_bytes (decoded size) | u32 payload bytes | u16 freq[1 << bits] | payload.
// The payload is a byte-renormalised rANS stream, written back to front so that the decoder reads forwards.
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

constexpr uint32_t kProbBits = 12;
constexpr uint32_t kProbScale = 1u << kProbBits;
constexpr uint32_t kLow = 1u << 23;   // lower bound of the normalised state interval [kLow, kLow << 8)

inline int symbol_at(const uint8_t* src, int64_t i, int bits) {
  return bits == 8 ? src[i] : ((src[i >> 1] >> ((i & 1) * 4)) & 0xF);
}

// counts -> frequencies that sum to kProbScale, every present symbol keeping at least 1
void normalise(const std::vector<uint64_t>& count, uint64_t total, std::vector<uint32_t>& freq) {
  const size_t n = count.size();
  freq.assign(n, 0);
  if (total == 0) { freq[0] = kProbScale; return; }
  uint32_t sum = 0;
  size_t largest = 0;
  for (size_t s = 0; s < n; ++s) {
    if (count[s] == 0) continue;
    uint64_t f = count[s] * kProbScale / total;
    freq[s] = static_cast<uint32_t>(f == 0 ? 1 : f);
    sum += freq[s];
    if (count[s] > count[largest] || count[largest] == 0) largest = s;
  }
  // hand the rounding error to the most frequent symbols (stealing from several if one cannot absorb it)
  while (sum != kProbScale) {
    if (sum < kProbScale) { freq[largest] += kProbScale - sum; sum = kProbScale; break; }
    uint32_t over = sum - kProbScale;
    size_t best = n;
    for (size_t s = 0; s < n; ++s)
      if (freq[s] > 1 && (best == n || freq[s] > freq[best])) best = s;
    if (best == n) break;   // cannot happen: n <= 256 symbols of frequency 1 sum to at most 256 < 4096
    uint32_t take = freq[best] - 1 < over ? freq[best] - 1 : over;
    freq[best] -= take;
    sum -= take;
  }
}

}  // namespace

extern "C" {

#define NFB_API __attribute__((visibility("default")))

// worst-case coded size of n_bytes input bytes (header + table + incompressible payload + flush)
NFB_API int64_t nfb200_rans_bound(int64_t n_bytes, int bits) {
  if (n_bytes < 0 || (bits != 4 && bits != 8)) return -1;
  return 10 + 2 * (int64_t(1) << bits) + n_bytes + n_bytes / 64 + 16;
}

// Returns the coded size, -1 on bad arguments, -2 when the coded form would exceed dst_cap (the budget).
NFB_API int64_t nfb200_rans_encode(const uint8_t* src, int64_t n_bytes, int bits, uint8_t* dst, int64_t dst_cap) {
  if (!src || !dst || n_bytes < 0 || n_bytes > 0x7fffffff || (bits != 4 && bits != 8)) return -1;
  const int nsym = 1 << bits;
  const int64_t n = bits == 8 ? n_bytes : 2 * n_bytes;
  const int64_t head = 10 + 2 * nsym;
  if (dst_cap < head + 4) return -2;
  std::vector<uint64_t> count(nsym, 0);
  for (int64_t i = 0; i < n; ++i) ++count[symbol_at(src, i, bits)];
  std::vector<uint32_t> freq, cum(nsym + 1, 0);
  normalise(count, static_cast<uint64_t>(n), freq);
  for (int s = 0; s < nsym; ++s) cum[s + 1] = cum[s] + freq[s];

  // code back to front into the tail of dst; bail out as soon as the budget is gone
  uint8_t* const lo = dst + head;
  uint8_t* p = dst + dst_cap;
  uint32_t x = kLow;
  for (int64_t i = n - 1; i >= 0; --i) {
    const int s = symbol_at(src, i, bits);
    const uint32_t f = freq[s];
    const uint32_t x_max = ((kLow >> kProbBits) << 8) * f;
    while (x >= x_max) {
      if (p == lo) return -2;
      *--p = static_cast<uint8_t>(x & 0xff);
      x >>= 8;
    }
    x = ((x / f) << kProbBits) + (x % f) + cum[s];
  }
  if (p - lo < 4) return -2;
  *--p = static_cast<uint8_t>(x); *--p = static_cast<uint8_t>(x >> 8);
  *--p = static_cast<uint8_t>(x >> 16); *--p = static_cast<uint8_t>(x >> 24);
  const int64_t payload = dst + dst_cap - p;
  std::memmove(lo, p, static_cast<size_t>(payload));
  dst[0] = 'R'; dst[1] = static_cast<uint8_t>(bits);
  const uint32_t nb = static_cast<uint32_t>(n_bytes), pb = static_cast<uint32_t>(payload);
  std::memcpy(dst + 2, &nb, 4);
  std::memcpy(dst + 6, &pb, 4);
  for (int s = 0; s < nsym; ++s) {
    const uint16_t f16 = static_cast<uint16_t>(freq[s]);
    std::memcpy(dst + 10 + 2 * s, &f16, 2);
  }
  return head + payload;
}

// decoded size of a stream, or a negative error
NFB_API int64_t nfb200_rans_decoded_size(const uint8_t* src, int64_t n_src) {
  if (!src || n_src < 10 || src[0] != 'R' || (src[1] != 4 && src[1] != 8)) return -1;
  uint32_t nb;
  std::memcpy(&nb, src + 2, 4);
  return nb;
}

// Returns the decoded byte count; negative on a malformed stream (bad magic -1, truncated -3, bad table -4, small dst -5).
NFB_API int64_t nfb200_rans_decode(const uint8_t* src, int64_t n_src, uint8_t* dst, int64_t dst_cap) {
  if (!src || !dst || n_src < 10 || src[0] != 'R' || (src[1] != 4 && src[1] != 8)) return -1;
  const int bits = src[1], nsym = 1 << bits;
  uint32_t nb, pb;
  std::memcpy(&nb, src + 2, 4);
  std::memcpy(&pb, src + 6, 4);
  const int64_t head = 10 + 2 * nsym;
  if (n_src < head + pb || pb < 4) return -3;
  if (dst_cap < nb) return -5;
  std::vector<uint32_t> freq(nsym), cum(nsym + 1, 0);
  for (int s = 0; s < nsym; ++s) {
    uint16_t f16;
    std::memcpy(&f16, src + 10 + 2 * s, 2);
    freq[s] = f16;
    cum[s + 1] = cum[s] + freq[s];
  }
  if (cum[nsym] != kProbScale) return -4;
  std::vector<uint8_t> slot2sym(kProbScale);
  for (int s = 0; s < nsym; ++s)
    for (uint32_t k = cum[s]; k < cum[s + 1]; ++k) slot2sym[k] = static_cast<uint8_t>(s);

  const uint8_t* p = src + head;
  const uint8_t* const end = p + pb;
  uint32_t x = (uint32_t(p[0]) << 24) | (uint32_t(p[1]) << 16) | (uint32_t(p[2]) << 8) | p[3];
  p += 4;
  const int64_t n = bits == 8 ? int64_t(nb) : 2 * int64_t(nb);
  if (bits == 4) std::memset(dst, 0, nb);
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t slot = x & (kProbScale - 1);
    const uint32_t s = slot2sym[slot];
    if (bits == 8) dst[i] = static_cast<uint8_t>(s);
    else dst[i >> 1] |= static_cast<uint8_t>(s << ((i & 1) * 4));
    x = freq[s] * (x >> kProbBits) + slot - cum[s];
    while (x < kLow) {
      if (p == end) return -3;
      x = (x << 8) | *p++;
    }
  }
  return nb;
}

}  // extern "C"
