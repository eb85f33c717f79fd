#include "digest.h"

#include <cstring>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

namespace agi {
namespace {

constexpr std::uint32_t kRound[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

inline std::uint32_t Rotr(std::uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

void BlocksPortable(std::uint32_t state[8], const std::uint8_t* p, std::size_t blocks) {
  std::uint32_t w[64];
  for (; blocks != 0; --blocks, p += 64) {
    for (int i = 0; i < 16; ++i)
      w[i] = std::uint32_t{p[4 * i]} << 24 | std::uint32_t{p[4 * i + 1]} << 16 | std::uint32_t{p[4 * i + 2]} << 8 |
             std::uint32_t{p[4 * i + 3]};
    for (int i = 16; i < 64; ++i) {
      const std::uint32_t s0 = Rotr(w[i - 15], 7) ^ Rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const std::uint32_t s1 = Rotr(w[i - 2], 17) ^ Rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    std::uint32_t a = state[0], b = state[1], c = state[2], d = state[3];
    std::uint32_t e = state[4], f = state[5], g = state[6], h = state[7];
    for (int i = 0; i < 64; ++i) {
      const std::uint32_t t1 = h + (Rotr(e, 6) ^ Rotr(e, 11) ^ Rotr(e, 25)) + ((e & f) ^ (~e & g)) + kRound[i] + w[i];
      const std::uint32_t t2 = (Rotr(a, 2) ^ Rotr(a, 13) ^ Rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    state[0] += a; state[1] += b; state[2] += c; state[3] += d;
    state[4] += e; state[5] += f; state[6] += g; state[7] += h;
  }
}

#if defined(__x86_64__)
// Four rounds per step with the SHA extensions; message schedule kept in four xmm registers.
__attribute__((target("sha,sse4.1,ssse3")))
void BlocksShaNi(std::uint32_t state[8], const std::uint8_t* p, std::size_t blocks) {
  const __m128i shuffle = _mm_set_epi64x(0x0c0d0e0f08090a0bULL, 0x0405060700010203ULL);
  __m128i tmp = _mm_loadu_si128(reinterpret_cast<const __m128i*>(state));        // a b c d
  __m128i st1 = _mm_loadu_si128(reinterpret_cast<const __m128i*>(state + 4));    // e f g h
  tmp = _mm_shuffle_epi32(tmp, 0xB1);                                            // c d a b
  st1 = _mm_shuffle_epi32(st1, 0x1B);                                            // h g f e
  __m128i st0 = _mm_alignr_epi8(tmp, st1, 8);                                    // a b e f
  st1 = _mm_blend_epi16(st1, tmp, 0xF0);                                         // c d g h
  const __m128i* k = reinterpret_cast<const __m128i*>(kRound);
  for (; blocks != 0; --blocks, p += 64) {
    const __m128i save0 = st0, save1 = st1;
    __m128i m[4];
    for (int i = 0; i < 4; ++i)
      m[i] = _mm_shuffle_epi8(_mm_loadu_si128(reinterpret_cast<const __m128i*>(p + 16 * i)), shuffle);
    for (int r = 0; r < 16; ++r) {
      __m128i cur = m[r & 3];
      __m128i wk = _mm_add_epi32(cur, _mm_loadu_si128(k + r));
      st1 = _mm_sha256rnds2_epu32(st1, st0, wk);
      st0 = _mm_sha256rnds2_epu32(st0, st1, _mm_shuffle_epi32(wk, 0x0E));
      if (r < 12) {
        // w[r+4] = msg2(msg1(w[r], w[r+1]) + alignr(w[r+3], w[r+2]), w[r+3])
        __m128i next = _mm_sha256msg1_epu32(cur, m[(r + 1) & 3]);
        next = _mm_add_epi32(next, _mm_alignr_epi8(m[(r + 3) & 3], m[(r + 2) & 3], 4));
        m[r & 3] = _mm_sha256msg2_epu32(next, m[(r + 3) & 3]);
      }
    }
    st0 = _mm_add_epi32(st0, save0);
    st1 = _mm_add_epi32(st1, save1);
  }
  tmp = _mm_shuffle_epi32(st0, 0x1B);                                            // f e b a
  st1 = _mm_shuffle_epi32(st1, 0xB1);                                            // d c h g
  st0 = _mm_blend_epi16(tmp, st1, 0xF0);                                         // d c b a
  st1 = _mm_alignr_epi8(st1, tmp, 8);                                            // h g f e
  _mm_storeu_si128(reinterpret_cast<__m128i*>(state), st0);
  _mm_storeu_si128(reinterpret_cast<__m128i*>(state + 4), st1);
}
#endif

using BlockFn = void (*)(std::uint32_t*, const std::uint8_t*, std::size_t);

BlockFn Choose() {
#if defined(__x86_64__)
  if (__builtin_cpu_supports("sha") && __builtin_cpu_supports("sse4.1") && __builtin_cpu_supports("ssse3"))
    return BlocksShaNi;
#endif
  return BlocksPortable;
}

BlockFn Blocks() {
  static const BlockFn fn = Choose();
  return fn;
}

}  // namespace

Digest Sha256::PortableOf(const void* data, std::size_t size) {
  // Same padding rule as Finish(), driven through the portable block function only.
  std::uint32_t state[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  const auto* p = static_cast<const std::uint8_t*>(data);
  BlocksPortable(state, p, size / 64);
  std::uint8_t last[128] = {};
  const std::size_t rest = size % 64;
  std::memcpy(last, p + size - rest, rest);
  last[rest] = 0x80;
  const std::size_t padded = rest < 56 ? 64 : 128;
  const std::uint64_t bits = static_cast<std::uint64_t>(size) * 8;
  for (int i = 0; i < 8; ++i) last[padded - 8 + i] = static_cast<std::uint8_t>(bits >> (56 - 8 * i));
  BlocksPortable(state, last, padded / 64);
  Digest out;
  for (int i = 0; i < 8; ++i)
    for (int j = 0; j < 4; ++j) out[4 * i + j] = static_cast<std::uint8_t>(state[i] >> (24 - 8 * j));
  return out;
}

const char* Sha256::Backend() { return Blocks() == BlocksPortable ? "portable" : "sha-ni"; }

Sha256::Sha256()
    : state_{0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19} {}

void Sha256::Update(const void* data, std::size_t size) {
  const auto* p = static_cast<const std::uint8_t*>(data);
  total_ += size;
  if (tail_size_ != 0) {
    const std::size_t take = size < 64 - tail_size_ ? size : 64 - tail_size_;
    std::memcpy(tail_ + tail_size_, p, take);
    tail_size_ += take; p += take; size -= take;
    if (tail_size_ < 64) return;
    Blocks()(state_, tail_, 1);
    tail_size_ = 0;
  }
  if (size >= 64) {
    Blocks()(state_, p, size / 64);
    p += size & ~std::size_t{63};
    size &= 63;
  }
  if (size != 0) {
    std::memcpy(tail_, p, size);
    tail_size_ = size;
  }
}

Digest Sha256::Finish() {
  const std::uint64_t bits = total_ * 8;
  std::uint8_t pad[72] = {0x80};
  const std::size_t pad_size = (tail_size_ < 56 ? 56 : 120) - tail_size_;
  for (int i = 0; i < 8; ++i) pad[pad_size + i] = static_cast<std::uint8_t>(bits >> (56 - 8 * i));
  Update(pad, pad_size + 8);
  Digest out;
  for (int i = 0; i < 8; ++i)
    for (int j = 0; j < 4; ++j) out[4 * i + j] = static_cast<std::uint8_t>(state_[i] >> (24 - 8 * j));
  return out;
}

}  // namespace agi
