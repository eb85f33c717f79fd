// SHA-256 for package integrity checks (role of the reference's cpp/sha256.{h,cc}).
// One streaming hasher; the block function is chosen once per process: x86 SHA
// extensions when the CPU has them, portable code otherwise.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>

namespace agi {

using Digest = std::array<std::uint8_t, 32>;

class Sha256 {
 public:
  Sha256();
  void Update(const void* data, std::size_t size);
  Digest Finish();

  static Digest Of(const void* data, std::size_t size) {
    Sha256 h;
    h.Update(data, size);
    return h.Finish();
  }
  // One-shot digest through the portable block function, whatever the CPU offers (tests).
  static Digest PortableOf(const void* data, std::size_t size);
  // Name of the block function in use ("sha-ni" or "portable"); for diagnostics and tests.
  static const char* Backend();

 private:
  std::uint32_t state_[8];
  std::uint8_t tail_[64];
  std::size_t tail_size_ = 0;
  std::uint64_t total_ = 0;
};

}  // namespace agi
