// A memory-mapped, fully verified AIM v1 package (the loader's `Model`).
// Layout and checks follow docs/aim-v1.md and the reference's Model::Load
// (cpp/runtime.cc:23-112, 373-425), with two additions: the sm100 target row and the
// CUBIN flavour nvcc >= 12.8 emits for sm_100 / sm_120 (architecture in e_flags bits 8-15).
// Integrity hashing runs the whole-file digest and the per-section digests on separate
// threads, so a load costs one pass over the file in wall time instead of two.
#pragma once

#include "status.h"

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

namespace agi {

namespace wire {
#pragma pack(push, 1)
struct AimHeader {
  char magic[8];
  std::uint16_t schema_major, schema_minor;
  std::uint32_t header_size, runtime_abi, platform, endian_tag, variant_count;
  std::uint64_t file_size, manifest_offset, manifest_size, graph_offset, graph_size, tensor_offset, tensor_size,
      directory_offset, directory_size;
  std::uint8_t directory_sha[32], file_sha[32], manifest_sha[32], graph_sha[32], reserved[24];
};
struct VariantEntry {
  std::uint32_t arch, flags;
  std::uint64_t kernel_offset, kernel_size, weight_offset, weight_size, plan_offset, plan_size;
  std::uint8_t kernel_sha[32], weight_sha[32], plan_sha[32], reserved[40];
};
#pragma pack(pop)
static_assert(sizeof(AimHeader) == 256 && sizeof(VariantEntry) == 192);
}  // namespace wire

constexpr std::uint32_t kRuntimeAbi = 1;

std::uint32_t HostPlatformId();          // 1 = linux-x86_64-gnu, 2 = linux-aarch64-sbsa, 0 = other
const char* HostPlatformName();
bool ArchAllowedOn(std::uint32_t platform, std::uint32_t arch);
bool LooksLikePtx(const std::uint8_t* data, std::size_t size);
// True when `data` is an NVIDIA CUDA ELF image built for exactly `arch`.
bool IsCubinFor(const std::uint8_t* data, std::size_t size, std::uint32_t arch);

class Package {
 public:
  ~Package();
  Package(const Package&) = delete;
  Package& operator=(const Package&) = delete;

  static Status Open(const std::string& path, std::unique_ptr<Package>* out);

  const std::uint8_t* data() const { return data_; }
  std::size_t size() const { return size_; }
  const wire::AimHeader& header() const { return *reinterpret_cast<const wire::AimHeader*>(data_); }
  const wire::VariantEntry* variants() const {
    return reinterpret_cast<const wire::VariantEntry*>(data_ + header().directory_offset);
  }
  const wire::VariantEntry* FindVariant(std::uint32_t arch) const;
  const std::string& manifest() const { return manifest_; }

 private:
  Package() = default;
  int fd_ = -1;
  const std::uint8_t* data_ = nullptr;
  std::size_t size_ = 0;
  std::string manifest_;
};

// Reads the unsigned integer stored under `"key":` anywhere in a JSON text.
Status ManifestUnsigned(const std::string& json, const std::string& key, std::uint64_t* out);

}  // namespace agi
