#include "package.h"

#include "digest.h"

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <limits>
#include <map>
#include <string_view>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace agi {
namespace {

constexpr std::size_t kFileShaAt = offsetof(wire::AimHeader, file_sha);
static_assert(kFileShaAt == 136);

bool Inside(std::size_t total, std::uint64_t offset, std::uint64_t size) {
  return offset >= sizeof(wire::AimHeader) && size > 0 && offset <= total && size <= total - offset;
}

bool SameDigest(const Digest& got, const std::uint8_t want[32]) {
  unsigned diff = 0;
  for (int i = 0; i < 32; ++i) diff |= got[i] ^ want[i];
  return diff == 0;
}

bool AnySet(const std::uint8_t* p, std::size_t n) {
  return std::any_of(p, p + n, [](std::uint8_t b) { return b != 0; });
}

struct Span {
  std::uint64_t offset, size;
  bool operator<(const Span& o) const { return offset != o.offset ? offset < o.offset : size < o.size; }
};

}  // namespace

std::uint32_t HostPlatformId() {
#if defined(__linux__) && defined(__x86_64__)
  return 1;
#elif defined(__linux__) && defined(__aarch64__)
  return 2;
#else
  return 0;
#endif
}

const char* HostPlatformName() {
  switch (HostPlatformId()) {
    case 1: return "linux-x86_64-gnu";
    case 2: return "linux-aarch64-sbsa";
    default: return "unsupported";
  }
}

bool ArchAllowedOn(std::uint32_t platform, std::uint32_t arch) {
  if (platform == 1) return arch == 89 || arch == 100 || arch == 120;
  if (platform == 2) return arch == 110;
  return false;
}

bool LooksLikePtx(const std::uint8_t* data, std::size_t size) {
  const std::string_view head(reinterpret_cast<const char*>(data), std::min<std::size_t>(size, 1u << 20));
  for (std::string_view marker : {".version ", ".target sm_", ".entry ", ".visible .entry"})
    if (head.find(marker) != std::string_view::npos) return true;
  return false;
}

bool IsCubinFor(const std::uint8_t* d, std::size_t size, std::uint32_t arch) {
  static constexpr std::uint8_t kElf64Le[7] = {0x7f, 'E', 'L', 'F', 2, 1, 1};
  if (size < 64 || std::memcmp(d, kElf64Le, 7) != 0) return false;
  const std::uint32_t machine = d[18] | d[19] << 8;
  if (machine != 190) return false;
  const std::uint32_t flags = d[48] | d[49] << 8 | d[50] << 16 | std::uint32_t{d[51]} << 24;
  // EI_OSABI 0x41 with ABI version >= 8: architecture in bits 8-15.  Older images: bits 0-7 / 16-23.
  if (d[7] == 0x41 && d[8] >= 8) return ((flags >> 8) & 0xff) == arch;
  return (flags & 0xff) == arch || ((flags >> 16) & 0xff) == arch;
}

Package::~Package() {
  if (data_ != nullptr) munmap(const_cast<std::uint8_t*>(data_), size_);
  if (fd_ >= 0) close(fd_);
}

const wire::VariantEntry* Package::FindVariant(std::uint32_t arch) const {
  const wire::VariantEntry* hit = nullptr;
  for (std::uint32_t i = 0; i < header().variant_count; ++i)
    if (variants()[i].arch == arch) hit = &variants()[i];
  return hit;
}

Status Package::Open(const std::string& path, std::unique_ptr<Package>* out) {
  std::unique_ptr<Package> pkg(new Package);
  pkg->fd_ = open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (pkg->fd_ < 0)
    return Status(errno == ENOENT ? kNotFound : kIoError, "cannot open AIM: " + std::string(std::strerror(errno)));
  struct stat st {};
  if (fstat(pkg->fd_, &st) != 0 || st.st_size < static_cast<off_t>(sizeof(wire::AimHeader)))
    return Status(kCorruptPackage, "AIM is smaller than its fixed header");
  pkg->size_ = static_cast<std::size_t>(st.st_size);
  void* mapped = mmap(nullptr, pkg->size_, PROT_READ, MAP_PRIVATE, pkg->fd_, 0);
  if (mapped == MAP_FAILED) return Status(kIoError, "cannot mmap AIM");
  pkg->data_ = static_cast<const std::uint8_t*>(mapped);
  madvise(mapped, pkg->size_, MADV_SEQUENTIAL);
  const std::uint8_t* base = pkg->data_;
  const std::size_t total = pkg->size_;
  const wire::AimHeader& h = pkg->header();

  if (std::memcmp(h.magic, "AIMAOT1\0", 8) != 0) return Status(kCorruptPackage, "bad AIM magic");
  if (h.schema_major != 1 || h.header_size != sizeof(wire::AimHeader) || h.endian_tag != 0x01020304u)
    return Status(kCorruptPackage, "unsupported AIM schema, header, or byte order");
  if (h.runtime_abi != kRuntimeAbi) return Status(kIncompatibleAbi, "AIM Runtime ABI mismatch");
  if (h.platform != HostPlatformId())
    return Status(kIncompatiblePlatform, std::string("AIM platform does not match host ") + HostPlatformName());
  if (h.file_size != total || !Inside(total, h.manifest_offset, h.manifest_size) ||
      !Inside(total, h.graph_offset, h.graph_size) || !Inside(total, h.tensor_offset, h.tensor_size) ||
      !Inside(total, h.directory_offset, h.directory_size) ||
      h.directory_size != std::uint64_t{h.variant_count} * sizeof(wire::VariantEntry))
    return Status(kCorruptPackage, "invalid AIM section bounds");

  // Whole-file digest on its own thread while this thread checks the sections.
  Digest file_digest{};
  std::thread whole([&] {
    Sha256 hash;
    static constexpr std::uint8_t kZeros[32] = {};
    hash.Update(base, kFileShaAt);
    hash.Update(kZeros, 32);
    hash.Update(base + kFileShaAt + 32, total - kFileShaAt - 32);
    file_digest = hash.Finish();
  });
  struct Joiner {
    std::thread& t;
    ~Joiner() { if (t.joinable()) t.join(); }
  } joiner{whole};

  if (!SameDigest(Sha256::Of(base + h.directory_offset, h.directory_size), h.directory_sha) ||
      !SameDigest(Sha256::Of(base + h.manifest_offset, h.manifest_size), h.manifest_sha) ||
      !SameDigest(Sha256::Of(base + h.graph_offset, h.graph_size), h.graph_sha))
    return Status(kCorruptPackage, "AIM metadata checksum mismatch");

  // Structural checks of every variant first (cheap), then payload digests, each distinct
  // region hashed once even when several variants share it.
  const wire::VariantEntry* variants = pkg->variants();
  Status deferred;  // first failure in directory order
  std::map<Span, Digest> digests;
  for (std::uint32_t i = 0; i < h.variant_count && deferred.ok(); ++i) {
    const wire::VariantEntry& v = variants[i];
    const bool layout_ok = ArchAllowedOn(h.platform, v.arch) && v.flags == 0 && !AnySet(v.reserved, sizeof v.reserved) &&
                           v.kernel_offset % 256 == 0 && v.weight_offset % 256 == 0 && v.plan_offset % 256 == 0 &&
                           Inside(total, v.kernel_offset, v.kernel_size) && Inside(total, v.weight_offset, v.weight_size) &&
                           Inside(total, v.plan_offset, v.plan_size);
    if (!layout_ok) {
      deferred = Status(kCorruptPackage, "invalid variant or payload checksum");
      break;
    }
    const Span spans[3] = {{v.kernel_offset, v.kernel_size}, {v.weight_offset, v.weight_size}, {v.plan_offset, v.plan_size}};
    const std::uint8_t* wants[3] = {v.kernel_sha, v.weight_sha, v.plan_sha};
    for (int s = 0; s < 3 && deferred.ok(); ++s) {
      auto it = digests.find(spans[s]);
      if (it == digests.end()) it = digests.emplace(spans[s], Sha256::Of(base + spans[s].offset, spans[s].size)).first;
      if (!SameDigest(it->second, wants[s])) deferred = Status(kCorruptPackage, "invalid variant or payload checksum");
    }
    if (!deferred.ok()) break;
    if (LooksLikePtx(base + v.kernel_offset, v.kernel_size))
      deferred = Status(kCorruptPackage, "PTX in an AIM kernel bundle is forbidden");
    else if (!IsCubinFor(base + v.kernel_offset, v.kernel_size, v.arch))
      deferred = Status(kCorruptPackage, "kernel bundle is not an exact-architecture NVIDIA CUBIN");
    else
      for (std::uint32_t j = 0; j < i; ++j)
        if (variants[j].arch == v.arch) deferred = Status(kCorruptPackage, "duplicate CUDA architecture variant");
  }

  whole.join();
  // Report in the reference's order: file digest, header reserved bytes, then variants.
  if (!SameDigest(file_digest, h.file_sha)) return Status(kCorruptPackage, "AIM file checksum mismatch");
  if (AnySet(h.reserved, sizeof h.reserved)) return Status(kCorruptPackage, "non-zero AIM reserved bytes");
  if (!deferred.ok()) return deferred;
  pkg->manifest_.assign(reinterpret_cast<const char*>(base + h.manifest_offset), h.manifest_size);
  madvise(mapped, pkg->size_, MADV_NORMAL);
  *out = std::move(pkg);
  return {};
}

Status ManifestUnsigned(const std::string& json, const std::string& key, std::uint64_t* out) {
  const std::string needle = "\"" + key + "\"";
  std::size_t at = json.find(needle);
  if (at == std::string::npos) return Status(kCorruptPackage, "manifest missing " + key);
  at = json.find(':', at + needle.size());
  if (at == std::string::npos) return Status(kCorruptPackage, "invalid manifest field " + key);
  ++at;
  while (at < json.size() && (json[at] == ' ' || json[at] == '\t')) ++at;
  std::uint64_t value = 0;
  bool any = false;
  for (; at < json.size() && json[at] >= '0' && json[at] <= '9'; ++at) {
    const unsigned digit = static_cast<unsigned>(json[at] - '0');
    if (value > (std::numeric_limits<std::uint64_t>::max() - digit) / 10)
      return Status(kCorruptPackage, "overflow in manifest field " + key);
    value = value * 10 + digit;
    any = true;
  }
  if (!any) return Status(kCorruptPackage, "invalid manifest integer " + key);
  *out = value;
  return {};
}

}  // namespace agi
