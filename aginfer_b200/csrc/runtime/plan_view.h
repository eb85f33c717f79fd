// Read-only view of a binary AIMPLN1 execution plan, validated in full before use.
// Record layouts are the wire format of the reference (cpp/plan.h:26-95); the checks are
// those of its ParsePlan / ValidateTensor (cpp/plan.cc:43-239).
#pragma once

#include "status.h"

#include <cstddef>
#include <cstdint>
#include <string_view>

namespace agi {

constexpr std::uint32_t kMaxRank = 8;

namespace wire {
enum DType : std::uint32_t { kF32 = 1, kF16 = 2, kBF16 = 3, kF8E4M3 = 4, kI32 = 5 };
enum Location : std::uint32_t { kHost = 1, kDevice = 2 };
enum IoKind : std::uint32_t { kInput = 1, kOutput = 2 };
enum ArgKind : std::uint32_t { kTensor = 1, kScalarU32 = 2, kScalarF32 = 3, kArenaOffset = 4, kWeightsOffset = 5 };

#pragma pack(push, 1)
struct PlanHeader {
  char magic[8];
  std::uint16_t schema_major, schema_minor;
  std::uint32_t header_size, arch, profile_count, tensor_count, launch_count, argument_count, string_bytes;
  std::uint64_t arena_bytes, workspace_bytes;
  std::uint64_t profiles_offset, tensors_offset, launches_offset, arguments_offset, strings_offset, file_size;
  std::uint8_t reserved[24];
};
struct Profile {
  std::uint32_t name, first_tensor, tensor_count, first_launch, launch_count, flags;
  std::uint8_t reserved[40];
};
struct Tensor {
  std::uint32_t name, dtype, location, io_kind, rank, flags;
  std::uint64_t byte_size;
  std::int64_t shape[kMaxRank];
  std::int64_t stride[kMaxRank];
};
struct Launch {
  std::uint32_t kernel, profile, first_argument, argument_count;
  std::uint32_t grid[3], block[3];
  std::uint32_t shared_bytes, flags;
  std::uint8_t reserved[16];
};
struct Argument {
  std::uint32_t kind, index;
  std::uint64_t offset, value, reserved;
};
#pragma pack(pop)
static_assert(sizeof(PlanHeader) == 128 && sizeof(Profile) == 64 && sizeof(Tensor) == 160 &&
              sizeof(Launch) == 64 && sizeof(Argument) == 32);
}  // namespace wire

struct PlanView {
  const wire::PlanHeader* header = nullptr;
  const wire::Profile* profiles = nullptr;
  const wire::Tensor* tensors = nullptr;
  const wire::Launch* launches = nullptr;
  const wire::Argument* arguments = nullptr;
  const char* strings = nullptr;

  // NUL-terminated entry of the string table; empty view when out of range or unterminated.
  std::string_view Text(std::uint32_t offset) const;
  const wire::Profile* Find(std::string_view profile_name) const;
};

// Validates `size` bytes at `data` as the plan of a variant built for `arch` whose weight
// blob holds `weight_bytes` bytes.  On success `*out` points into `data`.
Status OpenPlan(const std::uint8_t* data, std::size_t size, std::uint32_t arch, std::uint64_t weight_bytes,
                PlanView* out);

std::uint64_t DTypeBytes(std::uint32_t wire_dtype);

}  // namespace agi
