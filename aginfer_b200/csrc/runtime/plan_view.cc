#include "plan_view.h"

#include <cstring>
#include <limits>
#include <string>

namespace agi {
namespace {

constexpr std::uint64_t kU64Max = std::numeric_limits<std::uint64_t>::max();

Status Bad(std::string text) { return Status(kCorruptPackage, std::move(text)); }

bool Zero(const std::uint8_t* p, std::size_t n) {
  for (std::size_t i = 0; i < n; ++i)
    if (p[i] != 0) return false;
  return true;
}

// [offset, offset + count * item) lies inside [0, total)
bool TableFits(std::size_t total, std::uint64_t offset, std::uint64_t count, std::size_t item) {
  return offset <= total && count <= (total - offset) / item;
}

bool RangeFits(std::uint32_t total, std::uint32_t first, std::uint32_t count) {
  return first <= total && count <= total - first;
}

Status CheckTensor(const PlanView& plan, const wire::Tensor& t, std::uint32_t index) {
  const std::string where = "execution plan tensor " + std::to_string(index);
  if (plan.Text(t.name).empty()) return Bad(where + " has an invalid name");
  const std::uint64_t item = DTypeBytes(t.dtype);
  if (item == 0) return Bad(where + " has an invalid dtype");
  if (t.location != wire::kHost && t.location != wire::kDevice) return Bad(where + " has an invalid location");
  if (t.io_kind != wire::kInput && t.io_kind != wire::kOutput) return Bad(where + " has an invalid I/O kind");
  if (t.rank == 0 || t.rank > kMaxRank || t.flags != 0) return Bad(where + " has an invalid rank or flags");
  std::uint64_t last = 0;  // index of the last addressed element
  for (std::uint32_t d = 0; d < kMaxRank; ++d) {
    if (d >= t.rank) {
      if (t.shape[d] != 0 || t.stride[d] != 0) return Bad("execution plan tensor has non-zero dimensions beyond its rank");
      continue;
    }
    if (t.shape[d] <= 0 || t.stride[d] <= 0) return Bad(where + " has a non-positive shape or stride");
    const auto steps = static_cast<std::uint64_t>(t.shape[d] - 1);
    const auto stride = static_cast<std::uint64_t>(t.stride[d]);
    if (steps != 0 && stride > (kU64Max - last) / steps) return Bad("execution plan tensor size overflows");
    last += steps * stride;
  }
  if (last == kU64Max || last + 1 > kU64Max / item || t.byte_size < (last + 1) * item)
    return Bad("execution plan tensor byte size is too small");
  return {};
}

Status CheckArgument(const wire::PlanHeader& h, const PlanView& plan, const wire::Profile& profile,
                     const wire::Argument& a, std::uint64_t weight_bytes) {
  if (a.reserved != 0) return Bad("execution plan argument has non-zero reserved data");
  switch (a.kind) {
    case wire::kTensor:
      if (a.index < profile.first_tensor || a.index >= profile.first_tensor + profile.tensor_count ||
          plan.tensors[a.index].location != wire::kDevice)
        return Bad("execution plan launch references an invalid device tensor");
      if (a.offset != 0 || a.value != 0) return Bad("execution plan tensor argument has unexpected payload data");
      return {};
    case wire::kScalarU32:
    case wire::kScalarF32:
      if (a.index != 0 || a.offset != 0 || a.value > std::numeric_limits<std::uint32_t>::max())
        return Bad("execution plan scalar argument is out of range");
      return {};
    case wire::kArenaOffset:
      if (a.index != 0 || a.value != 0 || a.offset >= h.arena_bytes)
        return Bad("execution plan arena argument is out of bounds");
      return {};
    case wire::kWeightsOffset:
      if (a.index != 0 || a.value != 0 || a.offset >= weight_bytes)
        return Bad("execution plan weight argument is out of bounds");
      return {};
    default:
      return Bad("execution plan contains an unknown argument kind");
  }
}

}  // namespace

std::uint64_t DTypeBytes(std::uint32_t dtype) {
  switch (dtype) {
    case wire::kF32: case wire::kI32: return 4;
    case wire::kF16: case wire::kBF16: return 2;
    case wire::kF8E4M3: return 1;
    default: return 0;
  }
}

std::string_view PlanView::Text(std::uint32_t offset) const {
  if (header == nullptr || offset >= header->string_bytes) return {};
  const char* begin = strings + offset;
  const void* end = std::memchr(begin, 0, header->string_bytes - offset);
  if (end == nullptr) return {};
  return {begin, static_cast<std::size_t>(static_cast<const char*>(end) - begin)};
}

const wire::Profile* PlanView::Find(std::string_view profile_name) const {
  if (header == nullptr) return nullptr;
  for (std::uint32_t i = 0; i < header->profile_count; ++i)
    if (Text(profiles[i].name) == profile_name) return &profiles[i];
  return nullptr;
}

Status OpenPlan(const std::uint8_t* data, std::size_t size, std::uint32_t arch, std::uint64_t weight_bytes,
                PlanView* out) {
  if (data == nullptr || out == nullptr || size < sizeof(wire::PlanHeader))
    return Bad("execution plan is smaller than its fixed header");
  const auto& h = *reinterpret_cast<const wire::PlanHeader*>(data);
  if (std::memcmp(h.magic, "AIMPLN1\0", 8) != 0) return Bad("bad AIM execution plan magic");
  if (h.schema_major != 1 || h.header_size != sizeof(wire::PlanHeader))
    return Bad("unsupported AIM execution plan schema");
  if (h.arch != arch) return Bad("execution plan architecture does not match its AIM variant");
  if (h.file_size != size || !Zero(h.reserved, sizeof h.reserved))
    return Bad("invalid execution plan size or reserved bytes");
  if (h.profile_count == 0 || h.tensor_count == 0 || h.launch_count == 0)
    return Bad("execution plan must contain profiles, tensors, and launches");
  if (!TableFits(size, h.profiles_offset, h.profile_count, sizeof(wire::Profile)) ||
      !TableFits(size, h.tensors_offset, h.tensor_count, sizeof(wire::Tensor)) ||
      !TableFits(size, h.launches_offset, h.launch_count, sizeof(wire::Launch)) ||
      !TableFits(size, h.arguments_offset, h.argument_count, sizeof(wire::Argument)) ||
      !TableFits(size, h.strings_offset, h.string_bytes, 1) || h.string_bytes == 0 ||
      h.strings_offset + h.string_bytes != size)
    return Bad("execution plan contains an invalid table region");
  // Tables must follow one another with no gaps, in this order.
  std::uint64_t cursor = sizeof(wire::PlanHeader);
  const std::uint64_t starts[5] = {h.profiles_offset, h.tensors_offset, h.launches_offset, h.arguments_offset,
                                   h.strings_offset};
  const std::uint64_t extents[4] = {std::uint64_t{h.profile_count} * sizeof(wire::Profile),
                                    std::uint64_t{h.tensor_count} * sizeof(wire::Tensor),
                                    std::uint64_t{h.launch_count} * sizeof(wire::Launch),
                                    std::uint64_t{h.argument_count} * sizeof(wire::Argument)};
  for (int i = 0; i < 5; ++i) {
    if (starts[i] != cursor) return Bad("execution plan tables are not in canonical order");
    if (i < 4) cursor += extents[i];
  }

  PlanView plan;
  plan.header = &h;
  plan.profiles = reinterpret_cast<const wire::Profile*>(data + h.profiles_offset);
  plan.tensors = reinterpret_cast<const wire::Tensor*>(data + h.tensors_offset);
  plan.launches = reinterpret_cast<const wire::Launch*>(data + h.launches_offset);
  plan.arguments = reinterpret_cast<const wire::Argument*>(data + h.arguments_offset);
  plan.strings = reinterpret_cast<const char*>(data + h.strings_offset);
  if (plan.strings[0] != '\0') return Bad("execution plan string table has an invalid sentinel");

  std::uint32_t tensors_seen = 0, launches_seen = 0;
  for (std::uint32_t p = 0; p < h.profile_count; ++p) {
    const wire::Profile& profile = plan.profiles[p];
    if (plan.Text(profile.name).empty() || profile.first_tensor != tensors_seen ||
        profile.first_launch != launches_seen || profile.tensor_count == 0 || profile.launch_count == 0 ||
        !RangeFits(h.tensor_count, profile.first_tensor, profile.tensor_count) ||
        !RangeFits(h.launch_count, profile.first_launch, profile.launch_count) || (profile.flags & ~1u) != 0 ||
        !Zero(profile.reserved, sizeof profile.reserved))
      return Bad("execution plan contains an invalid profile record");
    for (std::uint32_t q = 0; q < p; ++q)
      if (plan.Text(plan.profiles[q].name) == plan.Text(profile.name))
        return Bad("execution plan contains duplicate profile names");
    tensors_seen += profile.tensor_count;
    launches_seen += profile.launch_count;
  }
  if (tensors_seen != h.tensor_count || launches_seen != h.launch_count)
    return Bad("execution plan profile ranges do not cover their tables");

  for (std::uint32_t t = 0; t < h.tensor_count; ++t) AGI_RETURN_IF_ERROR(CheckTensor(plan, plan.tensors[t], t));
  for (std::uint32_t p = 0; p < h.profile_count; ++p) {
    const wire::Profile& profile = plan.profiles[p];
    std::uint32_t inputs = 0;
    for (std::uint32_t i = 0; i < profile.tensor_count; ++i) {
      const wire::Tensor& t = plan.tensors[profile.first_tensor + i];
      inputs += t.io_kind == wire::kInput;
      for (std::uint32_t j = 0; j < i; ++j)
        if (plan.Text(plan.tensors[profile.first_tensor + j].name) == plan.Text(t.name))
          return Bad("execution plan profile contains duplicate tensor names");
    }
    if (inputs == 0 || inputs == profile.tensor_count)
      return Bad("execution plan profile must contain inputs and outputs");
  }

  std::uint32_t arguments_seen = 0;
  for (std::uint32_t l = 0; l < h.launch_count; ++l) {
    const wire::Launch& launch = plan.launches[l];
    bool dims_ok = true;
    for (int d = 0; d < 3; ++d) dims_ok = dims_ok && launch.grid[d] != 0 && launch.block[d] != 0;
    if (launch.profile >= h.profile_count || plan.Text(launch.kernel).empty() ||
        launch.first_argument != arguments_seen ||
        !RangeFits(h.argument_count, launch.first_argument, launch.argument_count) || !dims_ok ||
        std::uint64_t{launch.block[0]} * launch.block[1] * launch.block[2] > 1024 || launch.flags != 0 ||
        !Zero(launch.reserved, sizeof launch.reserved))
      return Bad("execution plan contains an invalid launch record");
    const wire::Profile& profile = plan.profiles[launch.profile];
    if (l < profile.first_launch || l >= profile.first_launch + profile.launch_count)
      return Bad("execution plan launch belongs to the wrong profile");
    for (std::uint32_t a = 0; a < launch.argument_count; ++a)
      AGI_RETURN_IF_ERROR(CheckArgument(h, plan, profile, plan.arguments[launch.first_argument + a], weight_bytes));
    arguments_seen += launch.argument_count;
  }
  if (arguments_seen != h.argument_count) return Bad("execution plan launch ranges do not cover the argument table");
  *out = plan;
  return {};
}

}  // namespace agi
