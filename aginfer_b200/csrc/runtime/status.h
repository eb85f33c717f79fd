// Result type shared by the loader's internals.  Codes and their numbering are the
// reference's StatusCode (include/aginfer/runtime.h:14-25); they cross the C boundary as ints.
#pragma once

#include <string>
#include <utility>

namespace agi {

enum Code : int {
  kOk = 0,
  kInvalidArgument = 1,
  kNotFound = 2,
  kIoError = 3,
  kCorruptPackage = 4,
  kIncompatiblePlatform = 5,
  kIncompatibleArchitecture = 6,
  kIncompatibleAbi = 7,
  kCudaError = 8,
  kOutOfMemory = 9,
};

struct Status {
  Code code = kOk;
  std::string message;
  Status() = default;
  Status(Code c, std::string m) : code(c), message(std::move(m)) {}
  bool ok() const { return code == kOk; }
};

inline const char* CodeName(int code) {
  switch (code) {
    case kOk: return "OK";
    case kInvalidArgument: return "INVALID_ARGUMENT";
    case kNotFound: return "NOT_FOUND";
    case kIoError: return "IO_ERROR";
    case kCorruptPackage: return "CORRUPT_PACKAGE";
    case kIncompatiblePlatform: return "INCOMPATIBLE_PLATFORM";
    case kIncompatibleArchitecture: return "INCOMPATIBLE_ARCHITECTURE";
    case kIncompatibleAbi: return "INCOMPATIBLE_ABI";
    case kCudaError: return "CUDA_ERROR";
    case kOutOfMemory: return "OUT_OF_MEMORY";
  }
  return "UNKNOWN";
}

#define AGI_RETURN_IF_ERROR(expr)            \
  do {                                       \
    ::agi::Status agi_status_ = (expr);      \
    if (!agi_status_.ok()) return agi_status_; \
  } while (0)

}  // namespace agi
