// The calling thread's "last error" text behind agi_last_error(), for entry points that live in
// other translation units than capi.cc.
#pragma once

#include "aginfer_b200.h"

#include <string>

namespace agi {
// Stores `message` for agi_last_error() on this thread and returns `code` as an agi_status.
agi_status RecordFailure(int code, const std::string& message);
}  // namespace agi
