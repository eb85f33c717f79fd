// Drives the reference's C++ runtime (linked from its own sources by oracle/Makefile) on
// one AIM file and prints what it reports, one "key=value" line each.  Test
// infrastructure: the loader tests compare this library's answers with these.
//
//   ref_probe <file.aim> <cuda_arch_override> [profile]
//
// All five RuntimeOptions overrides are set, so no CUDA library is touched (the same way
// the reference's tests/runtime_test.cc runs without a GPU).
#include "aginfer/runtime.h"

#include <cstdlib>
#include <iostream>
#include <string>

namespace {
void Print(const char* stage, const aginfer::Status& status) {
  std::cout << stage << "=" << aginfer::StatusCodeName(status.code()) << "|" << status.message() << "\n";
}
void PrintInfo(const char* kind, const std::vector<aginfer::TensorInfo>& infos) {
  for (const auto& t : infos) {
    std::cout << kind << "=" << t.name << "|" << static_cast<int>(t.dtype) << "|" << static_cast<int>(t.location) << "|"
              << t.byte_size << "|";
    for (auto v : t.shape) std::cout << v << ",";
    std::cout << "|";
    for (auto v : t.stride) std::cout << v << ",";
    std::cout << "\n";
  }
}
}  // namespace

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  auto model = aginfer::Model::Load(argv[1]);
  Print("load", model.status());
  if (!model.ok()) return 0;
  aginfer::RuntimeOptions options;
  options.cuda_arch_override = static_cast<std::uint32_t>(std::atoi(argv[2]));
  options.cuda_driver_version_override = 12080;
  options.cuda_runtime_version_override = 12080;
  options.cublaslt_abi_override = 12;
  options.cudnn_abi_override = 9;
  auto runtime = aginfer::Runtime::Create(options);
  Print("runtime", runtime.status());
  if (!runtime.ok()) return 0;
  aginfer::SessionOptions session_options;
  if (argc > 3) session_options.profile = argv[3];
  auto session = aginfer::Session::Create(runtime.value(), model.value(), session_options);
  Print("session", session.status());
  if (!session.ok()) return 0;
  const auto target = session.value().GetTargetInfo();
  std::cout << "target=" << target.platform << "|" << target.cuda_arch << "|" << target.runtime_abi << "\n";
  PrintInfo("input", session.value().GetInputInfo());
  PrintInfo("output", session.value().GetOutputInfo());
  auto workspace = session.value().GetRequiredWorkspace("");
  if (workspace.ok())
    std::cout << "workspace=" << workspace.value().arena_bytes << "|" << workspace.value().workspace_bytes << "\n";
  auto missing = session.value().GetRequiredWorkspace("no-such-profile");
  Print("workspace_missing", missing.status());
  return 0;
}
