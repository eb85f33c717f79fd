// Drives the reference's C++ runtime, carrying oracle/ref_sm100.patch (target row for sm_100, the new CUBIN
// ELF flavour, the > 48 KB shared-memory opt-in), through a real Session::Enqueue on the current GPU.
// Test infrastructure: a GPU test feeds it one of this repository's sm100 packages and compares what the
// reference's own launch loop produces with what this repository's loader produces.
//
//   ref_probe_gpu <file.aim> <profile> <manifest.txt> [repeats]
//
// manifest lines:  in|out  <name>  <dtype 0..4>  <file of raw bytes>  <dim> [<dim> ...]
// Inputs are read from their files, outputs written to theirs after the last run.  Prints
// "enqueue=<status name>|<message>" and, with repeats > 1, "ms_per_enqueue=<wall time between synchronisations>".
#include "aginfer/runtime.h"

#include <cuda_runtime_api.h>

#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

namespace {
struct Entry {
  bool input = false;
  std::string name, path;
  aginfer::DType dtype = aginfer::DType::kFp32;
  std::vector<std::int64_t> shape, stride;
  std::size_t bytes = 0;
  void* device = nullptr;
};
std::size_t ItemSize(aginfer::DType t) {
  switch (t) {
    case aginfer::DType::kFp32: case aginfer::DType::kInt32: return 4;
    case aginfer::DType::kFp16: case aginfer::DType::kBf16: return 2;
    default: return 1;
  }
}
aginfer::TensorView View(const Entry& e) {
  aginfer::TensorView v;
  v.name = e.name; v.dtype = e.dtype; v.shape = e.shape; v.stride = e.stride; v.data = e.device; v.byte_size = e.bytes;
  v.location = aginfer::MemoryLocation::kDevice;
  return v;
}
}  // namespace

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  const int repeats = argc > 4 ? std::atoi(argv[4]) : 1;
  std::vector<Entry> entries;
  std::ifstream manifest(argv[3]);
  for (std::string line; std::getline(manifest, line);) {
    std::istringstream in(line);
    std::string kind;
    int dtype = 0;
    Entry e;
    if (!(in >> kind >> e.name >> dtype >> e.path)) continue;
    e.input = kind == "in";
    e.dtype = static_cast<aginfer::DType>(dtype);
    for (std::int64_t d; in >> d;) e.shape.push_back(d);
    e.stride.assign(e.shape.size(), 1);
    for (std::size_t i = e.shape.size(); i-- > 1;) e.stride[i - 1] = e.stride[i] * e.shape[i];
    e.bytes = ItemSize(e.dtype);
    for (auto d : e.shape) e.bytes *= static_cast<std::size_t>(d);
    if (cudaMalloc(&e.device, e.bytes) != cudaSuccess) return 3;
    if (e.input) {
      std::ifstream raw(e.path, std::ios::binary);
      std::vector<char> host(e.bytes);
      raw.read(host.data(), static_cast<std::streamsize>(e.bytes));
      if (static_cast<std::size_t>(raw.gcount()) != e.bytes) return 4;
      if (cudaMemcpy(e.device, host.data(), e.bytes, cudaMemcpyHostToDevice) != cudaSuccess) return 5;
    } else if (cudaMemset(e.device, 0xff, e.bytes) != cudaSuccess) {
      return 5;
    }
    entries.push_back(e);
  }

  aginfer::RuntimeOptions options;               // architecture and Driver version are probed for real
  options.cuda_runtime_version_override = 12080;
  options.cublaslt_abi_override = 12;
  options.cudnn_abi_override = 9;
  auto runtime = aginfer::Runtime::Create(options);
  if (!runtime.ok()) { std::cout << "runtime=" << runtime.status().message() << "\n"; return 0; }
  auto model = aginfer::Model::Load(argv[1]);
  if (!model.ok()) { std::cout << "load=" << aginfer::StatusCodeName(model.status().code()) << "|" << model.status().message() << "\n"; return 0; }
  aginfer::SessionOptions session_options;
  session_options.profile = argv[2];
  auto session = aginfer::Session::Create(runtime.value(), model.value(), session_options);
  if (!session.ok()) { std::cout << "session=" << aginfer::StatusCodeName(session.status().code()) << "|" << session.status().message() << "\n"; return 0; }

  std::vector<aginfer::TensorView> inputs, outputs;
  for (const Entry& e : entries) (e.input ? inputs : outputs).push_back(View(e));
  cudaStream_t stream = nullptr;
  if (cudaStreamCreate(&stream) != cudaSuccess) return 6;
  aginfer::Status status = session.value().Enqueue(inputs, outputs, aginfer::RunOptions{}, stream);   // first call: set-up
  cudaStreamSynchronize(stream);
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 1; i < repeats && status.ok(); ++i) {
    status = session.value().Enqueue(inputs, outputs, aginfer::RunOptions{}, stream);
    cudaStreamSynchronize(stream);
  }
  const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  std::cout << "enqueue=" << aginfer::StatusCodeName(status.code()) << "|" << status.message() << "\n";
  if (repeats > 1) std::cout << "ms_per_enqueue=" << seconds * 1e3 / (repeats - 1) << "\n";
  const cudaError_t finished = cudaDeviceSynchronize();
  std::cout << "device=" << cudaGetErrorName(finished) << "\n";
  for (const Entry& e : entries) {
    if (e.input) continue;
    std::vector<char> host(e.bytes);
    if (cudaMemcpy(host.data(), e.device, e.bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return 7;
    std::ofstream(e.path, std::ios::binary).write(host.data(), static_cast<std::streamsize>(e.bytes));
  }
  return 0;
}
