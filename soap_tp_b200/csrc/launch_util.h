// Host-side launch helpers shared by the kernels of this library.
#pragma once
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

namespace soapb200 {

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel: a process that
// drives several GPUs has to raise it on each of them before the first launch there.  One instance of
// this struct per kernel (a function-local static at the launch site) remembers which devices are done.
struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  bool done[kMaxDevices] = {};
};

inline void allow_dynamic_smem(const void* kernel, size_t bytes, PerDeviceOnce& once, const char* what) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": cudaGetDevice: " + cudaGetErrorString(err));
  const bool tracked = device >= 0 && device < PerDeviceOnce::kMaxDevices;
  if (tracked && once.done[device]) return;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + " attribute: " + cudaGetErrorString(err));
  if (tracked) once.done[device] = true;
}

}  // namespace soapb200
