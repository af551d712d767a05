// Device helpers of the CUDA backend (the reference's tc/core/cuda/cuda.h:79-131), implemented on
// the tcb200 C ABI so that this library does not link the CUDA runtime itself.
#pragma once

#include <stdexcept>
#include <string>

#include "tcb200.h"

namespace tc {

// Throws std::runtime_error naming the failed call when a tcb200 status is not OK.
void tcb200Enforce(int status, const char* what);
#define TC_TCB200_ENFORCE(call) ::tc::tcb200Enforce((call), #call)

// RAII: makes `newDevice` current for the calling thread and restores the previous one.
class WithCudaDevice {
 public:
  explicit WithCudaDevice(size_t newDevice);
  ~WithCudaDevice();

 private:
  int oldDevice_ = 0;
};

struct CudaGPUInfo {
  static CudaGPUInfo& GPUInfo();
  int NumberGPUs() const;
  int CurrentGPUId() const;
  std::string GetGPUName(int id = -1) const;
  std::string getCudaDeviceStr() const { return GetGPUName(); }
};

}  // namespace tc
