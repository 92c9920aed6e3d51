// Stream-ordered 32-bit memory operations (no kernel, no SM): "wait until *addr >= value" and
// "*addr = value". They order copy-engine transfers against flags that kernels on this or another
// GPU read and write, so an all-gather can run on the copy engines next to a GEMM that occupies
// every SM.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>

#include "host_utils.h"

namespace ob {

namespace {

using WaitValueFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
using WriteValueFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

void* driver_symbol(const char* name) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  const cudaError_t err = cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &qres);
  if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess || sym == nullptr)
    throw std::runtime_error(std::string("ohara_b200: driver entry point not available: ") + name);
  return sym;
}

void bind_context() {
  int dev = 0;
  OB_CUDA_CHECK(cudaGetDevice(&dev));
  OB_CUDA_CHECK(cudaSetDevice(dev));
}

}  // namespace

void stream_wait_value32(cudaStream_t stream, uint64_t addr, uint32_t value) {
  static WaitValueFn fn = reinterpret_cast<WaitValueFn>(driver_symbol("cuStreamWaitValue32"));
  bind_context();
  const CUresult res = fn(stream, static_cast<CUdeviceptr>(addr), value, CU_STREAM_WAIT_VALUE_GEQ);
  OB_CHECK(res == CUDA_SUCCESS, "cuStreamWaitValue32 failed with code " << (int)res);
}

void stream_write_value32(cudaStream_t stream, uint64_t addr, uint32_t value) {
  static WriteValueFn fn = reinterpret_cast<WriteValueFn>(driver_symbol("cuStreamWriteValue32"));
  bind_context();
  const CUresult res = fn(stream, static_cast<CUdeviceptr>(addr), value, CU_STREAM_WRITE_VALUE_DEFAULT);
  OB_CHECK(res == CUDA_SUCCESS, "cuStreamWriteValue32 failed with code " << (int)res);
}

}  // namespace ob
