// Device status word: one small allocation per device, created on first use and kept until the
// process exits. Kernels that can time out receive its address and record the first failure there.
#include "host_utils.h"

#include <mutex>

namespace ob {

namespace {
std::mutex g_mutex;
int* g_status[64] = {nullptr};
}  // namespace

int* status_ptr() {
  int dev = 0;
  OB_CUDA_CHECK(cudaGetDevice(&dev));
  OB_CHECK(dev >= 0 && dev < 64, "device index out of range");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status[dev] == nullptr) {
    int* ptr = nullptr;
    OB_CUDA_CHECK(cudaMalloc(&ptr, 4 * sizeof(int)));
    OB_CUDA_CHECK(cudaMemset(ptr, 0, 4 * sizeof(int)));
    g_status[dev] = ptr;
  }
  return g_status[dev];
}

void status_read(int out[4], bool clear) {
  int* ptr = status_ptr();
  OB_CUDA_CHECK(cudaMemcpy(out, ptr, 4 * sizeof(int), cudaMemcpyDeviceToHost));
  if (clear) OB_CUDA_CHECK(cudaMemset(ptr, 0, 4 * sizeof(int)));
}

}  // namespace ob
