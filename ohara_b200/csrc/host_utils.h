// Host-side helpers shared by the kernel launchers: error checks and TMA descriptor construction.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <sstream>
#include <stdexcept>
#include <string>

namespace ob {

#define OB_CHECK(cond, msg)                                                     \
  do {                                                                          \
    if (!(cond)) {                                                              \
      std::ostringstream oss__;                                                 \
      oss__ << "ohara_b200: " << msg << " (" << #cond << ") at " << __FILE__    \
            << ":" << __LINE__;                                                 \
      throw std::runtime_error(oss__.str());                                    \
    }                                                                           \
  } while (0)

#define OB_CUDA_CHECK(expr)                                                      \
  do {                                                                          \
    cudaError_t err__ = (expr);                                                 \
    if (err__ != cudaSuccess) {                                                 \
      std::ostringstream oss__;                                                 \
      oss__ << "ohara_b200: CUDA error " << cudaGetErrorString(err__) << " in " \
            << #expr << " at " << __FILE__ << ":" << __LINE__;                  \
      throw std::runtime_error(oss__.str());                                    \
    }                                                                           \
  } while (0)

// Counts kernel launches issued by this library (read by benchmarks through `launch_count`).
long long launch_count();
void count_launch();

#define OB_LAUNCH_CHECK()                    \
  do {                                       \
    ::ob::count_launch();                    \
    OB_CUDA_CHECK(cudaGetLastError());       \
  } while (0)

enum class TmapDtype { BF16, F32, U8 };
enum class TmapSwizzle { NONE, B128 };

// Up to 5-D tiled tensor map. dims[0] is the contiguous dimension; strides_bytes[i] is the byte
// stride of dims[i+1] (rank-1 entries, each a multiple of 16).
void make_tmap(CUtensorMap* out, const void* base, TmapDtype dtype, int rank, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, TmapSwizzle swizzle);

// (inner, rows, batches) view of a row-pitched, batch-strided matrix. `pitch` and `batch_stride`
// are in elements.
void make_tmap_3d(CUtensorMap* out, const void* base, TmapDtype dtype, uint64_t inner,
                  uint64_t rows, uint64_t batches, int64_t pitch, int64_t batch_stride,
                  uint32_t box_inner, uint32_t box_rows, TmapSwizzle swizzle);

int device_sm_count();

// Function attributes are per device. Opts `kernel` into `bytes` of dynamic shared memory the
// first time it is asked for on the current device (and again if a later call needs more);
// throws if the driver refuses. Thread-safe.
void ensure_dynamic_smem(const void* kernel, size_t bytes);
// Same, without throwing: returns the CUDA error instead (nothing is recorded on failure, so the
// next call tries again).
cudaError_t try_ensure_dynamic_smem(const void* kernel, size_t bytes);

// Device status word (see status.cpp): [0] first error code, [1] block that reported it, [2] number
// of waits that ran out of time.
int* status_ptr();
void status_read(int out[4], bool clear);

}  // namespace ob
