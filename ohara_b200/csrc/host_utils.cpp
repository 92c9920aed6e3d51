#include "host_utils.h"

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

namespace ob {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err =
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess || sym == nullptr)
      throw std::runtime_error("ohara_b200: cuTensorMapEncodeTiled is not available in the driver");
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

size_t dtype_size(TmapDtype d) {
  switch (d) {
    case TmapDtype::BF16: return 2;
    case TmapDtype::F32: return 4;
    case TmapDtype::U8: return 1;
  }
  return 1;
}

}  // namespace

void make_tmap(CUtensorMap* out, const void* base, TmapDtype dtype, int rank, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, TmapSwizzle swizzle) {
  OB_CHECK(rank >= 1 && rank <= 5, "tensor map rank must be 1..5");
  // The encoder is a driver-API entry point and needs a CUDA context bound to the calling thread.
  // A thread that has only ever seen the runtime's default device (autograd worker threads, for
  // example) may not have one yet; cudaSetDevice on the current device initialises the runtime
  // for this thread and binds the primary context.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    int dev = 0;
    OB_CUDA_CHECK(cudaGetDevice(&dev));
    OB_CUDA_CHECK(cudaSetDevice(dev));
    context_bound = true;
  }
  OB_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base address must be 16-byte aligned");
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    OB_CHECK(box[i] >= 1 && box[i] <= 256, "TMA box dimension must be 1..256");
  }
  for (int i = 0; i + 1 < rank; ++i) {
    gstrides[i] = strides_bytes[i];
    OB_CHECK(strides_bytes[i] % 16 == 0 && strides_bytes[i] > 0,
             "TMA global strides must be positive multiples of 16 bytes");
  }
  const size_t esz = dtype_size(dtype);
  OB_CHECK((box[0] * esz) % 16 == 0, "TMA inner box extent must be a multiple of 16 bytes");
  if (swizzle == TmapSwizzle::B128)
    OB_CHECK(box[0] * esz <= 128, "128-byte swizzle limits the inner box to 128 bytes");
  CUtensorMapDataType dt = dtype == TmapDtype::BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype == TmapDtype::F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUtensorMapSwizzle sw =
      swizzle == TmapSwizzle::B128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult res = encode_fn()(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstrides,
                             gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    std::ostringstream oss;
    oss << "ohara_b200: cuTensorMapEncodeTiled failed with code " << (int)res << " (rank " << rank
        << ", dims";
    for (int i = 0; i < rank; ++i) oss << " " << dims[i];
    oss << ", box";
    for (int i = 0; i < rank; ++i) oss << " " << box[i];
    oss << ")";
    throw std::runtime_error(oss.str());
  }
}

void make_tmap_3d(CUtensorMap* out, const void* base, TmapDtype dtype, uint64_t inner,
                  uint64_t rows, uint64_t batches, int64_t pitch, int64_t batch_stride,
                  uint32_t box_inner, uint32_t box_rows, TmapSwizzle swizzle) {
  const size_t esz = dtype_size(dtype);
  uint64_t dims[3] = {inner, rows, batches};
  uint64_t strides[2];
  strides[0] = (uint64_t)pitch * esz;
  strides[1] = (batches > 1) ? (uint64_t)batch_stride * esz : (uint64_t)pitch * esz * rows;
  if (strides[1] == 0) strides[1] = strides[0];
  uint32_t box[3] = {box_inner, box_rows, 1};
  make_tmap(out, base, dtype, 3, dims, strides, box, swizzle);
}

namespace {
std::atomic<long long> g_launches{0};
}
long long launch_count() { return g_launches.load(); }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

cudaError_t try_ensure_dynamic_smem(const void* kernel, size_t bytes) {
  static std::mutex mutex;
  static std::map<std::pair<const void*, int>, size_t> granted;  // (kernel, device) -> bytes
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return rc;
  std::lock_guard<std::mutex> lock(mutex);
  auto key = std::make_pair(kernel, dev);
  auto it = granted.find(key);
  if (it != granted.end() && it->second >= bytes) return cudaSuccess;
  rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (rc == cudaSuccess) granted[key] = bytes;
  return rc;
}

void ensure_dynamic_smem(const void* kernel, size_t bytes) {
  OB_CUDA_CHECK(try_ensure_dynamic_smem(kernel, bytes));
}

int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  OB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 64 && cached[dev] > 0) return cached[dev];
  int sms = 0;
  OB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (dev < 64) cached[dev] = sms;
  return sms;
}

}  // namespace ob
