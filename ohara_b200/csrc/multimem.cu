// Sum over the ranks of a multicast group with the NVSwitch doing the additions: one
// `multimem.ld_reduce` per 16 bytes reads the same offset of every rank's buffer through the switch
// and returns the sum, so a one-shot all-reduce moves each element over this GPU's links once
// instead of once per peer.
//
// The kernel has no waits of its own. The caller orders it between two barriers of the peer
// runtime (bounded waits, status word): every rank has written its buffer before the first, no
// rank overwrites its buffer before the second. The multicast address comes from the symmetric
// memory allocator that bound every rank's buffer to one multicast object; it must not be used
// after a peer has left the group.
#include "api.h"
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

template <bool BF16>
__global__ void __launch_bounds__(256)
multimem_sum_kernel(const char* __restrict__ multicast, char* __restrict__ out, int64_t vectors,
                    float scale) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vectors; i += stride) {
    const char* address = multicast + i * 16;
    uint4 value;
    if constexpr (BF16) {
      // bf16 pairs, accumulated in fp32 inside the switch
      asm volatile(
          "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
          : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
          : "l"(address)
          : "memory");
      if (scale != 1.f) {
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&value);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          float2 f = __bfloat1622float2(pairs[p]);
          pairs[p] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
        }
      }
    } else {
      float4 sum;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(sum.x), "=f"(sum.y), "=f"(sum.z), "=f"(sum.w)
                   : "l"(address)
                   : "memory");
      sum.x *= scale, sum.y *= scale, sum.z *= scale, sum.w *= scale;
      value = *reinterpret_cast<uint4*>(&sum);
    }
    *reinterpret_cast<uint4*>(out + i * 16) = value;
  }
}

}  // namespace

void multimem_sum(const void* multicast, void* out, int64_t bytes, bool bf16, float scale,
                  cudaStream_t stream) {
  OB_CHECK(bytes % 16 == 0, "multimem_sum: the size must be a multiple of 16 bytes");
  OB_CHECK(reinterpret_cast<uintptr_t>(multicast) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(out) % 16 == 0,
           "multimem_sum: addresses must be 16-byte aligned");
  if (bytes == 0) return;
  const int64_t vectors = bytes / 16;
  const int threads = 256;
  const int blocks = (int)std::max<int64_t>(
      1, std::min<int64_t>((vectors + threads - 1) / threads, (int64_t)device_sm_count() * 4));
  if (bf16)
    multimem_sum_kernel<true><<<blocks, threads, 0, stream>>>((const char*)multicast, (char*)out,
                                                              vectors, scale);
  else
    multimem_sum_kernel<false><<<blocks, threads, 0, stream>>>((const char*)multicast, (char*)out,
                                                               vectors, scale);
  OB_LAUNCH_CHECK();
}

}  // namespace ob
