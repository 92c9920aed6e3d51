// Skinny GEMM for decoding: y (M, N) = x (M, K) @ W (N, K)^T with M <= 16 rows. The weight matrix
// is streamed exactly once with 16-byte loads, one warp per output feature; x sits in shared memory.
// At these sizes the tensor-core GEMM is dominated by its fixed set-up cost, while this kernel is
// bound by the weight stream (and, for the small projections, by a single memory latency).
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ bf16x8 load_stream(const bf16x8* ptr) {
  uint4 raw;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
               : "l"(ptr));
  return *reinterpret_cast<bf16x8*>(&raw);
}

template <int M>
__global__ void __launch_bounds__(256)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                 __nv_bfloat16* __restrict__ y, int rows, int N, int K, int64_t ldx, int64_t ldw,
                 int64_t ldy) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16x8* xs = reinterpret_cast<bf16x8*>(smem_raw);  // M rows of K/8 vectors; unused rows are zero
  const int vecs = K >> 3;
  for (int idx = threadIdx.x; idx < M * vecs; idx += blockDim.x) {
    const int m = idx / vecs, v = idx - m * vecs;
    bf16x8 value;
#pragma unroll
    for (int i = 0; i < 4; ++i) value.v[i] = __floats2bfloat162_rn(0.f, 0.f);
    if (m < rows) value = *reinterpret_cast<const bf16x8*>(x + (int64_t)m * ldx + v * 8);
    xs[idx] = value;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int n = warp; n < N; n += warps) {
    const bf16x8* wr = reinterpret_cast<const bf16x8*>(w + (int64_t)n * ldw);
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    for (int v = lane; v < vecs; v += 32) {
      const bf16x8 wv = load_stream(wr + v);
      float wf[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(wv.v[i]);
        wf[2 * i] = f.x;
        wf[2 * i + 1] = f.y;
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const bf16x8 xv = xs[m * vecs + v];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(xv.v[i]);
          acc[m] = fmaf(wf[2 * i], f.x, acc[m]);
          acc[m] = fmaf(wf[2 * i + 1], f.y, acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m)
        if (m < rows) y[(int64_t)m * ldy + n] = __float2bfloat16(acc[m]);
    }
  }
}

}  // namespace

bool gemv_supported(int M, int N, int K) {
  return M >= 1 && M <= 16 && K % 8 == 0 && (size_t)16 * K * 2 <= 160 * 1024 && N >= 1;
}

void gemv_bf16(const void* x, const void* w, void* y, int M, int N, int K, int64_t ldx, int64_t ldw,
               int64_t ldy, cudaStream_t stream) {
  OB_CHECK(gemv_supported(M, N, K), "skinny GEMM needs 1..16 rows and K a multiple of 8");
  const int padded = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  const size_t smem = (size_t)padded * K * 2;
  const int blocks = std::min((N + 7) / 8, device_sm_count() * 4);
  auto launch = [&](auto kernel) {
    if (smem > 48 * 1024)
      ensure_dynamic_smem((const void*)kernel, smem);
    kernel<<<blocks, 256, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
        static_cast<__nv_bfloat16*>(y), M, N, K, ldx, ldw, ldy);
  };
  switch (padded) {
    case 1: launch(gemv_bf16_kernel<1>); break;
    case 2: launch(gemv_bf16_kernel<2>); break;
    case 4: launch(gemv_bf16_kernel<4>); break;
    case 8: launch(gemv_bf16_kernel<8>); break;
    default: launch(gemv_bf16_kernel<16>); break;
  }
  OB_LAUNCH_CHECK();
}

}  // namespace ob
