// Element-wise and reduction stages of the Muon step around the Newton-Schulz GEMMs, for a group
// of B same-shaped (rows x cols) fp32 matrices (reference: ohara/optimizer.py:283-371, which issues
// about twenty ATen passes over the stacked tensors). Parameters and gradients are reached through
// a pointer table, so nothing is stacked or copied back:
//
//   muon_momentum : M <- M + (1-mu)(G - M);  U = G + mu (M - G) -> bf16 stack;  ||U||^2 per matrix
//   muon_scale    : X = U / (1.01 ||U|| + 1e-6)                     (bf16, in place)
//   [Newton-Schulz iterations on X: tcgen05 GEMMs]
//   muon_variance : v = mean(X^2) over the longer-side index (per row, or per column)
//   muon_apply    : P <- P - lr X f - lr wd P [X f P >= 0]  with f the variance-normalising factor;
//                   optionally refreshes the bf16 compute copy of P
#include "api.h"
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float scratch[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < (blockDim.x >> 5)) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  return r;  // valid in thread 0
}

// grid: (chunks, B). Each thread handles 4 consecutive elements per step.
__global__ void __launch_bounds__(256)
muon_momentum_kernel(MuonTable grads, float* __restrict__ momentum, __nv_bfloat16* __restrict__ u,
                     float* __restrict__ norm2, int64_t numel, float mu, int per_pointer) {
  const int b = blockIdx.y;
  const float* g = static_cast<const float*>(grads.ptr[b / per_pointer]) +
                   (int64_t)(b % per_pointer) * numel;
  float* m = momentum + (int64_t)b * numel;
  __nv_bfloat16* out = u + (int64_t)b * numel;
  float acc = 0.f;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < numel;
       i += (int64_t)gridDim.x * blockDim.x * 4) {
    const float4 gv = *reinterpret_cast<const float4*>(g + i);
    float4 mv = *reinterpret_cast<const float4*>(m + i);
    mv.x += (1.f - mu) * (gv.x - mv.x);
    mv.y += (1.f - mu) * (gv.y - mv.y);
    mv.z += (1.f - mu) * (gv.z - mv.z);
    mv.w += (1.f - mu) * (gv.w - mv.w);
    *reinterpret_cast<float4*>(m + i) = mv;
    const float ux = gv.x + mu * (mv.x - gv.x), uy = gv.y + mu * (mv.y - gv.y);
    const float uz = gv.z + mu * (mv.z - gv.z), uw = gv.w + mu * (mv.w - gv.w);
    uint2 packed;
    packed.x = pack_bf16(ux, uy);
    packed.y = pack_bf16(uz, uw);
    *reinterpret_cast<uint2*>(out + i) = packed;
    // the norm is that of the rounded values, which is what the iteration starts from
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
    const float2 a = __bfloat1622float2(h[0]), c = __bfloat1622float2(h[1]);
    acc += a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
  }
  const float total = block_sum(acc);
  if (threadIdx.x == 0) atomicAdd(&norm2[b], total);
}

__global__ void __launch_bounds__(256)
muon_scale_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ norm2, int64_t numel) {
  const int b = blockIdx.y;
  // bf16 arithmetic like the reference: x / (bf16(norm) * 1.01 + 1e-6)
  const float norm = __bfloat162float(__float2bfloat16_rn(sqrtf(norm2[b])));
  const float denom = __bfloat162float(__float2bfloat16_rn(
      __bfloat162float(__float2bfloat16_rn(norm * 1.01f)) + 1e-6f));
  __nv_bfloat16* p = x + (int64_t)b * numel;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < numel;
       i += (int64_t)gridDim.x * blockDim.x * 8) {
    uint4 raw = *reinterpret_cast<const uint4*>(p + i);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      h[j] = __floats2bfloat162_rn(f.x / denom, f.y / denom);
    }
    *reinterpret_cast<uint4*>(p + i) = raw;
  }
}

// v[b, i] = mean_j X[b, i, j]^2 : one warp per row.
__global__ void __launch_bounds__(256)
muon_row_variance_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ v, int64_t rows_total,
                         int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows_total;
       row += warps) {
    const __nv_bfloat16* src = x + row * cols;
    float acc = 0.f;
    for (int j = lane * 8; j < cols; j += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + j);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc += f.x * f.x + f.y * f.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) v[row] = acc / (float)cols;
  }
}

// v[b, j] = mean_i X[b, i, j]^2 : grid (col chunks, row slices, B); slices add with atomics.
__global__ void __launch_bounds__(128)
muon_col_variance_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ v, int rows,
                         int cols, int rows_per_slice) {
  const int b = blockIdx.z;
  const int j = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (j >= cols) return;
  const int r0 = blockIdx.y * rows_per_slice;
  const int r1 = min(rows, r0 + rows_per_slice);
  const __nv_bfloat16* src = x + ((int64_t)b * rows) * cols + j;
  float a0 = 0.f, a1 = 0.f;
  for (int i = r0; i < r1; ++i) {
    const float2 f =
        __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + (int64_t)i * cols));
    a0 += f.x * f.x;
    a1 += f.y * f.y;
  }
  atomicAdd(&v[(int64_t)b * cols + j], a0 / (float)rows);
  atomicAdd(&v[(int64_t)b * cols + j + 1], a1 / (float)rows);
}

// P <- P - lr * (X f) - lr * wd * P * [(X f) P >= 0]; f is per row (by_row) or per column.
__global__ void __launch_bounds__(256)
muon_apply_kernel(MuonTable params, MuonTable shadows, const __nv_bfloat16* __restrict__ x,
                  const float* __restrict__ factor, int rows, int cols, float lr, float wd,
                  int by_row, int per_pointer, int has_shadow) {
  const int b = blockIdx.y;
  const int64_t numel = (int64_t)rows * cols;
  const int64_t base = (int64_t)(b % per_pointer) * numel;
  float* p = static_cast<float*>(params.ptr[b / per_pointer]) + base;
  __nv_bfloat16* shadow =
      has_shadow ? static_cast<__nv_bfloat16*>(shadows.ptr[b / per_pointer]) + base : nullptr;
  const __nv_bfloat16* xs = x + (int64_t)b * numel;
  const float* f = factor + (int64_t)b * (by_row ? rows : cols);
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < numel;
       i += (int64_t)gridDim.x * blockDim.x * 4) {
    const int row = (int)(i / cols);
    const int col = (int)(i - (int64_t)row * cols);
    const uint2 raw = *reinterpret_cast<const uint2*>(xs + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 x01 = __bfloat1622float2(h[0]), x23 = __bfloat1622float2(h[1]);
    float xv[4] = {x01.x, x01.y, x23.x, x23.y};
    float4 pv = *reinterpret_cast<const float4*>(p + i);
    float pe[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      // the update is formed in bf16 like the reference (X * factor rounded to bf16, then fp32)
      const float scale = by_row ? f[row] : f[col + q];
      const float upd = __bfloat162float(__float2bfloat16_rn(xv[q] * scale));
      const float keep = (upd * pe[q] >= 0.f) ? 1.f : 0.f;
      pe[q] -= lr * upd + lr * wd * pe[q] * keep;
    }
    *reinterpret_cast<float4*>(p + i) = make_float4(pe[0], pe[1], pe[2], pe[3]);
    if (has_shadow) {
      uint2 packed;
      packed.x = pack_bf16(pe[0], pe[1]);
      packed.y = pack_bf16(pe[2], pe[3]);
      *reinterpret_cast<uint2*>(shadow + i) = packed;
    }
  }
}

int chunks_for(int64_t numel, int per_thread, int threads) {
  const int64_t need = (numel + (int64_t)per_thread * threads - 1) / ((int64_t)per_thread * threads);
  return (int)std::max<int64_t>(1, std::min<int64_t>(need, 64));
}

}  // namespace

void muon_momentum(const MuonTable& grads, float* momentum, void* u, float* norm2, int batch,
                   int64_t numel, float mu, int per_pointer, cudaStream_t stream) {
  OB_CHECK(numel % 4 == 0, "muon: matrix size must be a multiple of 4");
  OB_CUDA_CHECK(cudaMemsetAsync(norm2, 0, sizeof(float) * batch, stream));
  dim3 grid(chunks_for(numel, 4, 256), batch);
  muon_momentum_kernel<<<grid, 256, 0, stream>>>(grads, momentum, (__nv_bfloat16*)u, norm2, numel,
                                                 mu, per_pointer);
  OB_LAUNCH_CHECK();
}

void muon_scale(void* x, const float* norm2, int batch, int64_t numel, cudaStream_t stream) {
  OB_CHECK(numel % 8 == 0, "muon: matrix size must be a multiple of 8");
  dim3 grid(chunks_for(numel, 8, 256), batch);
  muon_scale_kernel<<<grid, 256, 0, stream>>>((__nv_bfloat16*)x, norm2, numel);
  OB_LAUNCH_CHECK();
}

void muon_variance(const void* x, float* v, int batch, int rows, int cols, bool by_row,
                   cudaStream_t stream) {
  OB_CHECK(cols % 8 == 0, "muon: columns must be a multiple of 8");
  if (by_row) {
    const int64_t rows_total = (int64_t)batch * rows;
    const int blocks = (int)std::min<int64_t>((rows_total + 7) / 8, (int64_t)device_sm_count() * 8);
    muon_row_variance_kernel<<<std::max(blocks, 1), 256, 0, stream>>>((const __nv_bfloat16*)x, v,
                                                                      rows_total, cols);
  } else {
    OB_CUDA_CHECK(cudaMemsetAsync(v, 0, sizeof(float) * (size_t)batch * cols, stream));
    const int slices = std::max(1, std::min(rows / 64, 32));
    const int rows_per_slice = (rows + slices - 1) / slices;
    dim3 grid((cols / 2 + 127) / 128, slices, batch);
    muon_col_variance_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)x, v, rows, cols,
                                                       rows_per_slice);
  }
  OB_LAUNCH_CHECK();
}

void muon_apply(const MuonTable& params, const MuonTable* shadows, const void* x, const float* factor,
                int batch, int rows, int cols, float lr, float wd, bool by_row, int per_pointer,
                cudaStream_t stream) {
  OB_CHECK(cols % 4 == 0, "muon: columns must be a multiple of 4");
  dim3 grid(chunks_for((int64_t)rows * cols, 4, 256), batch);
  MuonTable none = {};
  muon_apply_kernel<<<grid, 256, 0, stream>>>(params, shadows ? *shadows : none,
                                              (const __nv_bfloat16*)x, factor, rows, cols, lr, wd,
                                              by_row ? 1 : 0, per_pointer, shadows ? 1 : 0);
  OB_LAUNCH_CHECK();
}

}  // namespace ob
