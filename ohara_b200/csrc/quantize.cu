// Quantisers of BitNet b1.58 layers (reference: experiments/bitnet/bitnet.py:29-43, two
// TorchScript functions of whole-tensor PyTorch operations).
//
// The layer computes  y = (q(norm(x)) @ t(W)^T) * dequant_row * scale_w  with
//   q: per-row absolute-maximum int8 quantisation of the (RMS-normalised) activations,
//   t: ternary quantisation of the weight by its mean absolute value.
// Both quantised operands hold small integers (|q| <= 128, t in {-1, 0, 1}); bf16 represents them
// exactly and the tensor cores accumulate in fp32, so the product runs on the bf16 tcgen05 GEMM
// without any rounding below 2^24 and the two scales are applied to the fp32 accumulators by
// `scale_rows`. The kernels here are bound by memory traffic:
//   * `act_quant`: one warp per row, the RMS norm fused in (sum of squares and the absolute maximum
//     of the normalised row come out of the same pass), integer values written as bf16 and one
//     fp32 de-quantisation factor per row;
//   * `weight_quant`: a deterministic two-stage sum of |w| (fixed partial count, fixed order), then
//     one pass that writes the ternary values; the scale stays on the device;
//   * `scale_rows`: fp32 accumulators x row factor x weight scale (+ bias) -> bf16.
#include "api.h"
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kPartials = 1024;  // partial sums of |w|: one per block of the first stage

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& in, float (&out)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(in.v[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ bf16x8 pack8(const float (&in)[8]) {
  bf16x8 out;
#pragma unroll
  for (int i = 0; i < 4; ++i) out.v[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
  return out;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void load_weights8(const float* w, int v, float (&out)[8]) {
  const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v];
  const float4 w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
  out[0] = w0.x, out[1] = w0.y, out[2] = w0.z, out[3] = w0.w;
  out[4] = w1.x, out[5] = w1.y, out[6] = w1.z, out[7] = w1.w;
}

// q[row] = clamp(rint(y * 127 / max(amax(|y|), 1e-5)), -128, 127) with y = x (HAS_NORM false) or
// y = x * rsqrt(mean(x^2) + eps) * w. dequant[row] = max(amax, 1e-5) / 127.
template <bool HAS_NORM>
__global__ void __launch_bounds__(256)
act_quant_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                 __nv_bfloat16* __restrict__ q, float* __restrict__ dequant,
                 float* __restrict__ rstd_out, int rows, int d, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vecs = d >> 3;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * d);
    float ss = 0.f, amax = 0.f;
    for (int v = lane; v < vecs; v += 32) {
      float f[8];
      unpack8(xr[v], f);
      if (HAS_NORM) {
        float ww[8];
        load_weights8(w, v, ww);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ss += f[i] * f[i];
          amax = fmaxf(amax, fabsf(f[i] * ww[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
    }
    amax = warp_max(amax);
    float rstd = 1.f;
    if (HAS_NORM) {
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / (float)d + eps);
      amax *= rstd;
    }
    const float clamped = fmaxf(amax, 1e-5f);
    const float scale = 127.f / clamped;
    if (lane == 0) {
      dequant[row] = clamped / 127.f;
      if (HAS_NORM && rstd_out != nullptr) rstd_out[row] = rstd;
    }
    bf16x8* qr = reinterpret_cast<bf16x8*>(q + (size_t)row * d);
    for (int v = lane; v < vecs; v += 32) {
      float f[8];
      unpack8(xr[v], f);  // second read of the row: it is still in L1 / L2
      if (HAS_NORM) {
        float ww[8];
        load_weights8(w, v, ww);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * ww[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = fminf(fmaxf(rintf(f[i] * scale), -128.f), 127.f);
      qr[v] = pack8(f);
    }
  }
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

// Block-wide sum in a fixed order: lanes by butterfly, warps serially by thread 0.
__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
  if (threadIdx.x == 0) {
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += scratch[i];
  }
  __syncthreads();
  return total;  // valid in thread 0
}

// Stage 1: partials[b] = sum of |w[i]| over the contiguous chunk of block b (a fixed partition of
// the tensor, so the result does not depend on the grid the device happens to schedule).
template <typename T>
__global__ void __launch_bounds__(256)
abs_sum_kernel(const T* __restrict__ w, int64_t n, float* __restrict__ partials) {
  __shared__ float scratch[8];
  const int64_t chunk = (n + gridDim.x - 1) / gridDim.x;
  const int64_t begin = (int64_t)blockIdx.x * chunk;
  const int64_t end = begin + chunk < n ? begin + chunk : n;
  float acc = 0.f;
  for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) acc += fabsf(to_float(w[i]));
  const float total = block_sum_256(acc, scratch);
  if (threadIdx.x == 0) partials[blockIdx.x] = total;
}

// Stage 2 (one block): scale = max(sum(partials) / n, 1e-5).
__global__ void __launch_bounds__(256)
abs_mean_finish_kernel(const float* __restrict__ partials, int count, int64_t n,
                       float* __restrict__ scale) {
  __shared__ float scratch[8];
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) acc += partials[i];
  const float total = block_sum_256(acc, scratch);
  if (threadIdx.x == 0) scale[0] = fmaxf(total / (float)n, 1e-5f);
}

// t[i] = clamp(rint(w[i] / scale), -1, 1), written as bf16.
template <typename T>
__global__ void __launch_bounds__(256)
ternary_kernel(const T* __restrict__ w, const float* __restrict__ scale,
               __nv_bfloat16* __restrict__ t, int64_t n) {
  const float inv = 1.f / scale[0];
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = fminf(fmaxf(rintf(to_float(w[i]) * inv), -1.f), 1.f);
    t[i] = __float2bfloat16_rn(v);
  }
}

// out[r, c] = acc[r, c] * row_factor[r] * weight_scale[0] (+ bias[c]); four columns per thread.
__global__ void __launch_bounds__(256)
scale_rows_kernel(const float* __restrict__ acc, const float* __restrict__ row_factor,
                  const float* __restrict__ weight_scale, const float* __restrict__ bias,
                  __nv_bfloat16* __restrict__ out, int64_t rows, int n) {
  const int quads = n >> 2;
  const int64_t total = rows * quads;
  const float ws = weight_scale[0];
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / quads;
    const int c = (int)(i - r * quads) << 2;
    const float s = row_factor[r] * ws;
    float4 v = *reinterpret_cast<const float4*>(acc + r * n + c);
    v.x *= s, v.y *= s, v.z *= s, v.w *= s;
    if (bias != nullptr) {
      const float4 b = *reinterpret_cast<const float4*>(bias + c);
      v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
    }
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(out + r * n + c);
    o[0] = __floats2bfloat162_rn(v.x, v.y);
    o[1] = __floats2bfloat162_rn(v.z, v.w);
  }
}

int blocks_for(int64_t threads_wanted, int threads) {
  const int64_t blocks = (threads_wanted + threads - 1) / threads;
  const int64_t cap = (int64_t)device_sm_count() * 8;
  return (int)std::max<int64_t>(1, std::min(blocks, cap));
}

}  // namespace

void bitnet_act_quant(const void* x, const float* norm_weight, void* q, float* dequant, float* rstd,
                      int rows, int d, float eps, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "act_quant: width must be a multiple of 8");
  if (rows == 0) return;
  const int threads = 256;
  const int blocks = blocks_for((int64_t)rows * 32, threads);
  if (norm_weight != nullptr)
    act_quant_kernel<true><<<blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, norm_weight, (__nv_bfloat16*)q, dequant, rstd, rows, d, eps);
  else
    act_quant_kernel<false><<<blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, nullptr, (__nv_bfloat16*)q, dequant, nullptr, rows, d, eps);
  OB_LAUNCH_CHECK();
}

int bitnet_partial_count() { return kPartials; }

void bitnet_weight_quant(const void* w, bool w_is_f32, int64_t n, void* ternary, float* scale,
                         float* partials, cudaStream_t stream) {
  if (n == 0) return;
  const int threads = 256;
  // A fixed partition (independent of the device): small tensors use fewer, never empty, chunks.
  const int parts = (int)std::max<int64_t>(1, std::min<int64_t>(kPartials, (n + 4095) / 4096));
  if (w_is_f32)
    abs_sum_kernel<float><<<parts, threads, 0, stream>>>((const float*)w, n, partials);
  else
    abs_sum_kernel<__nv_bfloat16><<<parts, threads, 0, stream>>>((const __nv_bfloat16*)w, n, partials);
  OB_LAUNCH_CHECK();
  abs_mean_finish_kernel<<<1, threads, 0, stream>>>(partials, parts, n, scale);
  OB_LAUNCH_CHECK();
  const int blocks = blocks_for(n, threads);
  if (w_is_f32)
    ternary_kernel<float><<<blocks, threads, 0, stream>>>((const float*)w, scale,
                                                          (__nv_bfloat16*)ternary, n);
  else
    ternary_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)w, scale, (__nv_bfloat16*)ternary, n);
  OB_LAUNCH_CHECK();
}

void bitnet_scale_rows(const float* acc, const float* row_factor, const float* weight_scale,
                       const float* bias, void* out, int64_t rows, int n, cudaStream_t stream) {
  OB_CHECK(n % 4 == 0, "scale_rows: width must be a multiple of 4");
  if (rows == 0) return;
  const int threads = 256;
  const int blocks = blocks_for(rows * (n / 4), threads);
  scale_rows_kernel<<<blocks, threads, 0, stream>>>(acc, row_factor, weight_scale, bias,
                                                    (__nv_bfloat16*)out, rows, n);
  OB_LAUNCH_CHECK();
}

}  // namespace ob
