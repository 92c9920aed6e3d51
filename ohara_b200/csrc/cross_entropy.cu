// Row-wise softmax cross-entropy over a chunk of bf16 logits, used by the chunked linear +
// cross-entropy op: the logits of one token chunk are produced by the tcgen05 GEMM, this kernel
// turns them in place into d(loss)/d(logits) and emits per-row loss, so the full (tokens x vocab)
// logits never exist and no fp32 copy is made.
//
// One CTA per row; the row is staged in shared memory so global memory is read once and written
// once. Rows whose target equals `ignore_index` get zero loss and zero gradient. Each logit is
// exponentiated once: the second pass replaces the staged logits by e = exp(x - max) (bf16) while
// it sums them in fp32, the third scales e by 1 / sum (the exponential unit, not memory, bounds
// this kernel at a 50k vocabulary).
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = blockDim.x >> 5;
  float r = (lane < nwarps) ? scratch[lane] : (is_max ? -INFINITY : 0.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, r, o);
    r = is_max ? fmaxf(r, other) : r + other;
  }
  return r;
}

// logits: (rows, pitch) bf16, first `vocab` columns valid. Writes dlogits in place when
// `write_grad`, loss per row, and (optionally) lse and whether argmax == target.
__global__ void ce_rows_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                               float* __restrict__ row_loss, float* __restrict__ row_lse,
                               int* __restrict__ row_correct, const float* __restrict__ scale_ptr,
                               int vocab, int64_t pitch, int64_t ignore_index, int write_grad) {
  extern __shared__ __align__(16) uint8_t ce_smem[];
  __nv_bfloat16* row_s = reinterpret_cast<__nv_bfloat16*>(ce_smem);
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  __nv_bfloat16* src = logits + row * pitch;
  const int64_t target = targets[row];
  const bool valid = target != ignore_index && target >= 0 && target < vocab;
  const int vecs = vocab >> 3;

  if (!valid && !row_correct) {
    if (threadIdx.x == 0) {
      row_loss[row] = 0.f;
      if (row_lse) row_lse[row] = 0.f;
    }
    if (write_grad) {
      bf16x8 z;
#pragma unroll
      for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
      for (int v = threadIdx.x; v < vecs; v += blockDim.x) reinterpret_cast<bf16x8*>(src)[v] = z;
      for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x)
        src[i] = __float2bfloat16_rn(0.f);
    }
    return;
  }

  __shared__ float target_logit;
  float vmax = -INFINITY;
  int arg = 0;
  const int tgt = valid ? (int)target : -1;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    const bf16x8 x = reinterpret_cast<const bf16x8*>(src)[v];
    reinterpret_cast<bf16x8*>(row_s)[v] = x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(x.v[i]);
      if (f.x > vmax) { vmax = f.x; arg = 8 * v + 2 * i; }
      if (f.y > vmax) { vmax = f.y; arg = 8 * v + 2 * i + 1; }
      if (8 * v + 2 * i == tgt) target_logit = f.x;
      if (8 * v + 2 * i + 1 == tgt) target_logit = f.y;
    }
  }
  for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
    const __nv_bfloat16 x = src[i];
    row_s[i] = x;
    const float f = __bfloat162float(x);
    if (f > vmax) { vmax = f; arg = i; }
    if (i == tgt) target_logit = f;
  }
  const float row_max = block_reduce(vmax, scratch, true);
  if (row_correct) {
    // Smallest index attaining the maximum, to match torch.argmax tie-breaking.
    __shared__ int best;
    if (threadIdx.x == 0) best = 0x7fffffff;
    __syncthreads();
    if (vmax == row_max) atomicMin(&best, arg);
    __syncthreads();
    if (threadIdx.x == 0) row_correct[row] = (valid && best == (int)target) ? 1 : 0;
  }
  __syncthreads();
  // e = exp(x - max), summed in fp32 and written back over the staged logits as bf16.
  float sum = 0.f;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    bf16x8 x = reinterpret_cast<const bf16x8*>(row_s)[v];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(x.v[i]);
      const float a = __expf(f.x - row_max), b = __expf(f.y - row_max);
      sum += a + b;
      x.v[i] = __floats2bfloat162_rn(a, b);
    }
    reinterpret_cast<bf16x8*>(row_s)[v] = x;
  }
  for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
    const float a = __expf(__bfloat162float(row_s[i]) - row_max);
    sum += a;
    row_s[i] = __float2bfloat16_rn(a);
  }
  const float total = block_reduce(sum, scratch, false);
  const float lse = row_max + logf(total);
  if (threadIdx.x == 0) {
    row_loss[row] = valid ? (lse - target_logit) : 0.f;
    if (row_lse) row_lse[row] = lse;
  }
  if (write_grad) {
    const float scale = valid ? (scale_ptr ? *scale_ptr : 1.f) : 0.f;
    const float inv = scale / total;  // softmax = e / total
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      const bf16x8 x = reinterpret_cast<const bf16x8*>(row_s)[v];
      bf16x8 o;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(x.v[i]);
        float a = f.x * inv, b = f.y * inv;
        const int c = 8 * v + 2 * i;
        if (c == tgt) a -= scale;
        if (c + 1 == tgt) b -= scale;
        o.v[i] = __floats2bfloat162_rn(a, b);
      }
      reinterpret_cast<bf16x8*>(src)[v] = o;
    }
    for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
      float a = __bfloat162float(row_s[i]) * inv;
      if (i == tgt) a -= scale;
      src[i] = __float2bfloat16_rn(a);
    }
  }
}

// The training form of the kernel above (no argmax output) with fewer instructions per logit (ncu,
// one B200, 5248 x 50304: 370 us either way, 2.85 TB/s of in-place traffic; the limiter is the
// shared-memory / special-function queue (MIO stalls), not issue slots and not DRAM: a persistent
// variant that double-buffered rows with bulk async copies measured the same and was dropped).
// The row maximum is taken on packed bf16 pairs without unpacking; the target logit is
// read once from global memory by one thread instead of being compared against in every
// iteration; the "- scale at the target column" of the gradient is folded into the staged row by
// one thread (e[target] -= sum) so that the last pass is a plain scaling, done on packed pairs
// with the scale split into a bf16 head and tail (no systematic rounding of the row's scale).
__global__ void __launch_bounds__(512)
ce_rows_train_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                     float* __restrict__ row_loss, float* __restrict__ row_lse,
                     const float* __restrict__ scale_ptr, int vocab, int64_t pitch,
                     int64_t ignore_index) {
  extern __shared__ __align__(16) uint8_t ce_smem[];
  __nv_bfloat16* row_s = reinterpret_cast<__nv_bfloat16*>(ce_smem);
  __shared__ float scratch[32];
  __shared__ float target_logit;
  const int64_t row = blockIdx.x;
  __nv_bfloat16* src = logits + row * pitch;
  const int64_t target = targets[row];
  const bool valid = target != ignore_index && target >= 0 && target < vocab;
  const int vecs = vocab >> 3;
  if (!valid) {
    if (threadIdx.x == 0) {
      row_loss[row] = 0.f;
      if (row_lse) row_lse[row] = 0.f;
    }
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) reinterpret_cast<uint4*>(src)[v] = z;
    for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x)
      src[i] = __float2bfloat16_rn(0.f);
    return;
  }
  if (threadIdx.x == 0) target_logit = __bfloat162float(src[target]);

  // pass 1: stage the row, maximum on packed pairs
  __nv_bfloat162 m2 = __floats2bfloat162_rn(-INFINITY, -INFINITY);
  // four independent 16-byte loads in flight per thread: with one, the 32 warps of an SM keep
  // too few bytes in flight to cover the DRAM latency
  {
    const int stride = blockDim.x;
    int v = threadIdx.x;
    for (; v + 3 * stride < vecs; v += 4 * stride) {
      bf16x8 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) x[u] = reinterpret_cast<const bf16x8*>(src)[v + u * stride];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        reinterpret_cast<bf16x8*>(row_s)[v + u * stride] = x[u];
        m2 = __hmax2(m2, __hmax2(__hmax2(x[u].v[0], x[u].v[1]), __hmax2(x[u].v[2], x[u].v[3])));
      }
    }
    for (; v < vecs; v += stride) {
      const bf16x8 x = reinterpret_cast<const bf16x8*>(src)[v];
      reinterpret_cast<bf16x8*>(row_s)[v] = x;
      m2 = __hmax2(m2, __hmax2(__hmax2(x.v[0], x.v[1]), __hmax2(x.v[2], x.v[3])));
    }
  }
  float vmax = fmaxf(__low2float(m2), __high2float(m2));
  for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
    const __nv_bfloat16 x = src[i];
    row_s[i] = x;
    vmax = fmaxf(vmax, __bfloat162float(x));
  }
  const float row_max = block_reduce(vmax, scratch, true);
  __syncthreads();

  // pass 2: e = 2^(x * log2e - max * log2e), summed in fp32, staged back as bf16
  constexpr float kLog2e = 1.4426950408889634f;
  const float shift = row_max * kLog2e;
  float sum0 = 0.f, sum1 = 0.f;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    bf16x8 x = reinterpret_cast<const bf16x8*>(row_s)[v];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(x.v[i]);
      const float a = fast_exp2(fmaf(f.x, kLog2e, -shift));
      const float b = fast_exp2(fmaf(f.y, kLog2e, -shift));
      sum0 += a;
      sum1 += b;
      x.v[i] = __floats2bfloat162_rn(a, b);
    }
    reinterpret_cast<bf16x8*>(row_s)[v] = x;
  }
  for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
    const float a = fast_exp2(fmaf(__bfloat162float(row_s[i]), kLog2e, -shift));
    sum0 += a;
    row_s[i] = __float2bfloat16_rn(a);
  }
  const float total = block_reduce(sum0 + sum1, scratch, false);
  const float lse = row_max + logf(total);
  if (threadIdx.x == 0) {
    row_loss[row] = lse - target_logit;
    if (row_lse) row_lse[row] = lse;
    // softmax - onehot at the target column: (e - total) / total
    row_s[target] = __float2bfloat16_rn(__bfloat162float(row_s[target]) - total);
  }
  __syncthreads();

  // pass 3: gradient = e * (scale / total) on packed pairs; head + tail keep the factor exact
  const float inv = (scale_ptr ? *scale_ptr : 1.f) / total;
  const __nv_bfloat16 inv_hi = __float2bfloat16_rn(inv);
  const __nv_bfloat16 inv_lo = __float2bfloat16_rn(inv - __bfloat162float(inv_hi));
  const __nv_bfloat162 hi2 = __halves2bfloat162(inv_hi, inv_hi);
  const __nv_bfloat162 lo2 = __halves2bfloat162(inv_lo, inv_lo);
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    bf16x8 x = reinterpret_cast<const bf16x8*>(row_s)[v];
#pragma unroll
    for (int i = 0; i < 4; ++i) x.v[i] = __hfma2(x.v[i], lo2, __hmul2(x.v[i], hi2));
    reinterpret_cast<bf16x8*>(src)[v] = x;
  }
  for (int i = (vecs << 3) + threadIdx.x; i < vocab; i += blockDim.x)
    src[i] = __float2bfloat16_rn(__bfloat162float(row_s[i]) * inv);
}

__global__ void scale_by_device_scalar_bf16(__nv_bfloat16* x, const float* s, int64_t n) {
  const float k = *s;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * k);
}
__global__ void scale_by_device_scalar_f32(float* x, const float* s, int64_t n) {
  const float k = *s;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    x[i] *= k;
}

}  // namespace

void cross_entropy_rows(void* logits, const int64_t* targets, float* row_loss, float* row_lse,
                        int* row_correct, const float* scale_ptr, int64_t rows, int vocab,
                        int64_t pitch, int64_t ignore_index, bool write_grad, cudaStream_t stream) {
  if (rows == 0) return;
  OB_CHECK(pitch % 8 == 0, "cross entropy: logits pitch must be a multiple of 8 elements");
  const size_t smem = (size_t)((vocab + 7) / 8) * 16;
  OB_CHECK(smem <= 200 * 1024, "cross entropy: vocabulary too large for the shared-memory row buffer");
  if (write_grad && row_correct == nullptr) {
    ensure_dynamic_smem((const void*)ce_rows_train_kernel, 200 * 1024);
    ce_rows_train_kernel<<<(unsigned)rows, 512, smem, stream>>>(
        (__nv_bfloat16*)logits, targets, row_loss, row_lse, scale_ptr, vocab, pitch, ignore_index);
    OB_LAUNCH_CHECK();
    return;
  }
  ensure_dynamic_smem((const void*)ce_rows_kernel, 200 * 1024);
  ce_rows_kernel<<<(unsigned)rows, 512, smem, stream>>>((__nv_bfloat16*)logits, targets, row_loss,
                                                        row_lse, row_correct, scale_ptr, vocab,
                                                        pitch, ignore_index, write_grad ? 1 : 0);
  OB_LAUNCH_CHECK();
}

void scale_by_scalar(void* x, bool is_bf16, const float* scalar, int64_t n, cudaStream_t stream) {
  if (n == 0) return;
  const int threads = 256;
  const int blocks = (int)std::min<int64_t>((n + threads - 1) / threads, device_sm_count() * 8);
  if (is_bf16)
    scale_by_device_scalar_bf16<<<blocks, threads, 0, stream>>>((__nv_bfloat16*)x, scalar, n);
  else
    scale_by_device_scalar_f32<<<blocks, threads, 0, stream>>>((float*)x, scalar, n);
  OB_LAUNCH_CHECK();
}

}  // namespace ob
