// Log-domain Sinkhorn normalisation of many small square matrices (hyper-connection mixing
// weights, reference: experiments/mHC/sinkhorn.py:59-200, a Triton kernel with one program per
// matrix). Here one thread owns one N x N matrix in registers (N <= 4): after subtracting the
// global maximum it alternates "subtract the row log-sum-exp" and "subtract the column
// log-sum-exp" `iters` times and returns exp(x), a doubly stochastic matrix.
//
// Backward: a half-step y = x - lse(x) has the Jacobian-vector product g_x = g_y - exp(y) * sum(g_y)
// along the normalised axis, which needs only the *output* of the half-step. The backward kernel
// therefore replays the forward once, keeps every half-step output on a per-thread tape (local
// memory, 2 * iters * N * N floats) and walks it back; the reference recomputes the forward for
// every step instead.
#include "api.h"
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kMaxIters = 32;

template <int N>
__device__ __forceinline__ void normalise_rows(float (&x)[N * N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float m = x[i * N];
#pragma unroll
    for (int j = 1; j < N; ++j) m = fmaxf(m, x[i * N + j]);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) s += __expf(x[i * N + j] - m);
    const float lse = m + __logf(s);
#pragma unroll
    for (int j = 0; j < N; ++j) x[i * N + j] -= lse;
  }
}

template <int N>
__device__ __forceinline__ void normalise_cols(float (&x)[N * N]) {
#pragma unroll
  for (int j = 0; j < N; ++j) {
    float m = x[j];
#pragma unroll
    for (int i = 1; i < N; ++i) m = fmaxf(m, x[i * N + j]);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) s += __expf(x[i * N + j] - m);
    const float lse = m + __logf(s);
#pragma unroll
    for (int i = 0; i < N; ++i) x[i * N + j] -= lse;
  }
}

template <int N>
__device__ __forceinline__ void load_centered(const float* __restrict__ src, float (&x)[N * N]) {
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < N * N; ++i) {
    x[i] = src[i];
    m = fmaxf(m, x[i]);
  }
#pragma unroll
  for (int i = 0; i < N * N; ++i) x[i] -= m;
}

template <int N>
__global__ void sinkhorn_fwd_kernel(const float* __restrict__ in, float* __restrict__ out,
                                    int64_t count, int iters) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count) return;
  float x[N * N];
  load_centered<N>(in + idx * N * N, x);
  for (int it = 0; it < iters; ++it) {
    normalise_rows<N>(x);
    normalise_cols<N>(x);
  }
#pragma unroll
  for (int i = 0; i < N * N; ++i) out[idx * N * N + i] = __expf(x[i]);
}

template <int N>
__global__ void sinkhorn_bwd_kernel(const float* __restrict__ in, const float* __restrict__ grad_out,
                                    float* __restrict__ grad_in, int64_t count, int iters) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count) return;
  float tape[2 * kMaxIters][N * N];
  float x[N * N];
  load_centered<N>(in + idx * N * N, x);
  for (int it = 0; it < iters; ++it) {
    normalise_rows<N>(x);
#pragma unroll
    for (int i = 0; i < N * N; ++i) tape[2 * it][i] = x[i];
    normalise_cols<N>(x);
#pragma unroll
    for (int i = 0; i < N * N; ++i) tape[2 * it + 1][i] = x[i];
  }
  // d exp(x) = exp(x) * dx
  float g[N * N];
#pragma unroll
  for (int i = 0; i < N * N; ++i) g[i] = grad_out[idx * N * N + i] * __expf(x[i]);
  for (int it = iters - 1; it >= 0; --it) {
    // column half-step
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) s += g[i * N + j];
#pragma unroll
      for (int i = 0; i < N; ++i) g[i * N + j] -= __expf(tape[2 * it + 1][i * N + j]) * s;
    }
    // row half-step
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) s += g[i * N + j];
#pragma unroll
      for (int j = 0; j < N; ++j) g[i * N + j] -= __expf(tape[2 * it][i * N + j]) * s;
    }
  }
  // Subtracting the global maximum shifts every entry equally; the normalisations cancel a
  // constant shift, so the total gradient of that shift is zero up to rounding: nothing to add.
#pragma unroll
  for (int i = 0; i < N * N; ++i) grad_in[idx * N * N + i] = g[i];
}

// ---- matrices of 5 to 64 rows: one block per matrix, the matrix in shared memory ---------------
// Thread i owns row i in the row half-steps and column i in the column half-steps; the pitch of
// n + 1 floats keeps both access patterns free of bank conflicts. The backward pass replays the
// forward pass, writes every half-step output to a tape in global memory (2 * iters * n * n floats
// per matrix, provided by the caller) and walks it back with the same vector-Jacobian product as
// the register kernel.
constexpr int kBlockMaxN = 64;

__device__ __forceinline__ void block_half_step(float* x, int n, int pitch, bool rows, int t) {
  if (t < n) {
    const int step = rows ? 1 : pitch;
    float* line = x + (rows ? t * pitch : t);
    float m = -INFINITY;
    for (int j = 0; j < n; ++j) m = fmaxf(m, line[j * step]);
    float sum = 0.f;
    for (int j = 0; j < n; ++j) sum += __expf(line[j * step] - m);
    const float lse = m + __logf(sum);
    for (int j = 0; j < n; ++j) line[j * step] -= lse;
  }
  __syncthreads();
}

template <bool BACKWARD>
__global__ void __launch_bounds__(kBlockMaxN)
sinkhorn_block_kernel(const float* __restrict__ in, const float* __restrict__ grad_out,
                      float* __restrict__ out, float* __restrict__ tape, int n, int iters) {
  extern __shared__ float sk_smem[];
  const int pitch = n + 1;
  float* x = sk_smem;
  float* g = sk_smem + n * pitch;  // backward only
  __shared__ float red[kBlockMaxN];
  const int t = threadIdx.x;
  const int64_t mat = blockIdx.x;
  const float* src = in + mat * n * n;
  float m = -INFINITY;
  for (int e = t; e < n * n; e += blockDim.x) {
    const float v = src[e];
    x[(e / n) * pitch + e % n] = v;
    m = fmaxf(m, v);
  }
  red[t] = m;
  __syncthreads();
  m = red[0];
  for (int i = 1; i < blockDim.x; ++i) m = fmaxf(m, red[i]);
  for (int e = t; e < n * n; e += blockDim.x) x[(e / n) * pitch + e % n] -= m;
  __syncthreads();
  float* my_tape = BACKWARD ? tape + mat * 2 * iters * n * n : nullptr;
  for (int it = 0; it < iters; ++it) {
    block_half_step(x, n, pitch, true, t);
    if (BACKWARD)
      for (int e = t; e < n * n; e += blockDim.x)
        my_tape[(2 * it) * n * n + e] = x[(e / n) * pitch + e % n];
    block_half_step(x, n, pitch, false, t);
    if (BACKWARD)
      for (int e = t; e < n * n; e += blockDim.x)
        my_tape[(2 * it + 1) * n * n + e] = x[(e / n) * pitch + e % n];
  }
  if (!BACKWARD) {
    for (int e = t; e < n * n; e += blockDim.x) out[mat * n * n + e] = __expf(x[(e / n) * pitch + e % n]);
    return;
  }
  for (int e = t; e < n * n; e += blockDim.x)
    g[(e / n) * pitch + e % n] = grad_out[mat * n * n + e] * __expf(x[(e / n) * pitch + e % n]);
  __syncthreads();
  for (int it = iters - 1; it >= 0; --it) {
    const float* col_out = my_tape + (2 * it + 1) * n * n;
    if (t < n) {  // column half-step: thread t owns column t
      float sum = 0.f;
      for (int i = 0; i < n; ++i) sum += g[i * pitch + t];
      for (int i = 0; i < n; ++i) g[i * pitch + t] -= __expf(col_out[i * n + t]) * sum;
    }
    __syncthreads();
    const float* row_out = my_tape + (2 * it) * n * n;
    if (t < n) {  // row half-step: thread t owns row t
      float sum = 0.f;
      for (int j = 0; j < n; ++j) sum += g[t * pitch + j];
      for (int j = 0; j < n; ++j) g[t * pitch + j] -= __expf(row_out[t * n + j]) * sum;
    }
    __syncthreads();
  }
  for (int e = t; e < n * n; e += blockDim.x) out[mat * n * n + e] = g[(e / n) * pitch + e % n];
}

}  // namespace

bool sinkhorn_supported(int n, int iters) {
  return n >= 2 && n <= kBlockMaxN && iters >= 1 && iters <= kMaxIters;
}

// Floats of scratch the backward pass needs per matrix (0 for the register kernel).
int64_t sinkhorn_tape_floats(int n, int iters) {
  return n <= 4 ? 0 : (int64_t)2 * iters * n * n;
}

void sinkhorn_forward(const float* in, float* out, int64_t count, int n, int iters,
                      cudaStream_t stream) {
  OB_CHECK(sinkhorn_supported(n, iters), "sinkhorn: matrices of 2..64 rows, 1..32 iterations");
  if (count == 0) return;
  if (n > 4) {
    const size_t smem = (size_t)n * (n + 1) * sizeof(float);
    sinkhorn_block_kernel<false><<<(unsigned)count, kBlockMaxN, smem, stream>>>(in, nullptr, out,
                                                                                 nullptr, n, iters);
    OB_LAUNCH_CHECK();
    return;
  }
  const int threads = 128;
  const int blocks = (int)((count + threads - 1) / threads);
  if (n == 2)
    sinkhorn_fwd_kernel<2><<<blocks, threads, 0, stream>>>(in, out, count, iters);
  else if (n == 3)
    sinkhorn_fwd_kernel<3><<<blocks, threads, 0, stream>>>(in, out, count, iters);
  else
    sinkhorn_fwd_kernel<4><<<blocks, threads, 0, stream>>>(in, out, count, iters);
  OB_LAUNCH_CHECK();
}

void sinkhorn_backward(const float* in, const float* grad_out, float* grad_in, float* tape,
                       int64_t count, int n, int iters, cudaStream_t stream) {
  OB_CHECK(sinkhorn_supported(n, iters), "sinkhorn: matrices of 2..64 rows, 1..32 iterations");
  if (count == 0) return;
  if (n > 4) {
    OB_CHECK(tape != nullptr, "sinkhorn backward of matrices wider than 4 needs a tape buffer");
    const size_t smem = (size_t)2 * n * (n + 1) * sizeof(float);
    sinkhorn_block_kernel<true><<<(unsigned)count, kBlockMaxN, smem, stream>>>(in, grad_out, grad_in,
                                                                                tape, n, iters);
    OB_LAUNCH_CHECK();
    return;
  }
  const int threads = 64;
  const int blocks = (int)((count + threads - 1) / threads);
  if (n == 2)
    sinkhorn_bwd_kernel<2><<<blocks, threads, 0, stream>>>(in, grad_out, grad_in, count, iters);
  else if (n == 3)
    sinkhorn_bwd_kernel<3><<<blocks, threads, 0, stream>>>(in, grad_out, grad_in, count, iters);
  else
    sinkhorn_bwd_kernel<4><<<blocks, threads, 0, stream>>>(in, grad_out, grad_in, count, iters);
  OB_LAUNCH_CHECK();
}

}  // namespace ob
