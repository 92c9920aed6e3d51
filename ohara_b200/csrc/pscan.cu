// First-order linear recurrence h[t] = a[t] * h[t-1] + x[t] (h[-1] = 0) along dim 1 of
// (B, L, C) fp32 tensors: the selective scan of Mamba and the RG-LRU (reference:
// ohara/modules/pscan.py:63-258, a Blelloch up/down sweep of whole-tensor PyTorch operations that
// moves the tensors 2*log2(L) times).
//
// The scan is bound by memory traffic, and the channel dimension is large (batch x d_inner x
// d_state is of the order of 10^5), so the kernel parallelises over channels only: a thread owns
// four adjacent channels and walks the sequence once. Every step of a warp is one coalesced 512-byte
// access per tensor, the loads of kUnroll steps are issued before the first dependent multiply-add,
// and each tensor crosses HBM exactly once (read a, read x, write h). The backward pass is the same
// recurrence in reverse time with the coefficient of the next step,
//     g[t] = dh[t] + a[t+1] * g[t+1],   dx[t] = g[t],   da[t] = g[t] * h[t-1],
// again one pass: read dh, a, h; write dx, da.
#include "api.h"
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kUnroll = 4;

template <int V>
__device__ __forceinline__ void load_vec(const float* p, float (&out)[V]) {
  if constexpr (V == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x, out[1] = v.y, out[2] = v.z, out[3] = v.w;
  } else {
    out[0] = *p;
  }
}

template <int V>
__device__ __forceinline__ void store_vec(float* p, const float (&in)[V]) {
  if constexpr (V == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
  } else {
    *p = in[0];
  }
}

// `groups` = B * C / V thread-owned channel groups; `c_groups` = C / V of them per batch row.
template <int V>
__global__ void __launch_bounds__(128)
pscan_fwd_kernel(const float* __restrict__ a, const float* __restrict__ x, float* __restrict__ h,
                 int64_t groups, int64_t c_groups, int length, int64_t channels) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const int64_t b = idx / c_groups, c = (idx - b * c_groups) * V;
  const int64_t base = b * length * channels + c;
  float state[V];
#pragma unroll
  for (int v = 0; v < V; ++v) state[v] = 0.f;
  int t = 0;
  for (; t + kUnroll <= length; t += kUnroll) {
    float av[kUnroll][V], xv[kUnroll][V];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      load_vec<V>(a + base + (int64_t)(t + u) * channels, av[u]);
      load_vec<V>(x + base + (int64_t)(t + u) * channels, xv[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
      for (int v = 0; v < V; ++v) state[v] = fmaf(av[u][v], state[v], xv[u][v]);
      store_vec<V>(h + base + (int64_t)(t + u) * channels, state);
    }
  }
  for (; t < length; ++t) {
    float av[V], xv[V];
    load_vec<V>(a + base + (int64_t)t * channels, av);
    load_vec<V>(x + base + (int64_t)t * channels, xv);
#pragma unroll
    for (int v = 0; v < V; ++v) state[v] = fmaf(av[v], state[v], xv[v]);
    store_vec<V>(h + base + (int64_t)t * channels, state);
  }
}

template <int V>
__global__ void __launch_bounds__(128)
pscan_bwd_kernel(const float* __restrict__ a, const float* __restrict__ h,
                 const float* __restrict__ dh, float* __restrict__ da, float* __restrict__ dx,
                 int64_t groups, int64_t c_groups, int length, int64_t channels) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const int64_t b = idx / c_groups, c = (idx - b * c_groups) * V;
  const int64_t base = b * length * channels + c;
  float carry[V];  // a[t+1] * g[t+1]; nothing follows the last step
#pragma unroll
  for (int v = 0; v < V; ++v) carry[v] = 0.f;
  int t = length - 1;
  for (; t - kUnroll + 1 >= 1; t -= kUnroll) {  // steps t .. t-kUnroll+1, all with a predecessor
    float gv[kUnroll][V], av[kUnroll][V], hv[kUnroll][V];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      load_vec<V>(dh + base + (int64_t)(t - u) * channels, gv[u]);
      load_vec<V>(a + base + (int64_t)(t - u) * channels, av[u]);
      load_vec<V>(h + base + (int64_t)(t - u - 1) * channels, hv[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float g[V], ga[V];
#pragma unroll
      for (int v = 0; v < V; ++v) {
        g[v] = gv[u][v] + carry[v];
        ga[v] = g[v] * hv[u][v];
        carry[v] = av[u][v] * g[v];
      }
      store_vec<V>(dx + base + (int64_t)(t - u) * channels, g);
      store_vec<V>(da + base + (int64_t)(t - u) * channels, ga);
    }
  }
  for (; t >= 0; --t) {
    float gv[V], av[V], hv[V], g[V], ga[V];
    load_vec<V>(dh + base + (int64_t)t * channels, gv);
    load_vec<V>(a + base + (int64_t)t * channels, av);
    if (t > 0) {
      load_vec<V>(h + base + (int64_t)(t - 1) * channels, hv);
    } else {
#pragma unroll
      for (int v = 0; v < V; ++v) hv[v] = 0.f;  // h[-1] = 0
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
      g[v] = gv[v] + carry[v];
      ga[v] = g[v] * hv[v];
      carry[v] = av[v] * g[v];
    }
    store_vec<V>(dx + base + (int64_t)t * channels, g);
    store_vec<V>(da + base + (int64_t)t * channels, ga);
  }
}

inline bool vec4_ok(int64_t channels, std::initializer_list<const void*> ptrs) {
  if (channels % 4 != 0) return false;
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
  return true;
}

}  // namespace

void pscan_forward(const float* a, const float* x, float* h, int64_t batch, int length,
                   int64_t channels, cudaStream_t stream) {
  if (batch == 0 || length == 0 || channels == 0) return;
  const int threads = 128;
  if (vec4_ok(channels, {a, x, h})) {
    const int64_t groups = batch * (channels / 4);
    pscan_fwd_kernel<4><<<(unsigned)((groups + threads - 1) / threads), threads, 0, stream>>>(
        a, x, h, groups, channels / 4, length, channels);
  } else {
    const int64_t groups = batch * channels;
    pscan_fwd_kernel<1><<<(unsigned)((groups + threads - 1) / threads), threads, 0, stream>>>(
        a, x, h, groups, channels, length, channels);
  }
  OB_LAUNCH_CHECK();
}

void pscan_backward(const float* a, const float* h, const float* dh, float* da, float* dx,
                    int64_t batch, int length, int64_t channels, cudaStream_t stream) {
  if (batch == 0 || length == 0 || channels == 0) return;
  const int threads = 128;
  if (vec4_ok(channels, {a, h, dh, da, dx})) {
    const int64_t groups = batch * (channels / 4);
    pscan_bwd_kernel<4><<<(unsigned)((groups + threads - 1) / threads), threads, 0, stream>>>(
        a, h, dh, da, dx, groups, channels / 4, length, channels);
  } else {
    const int64_t groups = batch * channels;
    pscan_bwd_kernel<1><<<(unsigned)((groups + threads - 1) / threads), threads, 0, stream>>>(
        a, h, dh, da, dx, groups, channels, length, channels);
  }
  OB_LAUNCH_CHECK();
}

}  // namespace ob
