// Mixture-of-experts bookkeeping kernels: router top-k(+1) with gate weights and expert counts,
// the dispatch plan (tile-padded expert segments), row permutation / weighted combine, and the
// per-expert quantile used by quantile balancing. None of them synchronises with the host.
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kMaxExpertsPerLane = 8;  // up to 256 experts, one warp per token
constexpr int kMaxTopK = 16;

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------------
// Router: for each token pick the k best experts by (logit + bias); the (k+1)-th biased score is
// the balancing threshold alpha. Gate weights come from the *unbiased* logits of the chosen
// experts: softmax over the k, or sigmoid (optionally normalised to sum 1). Ties go to the lower
// expert index, as torch.topk does. One warp per token; expert e lives in lane e % 32.
// ------------------------------------------------------------------------------------------------
__global__ void route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                  int* __restrict__ indices, float* __restrict__ weights,
                                  float* __restrict__ alpha, int* __restrict__ counts, int tokens,
                                  int experts, int k, bool sigmoid_gate, bool normalize,
                                  bool want_alpha) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < tokens; t += warps) {
    float raw[kMaxExpertsPerLane], biased[kMaxExpertsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      raw[i] = e < experts ? logits[(size_t)t * experts + e] : -INFINITY;
      biased[i] = e < experts ? raw[i] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
    }
    float chosen_raw = 0.f;  // lane j < k keeps the raw logit of the j-th pick
    int chosen_idx = 0;
    const int rounds = want_alpha ? k + 1 : k;
    for (int r = 0; r < rounds; ++r) {
      float best = -INFINITY;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        if (biased[i] > best) {  // strict: the lowest index wins inside a lane
          best = biased[i];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if (r == k) {
        if (lane == 0) alpha[t] = best;
        break;
      }
      // The owner of the winner retires it and publishes its raw logit.
      float win_raw = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        if (lane + 32 * i == best_e) {
          win_raw = raw[i];
          biased[i] = -INFINITY;
        }
      }
      win_raw = __shfl_sync(0xffffffffu, win_raw, best_e & 31);
      if (lane == r) {
        chosen_raw = win_raw;
        chosen_idx = best_e;
      }
    }
    const bool active = lane < k;
    float w;
    if (sigmoid_gate) {
      w = active ? 1.f / (1.f + __expf(-chosen_raw)) : 0.f;
      if (normalize) w = w / fmaxf(warp_sum(w), 1e-9f);
    } else {
      const float m = warp_max(active ? chosen_raw : -INFINITY);
      const float ex = active ? __expf(chosen_raw - m) : 0.f;
      w = ex / warp_sum(ex);
    }
    if (active) {
      indices[(size_t)t * k + lane] = chosen_idx;
      weights[(size_t)t * k + lane] = w;
      if (counts != nullptr) atomicAdd(&counts[chosen_idx], 1);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Dispatch plan from the expert counts (one CTA): every expert's segment starts on a multiple of
// `tile` rows. Writes segment boundaries k_offsets[E+1], the expert of every tile (-1 for unused
// tiles) and resets the placement cursors.
// ------------------------------------------------------------------------------------------------
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ seg_start,
                                int* __restrict__ k_offsets, int* __restrict__ tile_expert,
                                int* __restrict__ cursor, int experts, int tile, int num_tiles) {
  extern __shared__ int ends[];  // experts entries
  if (threadIdx.x == 0) {
    int at = 0;
    k_offsets[0] = 0;
    for (int e = 0; e < experts; ++e) {
      seg_start[e] = at;
      at += (counts[e] + tile - 1) / tile * tile;
      ends[e] = at;
      k_offsets[e + 1] = at;
    }
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  for (int t = threadIdx.x; t < num_tiles; t += blockDim.x) {
    const int begin = t * tile;
    int lo = 0, hi = experts;  // first expert whose segment end exceeds `begin`
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (ends[mid] > begin) hi = mid; else lo = mid + 1;
    }
    tile_expert[t] = lo < experts ? lo : -1;
  }
}

// ------------------------------------------------------------------------------------------------
// Placement: pair j = (token j / k, slot j % k) gets the next free row of its expert's segment.
// The order of rows inside a segment depends on scheduling, but every consumer addresses rows
// through `dest_row`, so results do not.
// ------------------------------------------------------------------------------------------------
__global__ void moe_place_kernel(const int* __restrict__ indices, const int* __restrict__ seg_start,
                                 int* __restrict__ cursor, int* __restrict__ dest_row,
                                 int* __restrict__ row_pair, int64_t pairs) {
  for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < pairs;
       j += (int64_t)gridDim.x * blockDim.x) {
    const int e = indices[j];
    const int row = seg_start[e] + atomicAdd(&cursor[e], 1);
    dest_row[j] = row;
    row_pair[row] = (int)j;
  }
}

// ------------------------------------------------------------------------------------------------
// Scatter rows: dst[dest_row[j]] = scale_j * src[j / k]. One warp per pair.
// Used for the forward permutation (scale = 1) and for the backward of the combine (scale = gate
// weight of the pair).
// ------------------------------------------------------------------------------------------------
__global__ void moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src,
                                        const int* __restrict__ dest_row,
                                        const float* __restrict__ scale,
                                        __nv_bfloat16* __restrict__ dst, int64_t pairs, int k, int d) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int vecs = d >> 3;
  for (int64_t j = warp; j < pairs; j += warps) {
    const bf16x8* in = reinterpret_cast<const bf16x8*>(src + (j / k) * (int64_t)d);
    bf16x8* out = reinterpret_cast<bf16x8*>(dst + (int64_t)dest_row[j] * d);
    const float s = scale != nullptr ? scale[j] : 1.f;
    for (int v = lane; v < vecs; v += 32) {
      bf16x8 x = in[v];
      if (scale != nullptr) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(x.v[i]);
          x.v[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
      }
      out[v] = x;
    }
  }
}

// Rows of a padded buffer that no pair maps to (row_pair < 0) must read as zero: they sit inside
// expert segments and take part in the weight-gradient GEMMs.
__global__ void moe_zero_padding_kernel(const int* __restrict__ row_pair,
                                        __nv_bfloat16* __restrict__ dst, int64_t rows, int d) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int vecs = d >> 3;
  for (int64_t row = warp; row < rows; row += warps) {
    if (row_pair[row] >= 0) continue;
    uint4* out = reinterpret_cast<uint4*>(dst + row * d);
    for (int v = lane; v < vecs; v += 32) out[v] = make_uint4(0u, 0u, 0u, 0u);
  }
}

// ------------------------------------------------------------------------------------------------
// Gather-combine: out[t] = sum_i scale[t,i] * rows[dest_row[t*k+i]] (fp32 accumulation). With
// `other` given it also writes dot[t,i] = <rows[dest_row[t*k+i]], other[t]>, the gradient of the
// gate weight. One warp per token. Used for the forward combine (scale = gate weights) and for
// the backward of the permutation (scale = nullptr, i.e. 1).
// ------------------------------------------------------------------------------------------------
__global__ void moe_gather_combine_kernel(const __nv_bfloat16* __restrict__ rows,
                                          const int* __restrict__ dest_row,
                                          const float* __restrict__ scale,
                                          const __nv_bfloat16* __restrict__ other,
                                          __nv_bfloat16* __restrict__ out, float* __restrict__ dot,
                                          int64_t tokens, int k, int d) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int vecs = d >> 3;
  for (int64_t t = warp; t < tokens; t += warps) {
    float dots[kMaxTopK];
#pragma unroll
    for (int i = 0; i < kMaxTopK; ++i) dots[i] = 0.f;
    for (int v = lane; v < vecs; v += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      float oth[8];
      if (other != nullptr) {
        const bf16x8 o = reinterpret_cast<const bf16x8*>(other + t * (int64_t)d)[v];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(o.v[i]);
          oth[2 * i] = f.x;
          oth[2 * i + 1] = f.y;
        }
      }
#pragma unroll
      for (int i = 0; i < kMaxTopK; ++i) {
        if (i >= k) break;
        const int64_t j = t * k + i;
        const bf16x8 r = reinterpret_cast<const bf16x8*>(rows + (int64_t)dest_row[j] * d)[v];
        const float s = scale != nullptr ? scale[j] : 1.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float2 f = __bfloat1622float2(r.v[c]);
          acc[2 * c] += s * f.x;
          acc[2 * c + 1] += s * f.y;
          if (other != nullptr) dots[i] += f.x * oth[2 * c] + f.y * oth[2 * c + 1];
        }
      }
      if (out != nullptr) {
        bf16x8 packed;
#pragma unroll
        for (int c = 0; c < 4; ++c) packed.v[c] = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
        reinterpret_cast<bf16x8*>(out + t * (int64_t)d)[v] = packed;
      }
    }
    if (other != nullptr && dot != nullptr) {
#pragma unroll
      for (int i = 0; i < kMaxTopK; ++i) {
        if (i >= k) break;
        const float total = warp_sum(dots[i]);
        if (lane == 0) dot[t * k + i] = total;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Quantile select: beta[e] = the `rank`-th largest value of (logits[t, e] - alpha[t]) over tokens.
// One CTA per expert; an exact 4-pass radix select on order-preserving 32-bit keys.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__global__ void qb_quantile_kernel(const float* __restrict__ logits, const float* __restrict__ alpha,
                                   float* __restrict__ beta_sum, int tokens, int experts, int rank) {
  __shared__ int hist[256];
  __shared__ uint32_t prefix_s;
  __shared__ int remaining_s;
  const int e = blockIdx.x;
  if (threadIdx.x == 0) {
    prefix_s = 0;
    remaining_s = rank;  // looking for the `remaining`-th largest among keys matching the prefix
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = prefix_s;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int t = threadIdx.x; t < tokens; t += blockDim.x) {
      const uint32_t key = ordered_key(logits[(size_t)t * experts + e] - alpha[t]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int remaining = remaining_s;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (hist[bin] >= remaining) break;
        remaining -= hist[bin];
      }
      prefix_s = prefix | ((uint32_t)bin << shift);
      remaining_s = remaining;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) beta_sum[e] += key_to_float(prefix_s);
}

}  // namespace

void route_topk(const float* logits, const float* bias, int* indices, float* weights, float* alpha,
                int* counts, int tokens, int experts, int k, bool sigmoid_gate, bool normalize,
                bool want_alpha, cudaStream_t stream) {
  OB_CHECK(experts >= 1 && experts <= 32 * kMaxExpertsPerLane, "router supports up to 256 experts");
  OB_CHECK(k >= 1 && k <= kMaxTopK && k + (want_alpha ? 1 : 0) <= experts, "invalid top-k");
  if (tokens == 0) return;
  const int threads = 256;
  const int blocks = std::min((tokens + 7) / 8, device_sm_count() * 8);
  route_topk_kernel<<<blocks, threads, 0, stream>>>(logits, bias, indices, weights, alpha, counts,
                                                    tokens, experts, k, sigmoid_gate, normalize,
                                                    want_alpha);
  OB_LAUNCH_CHECK();
}

void moe_plan(const int* indices, const int* counts, int* seg_start, int* k_offsets,
              int* tile_expert, int* cursor, int* dest_row, int* row_pair, int64_t pairs,
              int experts, int tile, int num_tiles, cudaStream_t stream) {
  OB_CHECK(experts >= 1 && experts <= 4096, "too many experts for the plan kernel");
  moe_plan_kernel<<<1, 256, experts * sizeof(int), stream>>>(counts, seg_start, k_offsets,
                                                             tile_expert, cursor, experts, tile,
                                                             num_tiles);
  OB_LAUNCH_CHECK();
  if (pairs == 0) return;
  const int blocks = (int)std::min<int64_t>((pairs + 255) / 256, device_sm_count() * 8);
  moe_place_kernel<<<blocks, 256, 0, stream>>>(indices, seg_start, cursor, dest_row, row_pair, pairs);
  OB_LAUNCH_CHECK();
}

void moe_scatter_rows(const void* src, const int* dest_row, const float* scale,
                      const int* row_pair, int64_t padded_rows, void* dst, int64_t pairs, int k,
                      int d, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "row width must be a multiple of 8");
  if (row_pair != nullptr && padded_rows > 0) {
    const int zblocks = (int)std::min<int64_t>((padded_rows + 7) / 8, device_sm_count() * 16);
    moe_zero_padding_kernel<<<zblocks, 256, 0, stream>>>(row_pair, static_cast<__nv_bfloat16*>(dst),
                                                         padded_rows, d);
    OB_LAUNCH_CHECK();
  }
  if (pairs == 0) return;
  const int blocks = (int)std::min<int64_t>((pairs + 7) / 8, device_sm_count() * 16);
  moe_scatter_rows_kernel<<<blocks, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(src), dest_row, scale, static_cast<__nv_bfloat16*>(dst),
      pairs, k, d);
  OB_LAUNCH_CHECK();
}

void moe_gather_combine(const void* rows, const int* dest_row, const float* scale, const void* other,
                        void* out, float* dot, int64_t tokens, int k, int d, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "row width must be a multiple of 8");
  OB_CHECK(k >= 1 && k <= kMaxTopK, "top-k out of range");
  if (tokens == 0) return;
  const int blocks = (int)std::min<int64_t>((tokens + 7) / 8, device_sm_count() * 16);
  moe_gather_combine_kernel<<<blocks, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(rows), dest_row, scale,
      static_cast<const __nv_bfloat16*>(other), static_cast<__nv_bfloat16*>(out), dot, tokens, k, d);
  OB_LAUNCH_CHECK();
}

void qb_quantile(const float* logits, const float* alpha, float* beta_sum, int tokens, int experts,
                 int rank, cudaStream_t stream) {
  OB_CHECK(rank >= 1 && rank <= tokens, "quantile rank out of range");
  qb_quantile_kernel<<<experts, 512, 0, stream>>>(logits, alpha, beta_sum, tokens, experts, rank);
  OB_LAUNCH_CHECK();
}

}  // namespace ob
