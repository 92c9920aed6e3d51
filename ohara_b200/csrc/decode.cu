// Serving kernels: fused RoPE + KV-cache append (bf16 or int8 cache), split-KV decode attention that
// reads the cache in place (native GQA, no mask tensor, no head expansion) and a fused
// temperature / top-k / top-p sampler. Positions and step counters may live on the device so a
// whole decode step can be replayed from a CUDA graph without host involvement.
#include <cfloat>

#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};
struct alignas(8) i8x8 {
  int8_t v[8];
};

__device__ __forceinline__ void unpack8(const bf16x8& in, float (&out)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(in.v[i]);
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

// ------------------------------------------------------------------------------------------------
// RoPE + cache append. Rows are (b, t, head) of q, k and v. One warp per row, lane l owns elements
// [8l, 8l+8) of the head (D <= 256). q and k rows are rotated on interleaved pairs with the table
// row of absolute position pos + t; k and v rows are then written into the cache at that
// position, either as bf16 or affine-quantised to int8 with one fp32 (scale, minimum) per row.
// ------------------------------------------------------------------------------------------------
template <bool INT8>
__global__ void rope_append_kernel(const __nv_bfloat16* __restrict__ q,
                                   const __nv_bfloat16* __restrict__ k,
                                   const __nv_bfloat16* __restrict__ v,
                                   __nv_bfloat16* __restrict__ q_out, void* __restrict__ cache_k,
                                   void* __restrict__ cache_v, float* __restrict__ k_scale,
                                   float* __restrict__ k_min, float* __restrict__ v_scale,
                                   float* __restrict__ v_min, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, int B, int T, int H, int Hk, int D,
                                   int pos_host, const int* __restrict__ pos_dev, int cache_len,
                                   int table_len) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int per_token = H + 2 * Hk;
  const int64_t rows = (int64_t)B * T * per_token;
  const int pos0 = pos_dev != nullptr ? *pos_dev : pos_host;
  const bool owner = lane * 8 < D;
  for (int64_t row = warp; row < rows; row += warps) {
    const int r = (int)(row % per_token);
    const int64_t bt = row / per_token;
    const int t = (int)(bt % T);
    const int b = (int)(bt / T);
    const int pos = pos0 + t;
    if (pos >= cache_len || pos >= table_len) continue;  // never write past the buffers
    const bool is_q = r < H;
    const bool is_k = !is_q && r < H + Hk;
    const int head = is_q ? r : (is_k ? r - H : r - H - Hk);
    const __nv_bfloat16* src = is_q ? q + (bt * H + head) * (int64_t)D
                                    : (is_k ? k : v) + (bt * Hk + head) * (int64_t)D;
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (owner) {
      unpack8(*reinterpret_cast<const bf16x8*>(src + lane * 8), f);
      if (is_q || is_k) {
        const float4 cs = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * (D >> 1) + lane * 4);
        const float4 sn = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * (D >> 1) + lane * 4);
        const float cc[4] = {cs.x, cs.y, cs.z, cs.w};
        const float ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = f[2 * i], c = f[2 * i + 1];
          f[2 * i] = a * cc[i] - c * ss[i];
          f[2 * i + 1] = a * ss[i] + c * cc[i];
        }
      }
    }
    if (is_q) {
      if (owner) *reinterpret_cast<bf16x8*>(q_out + (bt * H + head) * (int64_t)D + lane * 8) = pack8(f);
      continue;
    }
    const int64_t slot = ((int64_t)b * cache_len + pos) * Hk + head;
    if (!INT8) {
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(is_k ? cache_k : cache_v) + slot * D;
      if (owner) *reinterpret_cast<bf16x8*>(dst + lane * 8) = pack8(f);
    } else {
      // Quantise what a bf16 cache would hold, so both cache kinds see the same inputs.
      bf16x8 rounded = pack8(f);
      unpack8(rounded, f);
      float lo = FLT_MAX, hi = -FLT_MAX;
      if (owner) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          lo = fminf(lo, f[i]);
          hi = fmaxf(hi, f[i]);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      const float scale = fmaxf((hi - lo) / 255.f, 1e-8f);
      if (owner) {
        i8x8 packed;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float qv = rintf((f[i] - lo) / scale - 128.f);
          packed.v[i] = (int8_t)fminf(fmaxf(qv, -128.f), 127.f);
        }
        int8_t* dst = static_cast<int8_t*>(is_k ? cache_k : cache_v) + slot * D;
        *reinterpret_cast<i8x8*>(dst + lane * 8) = packed;
      }
      if (lane == 0) {
        (is_k ? k_scale : v_scale)[slot] = scale;
        (is_k ? k_min : v_min)[slot] = lo;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Decode attention: one query token per sequence against `len` cached keys. Grid (kv head, batch,
// split). A half-warp owns one key at a time (16 lanes x 8 elements = D 128; D 64 uses 8 lanes),
// keeps an online-softmax state for each of the G = H / Hk query heads of the group, and the
// eight half-warps of a CTA are merged through shared memory. With more than one split the CTA
// writes (max, sum, unnormalised output) and a second kernel merges the splits.
// ------------------------------------------------------------------------------------------------
constexpr int kDecodeThreads = 128;
constexpr int kMaxGroup = 8;

template <int D, int G, bool INT8>
__global__ void __launch_bounds__(kDecodeThreads)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const void* __restrict__ cache_k,
                   const void* __restrict__ cache_v, const float* __restrict__ k_scale,
                   const float* __restrict__ k_min, const float* __restrict__ v_scale,
                   const float* __restrict__ v_min, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ partial, int H, int Hk, int cache_len, int len_host,
                   const int* __restrict__ pos_dev, int splits, float scale_log2) {
  constexpr int LANES = D / 8;              // lanes that cooperate on one key
  constexpr int KEYS_PER_WARP = 32 / LANES; // keys a warp handles at once
  constexpr int GROUPS = (kDecodeThreads / 32) * KEYS_PER_WARP;
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int len = min(pos_dev != nullptr ? *pos_dev + 1 : len_host, cache_len);
  const int per_split = (len + splits - 1) / splits;
  const int begin = split * per_split;
  const int end = min(begin + per_split, len);
  const int sub = threadIdx.x % LANES;      // which 8 elements of the head this lane owns
  const int group = threadIdx.x / LANES;    // which key stream this lane belongs to

  float qf[G][8];
  float qtot[G];  // sum of the whole query head; the int8 path needs min_k * sum(q)
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int h = kvh * G + g;
    unpack8(*reinterpret_cast<const bf16x8*>(q + ((int64_t)b * H + h) * D + sub * 8), qf[g]);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += qf[g][i];
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    qtot[g] = s;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  // Every thread runs the same number of iterations (the shuffles below need whole warps); keys
  // past the end are loaded as zeros and skipped. Two keys per stream are in flight at a time.
  constexpr int U = 2;
  for (int base = begin; base < end; base += GROUPS * U) {
    float kf[U][8], vf[U][8], ks[U], km[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int key = base + u * GROUPS + group;
      valid[u] = key < end;
      ks[u] = 1.f;
      km[u] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) kf[u][i] = vf[u][i] = 0.f;
      if (valid[u]) {
        const int64_t slot = ((int64_t)b * cache_len + key) * Hk + kvh;
        if (INT8) {
          const i8x8 kq = *reinterpret_cast<const i8x8*>(static_cast<const int8_t*>(cache_k) + slot * D + sub * 8);
          const i8x8 vq = *reinterpret_cast<const i8x8*>(static_cast<const int8_t*>(cache_v) + slot * D + sub * 8);
          ks[u] = k_scale[slot];
          km[u] = k_min[slot];
          const float vs = v_scale[slot], vm = v_min[slot];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            kf[u][i] = (float)kq.v[i] + 128.f;
            vf[u][i] = ((float)vq.v[i] + 128.f) * vs + vm;
          }
        } else {
          unpack8(*reinterpret_cast<const bf16x8*>(static_cast<const __nv_bfloat16*>(cache_k) + slot * D + sub * 8), kf[u]);
          unpack8(*reinterpret_cast<const bf16x8*>(static_cast<const __nv_bfloat16*>(cache_v) + slot * D + sub * 8), vf[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += qf[g][i] * kf[u][i];
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (INT8) s = s * ks[u] + km[u] * qtot[g];
        if (valid[u]) {
          s *= scale_log2;
          const float m_new = fmaxf(m[g], s);
          const float corr = exp2f(m[g] - m_new);  // exp2(-inf) = 0 on the first key
          const float p = exp2f(s - m_new);
          l[g] = l[g] * corr + p;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * corr + p * vf[u][i];
          m[g] = m_new;
        }
      }
    }
  }

  // Merge the key streams of the CTA.
  __shared__ float sm_m[GROUPS][G];
  __shared__ float sm_l[GROUPS][G];
  __shared__ float sm_acc[GROUPS][G][D];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (sub == 0) {
      sm_m[group][g] = m[g];
      sm_l[group][g] = l[g];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_acc[group][g][sub * 8 + i] = acc[g][i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kDecodeThreads) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int s = 0; s < GROUPS; ++s) mm = fmaxf(mm, sm_m[s][g]);
    float ll = 0.f, o = 0.f;
#pragma unroll
    for (int s = 0; s < GROUPS; ++s) {
      const float w = sm_m[s][g] == -INFINITY ? 0.f : exp2f(sm_m[s][g] - mm);
      ll += sm_l[s][g] * w;
      o += sm_acc[s][g][d] * w;
    }
    const int h = kvh * G + g;
    if (splits == 1) {
      out[((int64_t)b * H + h) * D + d] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
    } else {
      float* dst = partial + (((int64_t)b * H + h) * splits + split) * (D + 2);
      dst[2 + d] = o;
      if (d == 0) {
        dst[0] = mm;
        dst[1] = ll;
      }
    }
  }
}

template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                    int splits) {
  const int64_t bh = blockIdx.x;
  const float* src = partial + bh * splits * (D + 2);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, src[s * (D + 2)]);
    float ll = 0.f, o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = src[s * (D + 2)];
      const float w = ms == -INFINITY ? 0.f : exp2f(ms - mm);
      ll += src[s * (D + 2) + 1] * w;
      o += src[s * (D + 2) + 2 + d] * w;
    }
    out[bh * D + d] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
  }
}

// ------------------------------------------------------------------------------------------------
// Sampler. One CTA per row of logits; the row lives in shared memory as fp32 when the vocabulary
// fits (else in a global workspace row). Steps:
//   1. mask ids >= valid_vocab; temperature 0 is a plain argmax (lowest id wins)
//   2. top-k: the exact k-th largest value, found by a two-bits-per-round search on the
//      order-preserving integer image of the floats; each round is a count of elements at or above
//      three pivots (no histograms, no atomics). Smaller values are dropped, ties are kept.
//   3. softmax over what is left
//   4. top-p: a token is dropped when the probability mass of the tokens ahead of it (more likely,
//      or equally likely with a lower id) already exceeds top_p, so the most likely token always
//      survives. With at most 1024 survivors (the usual case after top-k) every survivor sums the
//      mass ahead of it directly; otherwise a one-bit-per-round search finds the cut-off
//      probability (all tokens tied at the cut-off are then kept).
//   5. inverse-CDF draw over the kept tokens in index order with the caller's uniform number
// The chosen id goes to out_tokens[row * out_stride + step] and, optionally, next_input[row];
// the step counter and position are advanced by the last CTA to finish.
// ------------------------------------------------------------------------------------------------
constexpr int kSampleThreads = 1024;
constexpr int kMaxCandidates = 1024;

__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct MaxOp {
  template <typename T> __device__ T operator()(T a, T b) const { return a > b ? a : b; }
};
struct SumOp {
  template <typename T> __device__ T operator()(T a, T b) const { return a + b; }
};

// Block-wide reduction for 1024 threads; every thread gets the result. `scratch` holds 33 values.
template <typename T, typename Op>
__device__ T block_reduce(T v, T identity, Op op, T* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();  // protects scratch from the previous use
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    T r = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : identity;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = op(r, __shfl_xor_sync(0xffffffffu, r, o));
    if (threadIdx.x == 0) scratch[32] = r;
  }
  __syncthreads();
  return scratch[32];
}

template <typename LogitT>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const LogitT* __restrict__ logits, int64_t row_stride, int vocab, int valid_vocab,
              float temperature, int top_k, float top_p, const float* __restrict__ uniforms,
              int64_t* __restrict__ out_tokens, int64_t out_stride, int64_t* __restrict__ next_input,
              int* __restrict__ step_dev, int* __restrict__ pos_dev, unsigned int* __restrict__ done,
              float* __restrict__ workspace, bool use_smem) {
  extern __shared__ float smem_vals[];
  __shared__ float scratch_f[33];
  __shared__ unsigned long long scratch_u[33];
  __shared__ float cand_p[kMaxCandidates];
  __shared__ int cand_i[kMaxCandidates];
  __shared__ int cand_count;
  __shared__ int chosen_s;
  __shared__ float warp_tot[32];

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int step = step_dev != nullptr ? *step_dev : 0;
  float* vals = use_smem ? smem_vals : workspace + (size_t)row * vocab;
  const LogitT* src = logits + (size_t)row * row_stride;
  const int n = min(valid_vocab, vocab);

  // 1. load, find the maximum (and its first index for the greedy case)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < n; i += kSampleThreads) {
    const float x = (float)src[i];
    vals[i] = x;
    if (x > best) {
      best = x;
      best_i = i;
    }
  }
  const float vmax = block_reduce(best, -INFINITY, MaxOp(), scratch_f);
  int token;
  if (temperature <= 0.f) {
    if (tid == 0) chosen_s = 0x7fffffff;
    __syncthreads();
    if (best == vmax) atomicMin(&chosen_s, best_i);
    __syncthreads();
    token = chosen_s;
  } else {
    const float inv_t = 1.f / temperature;
    // 2. top-k threshold: the largest key T with count(key >= T) >= k, two bits per round.
    float threshold = -INFINITY;
    if (top_k > 0 && top_k < n) {
      uint32_t T = 0;
      for (int bit = 30; bit >= 0; bit -= 2) {
        const uint32_t p1 = T | (1u << bit), p2 = T | (2u << bit), p3 = T | (3u << bit);
        unsigned long long packed = 0;  // three 21-bit counters
        for (int i = tid; i < n; i += kSampleThreads) {
          const uint32_t key = ordered_key(vals[i]);
          packed += (unsigned long long)(key >= p1) + ((unsigned long long)(key >= p2) << 21) +
                    ((unsigned long long)(key >= p3) << 42);
        }
        packed = block_reduce(packed, 0ull, SumOp(), scratch_u);
        const int c1 = (int)(packed & 0x1fffff), c2 = (int)((packed >> 21) & 0x1fffff),
                  c3 = (int)((packed >> 42) & 0x1fffff);
        if (c3 >= top_k) T = p3; else if (c2 >= top_k) T = p2; else if (c1 >= top_k) T = p1;
      }
      threshold = key_to_float(T);
    }
    // 3. unnormalised probabilities of what survived top-k
    float local = 0.f;
    int survivors = 0;
    for (int i = tid; i < n; i += kSampleThreads) {
      const float x = vals[i];
      const float p = x >= threshold ? __expf((x - vmax) * inv_t) : 0.f;
      vals[i] = p;
      local += p;
      survivors += p > 0.f;
    }
    float total = block_reduce(local, 0.f, SumOp(), scratch_f);
    // 4. top-p
    if (top_p > 0.f && top_p < 1.f) {
      const int alive = (int)block_reduce((unsigned long long)survivors, 0ull, SumOp(), scratch_u);
      const float budget = top_p * total;
      if (alive <= kMaxCandidates) {
        if (tid == 0) cand_count = 0;
        __syncthreads();
        for (int i = tid; i < n; i += kSampleThreads) {
          const float p = vals[i];
          if (p > 0.f) {
            const int at = atomicAdd(&cand_count, 1);
            cand_p[at] = p;
            cand_i[at] = i;
          }
        }
        __syncthreads();
        if (tid < alive) {
          const float p = cand_p[tid];
          const int idx = cand_i[tid];
          float ahead = 0.f;
          for (int j = 0; j < alive; ++j) {
            const float pj = cand_p[j];
            if (pj > p || (pj == p && cand_i[j] < idx)) ahead += pj;
          }
          if (ahead > budget) vals[idx] = 0.f;
        }
      } else {
        // Largest probability T (as bits) with mass(p >= T) > budget; tokens below it are dropped.
        uint32_t T = 0;
        for (int bit = 30; bit >= 0; --bit) {
          const uint32_t pivot = T | (1u << bit);
          float mass = 0.f;
          for (int i = tid; i < n; i += kSampleThreads) {
            const float p = vals[i];
            if (__float_as_uint(p) >= pivot) mass += p;  // positive floats order like their bits
          }
          mass = block_reduce(mass, 0.f, SumOp(), scratch_f);
          if (mass > budget) T = pivot;
        }
        // Tokens above the cut-off all stay. Tokens exactly at it stay, in index order, while the
        // mass ahead of them is within the budget.
        const float cut = __uint_as_float(T);
        float above = 0.f;
        for (int i = tid; i < n; i += kSampleThreads) {
          const float p = vals[i];
          if (__float_as_uint(p) > T) above += p;
        }
        above = block_reduce(above, 0.f, SumOp(), scratch_f);
        const int keep_ties = cut > 0.f ? (int)fminf(floorf(fmaxf(budget - above, 0.f) / cut), 2.0e9f) + 1 : 0;
        const int per = (n + kSampleThreads - 1) / kSampleThreads;
        const int first = min(tid * per, n), last = min(first + per, n);
        int ties = 0;
        for (int i = first; i < last; ++i) ties += __float_as_uint(vals[i]) == T;
        int incl_t = ties;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl_t, o);
          if ((tid & 31) >= o) incl_t += up;
        }
        __syncthreads();
        if ((tid & 31) == 31) cand_i[tid >> 5] = incl_t;
        __syncthreads();
        int tie_rank = incl_t - ties;  // ties before this thread's chunk
        for (int w = 0; w < (tid >> 5); ++w) tie_rank += cand_i[w];
        for (int i = first; i < last; ++i) {
          const uint32_t bits = __float_as_uint(vals[i]);
          if (bits < T) vals[i] = 0.f;
          else if (bits == T && tie_rank++ >= keep_ties) vals[i] = 0.f;
        }
      }
      __syncthreads();
    }
    // 5. inverse CDF in index order: thread t owns a contiguous chunk
    const int chunk = (n + kSampleThreads - 1) / kSampleThreads;
    const int lo = min(tid * chunk, n), hi = min(lo + chunk, n);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i) mine += vals[i];
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if ((tid & 31) >= o) incl += up;
    }
    if ((tid & 31) == 31) warp_tot[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
      float w = warp_tot[tid];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, w, o);
        if (tid >= o) w += up;
      }
      warp_tot[tid] = w;
    }
    if (tid == 0) chosen_s = -1;
    __syncthreads();
    const float before = incl - mine + ((tid >> 5) > 0 ? warp_tot[(tid >> 5) - 1] : 0.f);
    const float grand = warp_tot[31];
    const float u = uniforms != nullptr ? uniforms[(size_t)step * gridDim.x + row] : 0.5f;
    const float target = fminf(fmaxf(u, 0.f), 0.99999994f) * grand;
    if (mine > 0.f && target >= before && target < before + mine) {
      float run = before;
      int pick = -1;
      for (int i = lo; i < hi; ++i) {
        if (vals[i] > 0.f) {
          pick = i;  // falls back to the chunk's last kept token against round-off
          run += vals[i];
          if (target < run) break;
        }
      }
      atomicMax(&chosen_s, pick);
    }
    __syncthreads();
    const int found = chosen_s;
    __syncthreads();  // everyone has read the result before anyone may change it
    if (found < 0) {
      // Round-off left the target beyond the last chunk: take the last kept token.
      int last = -1;
      for (int i = lo; i < hi; ++i)
        if (vals[i] > 0.f) last = i;
      atomicMax(&chosen_s, last);
      __syncthreads();
    }
    token = chosen_s;
  }
  if (tid == 0) {
    out_tokens[(size_t)row * out_stride + step] = token;
    if (next_input != nullptr) next_input[row] = token;
    if (done != nullptr) {
      __threadfence();
      const unsigned int finished = atomicAdd(done, 1u) + 1;
      if (finished == gridDim.x) {  // last row of this step: advance the device-side counters
        *done = 0;
        if (step_dev != nullptr) *step_dev = step + 1;
        if (pos_dev != nullptr) *pos_dev = *pos_dev + 1;
      }
    }
  }
}

}  // namespace

void rope_append(const void* q, const void* k, const void* v, void* q_out, void* cache_k,
                 void* cache_v, float* k_scale, float* k_min, float* v_scale, float* v_min,
                 const float* cos_t, const float* sin_t, int B, int T, int H, int Hk, int D, int pos,
                 const int* pos_dev, int cache_len, int table_len, bool int8, cudaStream_t stream) {
  OB_CHECK(D % 8 == 0 && D <= 256, "rope_append: head_dim must be a multiple of 8, at most 256");
  const int64_t rows = (int64_t)B * T * (H + 2 * Hk);
  if (rows == 0) return;
  const int blocks = (int)std::min<int64_t>((rows + 7) / 8, device_sm_count() * 16);
  auto launch = [&](auto kernel) {
    kernel<<<blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
        static_cast<const __nv_bfloat16*>(v), static_cast<__nv_bfloat16*>(q_out), cache_k, cache_v,
        k_scale, k_min, v_scale, v_min, cos_t, sin_t, B, T, H, Hk, D, pos, pos_dev, cache_len,
        table_len);
  };
  if (int8) launch(rope_append_kernel<true>); else launch(rope_append_kernel<false>);
  OB_LAUNCH_CHECK();
}

int decode_attention_splits(int B, int Hk, int len) {
  // Enough CTAs to cover the machine, at least 256 keys per CTA, at most 16 splits.
  const int base = std::max(B * Hk, 1);
  int splits = (device_sm_count() + base - 1) / base;
  splits = std::min(splits, std::max(len / 256, 1));
  return std::max(1, std::min(splits, 16));
}

template <int D, bool INT8>
static void launch_decode(int G, dim3 grid, cudaStream_t stream, const void* q, const void* ck,
                          const void* cv, const float* ks, const float* km, const float* vs,
                          const float* vm, void* out, float* partial, int H, int Hk, int cache_len,
                          int len, const int* pos_dev, int splits, float scale_log2) {
#define OB_DECODE_CASE(GV)                                                                        \
  case GV:                                                                                        \
    decode_attn_kernel<D, GV, INT8><<<grid, kDecodeThreads, 0, stream>>>(                         \
        static_cast<const __nv_bfloat16*>(q), ck, cv, ks, km, vs, vm,                             \
        static_cast<__nv_bfloat16*>(out), partial, H, Hk, cache_len, len, pos_dev, splits,        \
        scale_log2);                                                                              \
    break;
  switch (G) {
    OB_DECODE_CASE(1)
    OB_DECODE_CASE(2)
    OB_DECODE_CASE(4)
    OB_DECODE_CASE(8)
    default:
      OB_CHECK(false, "decode attention supports 1, 2, 4 or 8 query heads per KV head");
  }
#undef OB_DECODE_CASE
}

void decode_attention(const void* q, const void* cache_k, const void* cache_v, const float* k_scale,
                      const float* k_min, const float* v_scale, const float* v_min, void* out,
                      float* partial, int B, int H, int Hk, int D, int cache_len, int len,
                      const int* pos_dev, int splits, float scale, bool int8, cudaStream_t stream) {
  OB_CHECK(D == 64 || D == 128, "decode attention supports head_dim 64 and 128");
  OB_CHECK(H % Hk == 0 && H / Hk <= kMaxGroup, "unsupported query/KV head ratio");
  OB_CHECK(splits >= 1 && (splits == 1 || partial != nullptr), "splits need a partial buffer");
  if (B == 0) return;
  const float scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid(Hk, B, splits);
  const int G = H / Hk;
  if (D == 128) {
    if (int8) launch_decode<128, true>(G, grid, stream, q, cache_k, cache_v, k_scale, k_min, v_scale, v_min, out, partial, H, Hk, cache_len, len, pos_dev, splits, scale_log2);
    else launch_decode<128, false>(G, grid, stream, q, cache_k, cache_v, k_scale, k_min, v_scale, v_min, out, partial, H, Hk, cache_len, len, pos_dev, splits, scale_log2);
  } else {
    if (int8) launch_decode<64, true>(G, grid, stream, q, cache_k, cache_v, k_scale, k_min, v_scale, v_min, out, partial, H, Hk, cache_len, len, pos_dev, splits, scale_log2);
    else launch_decode<64, false>(G, grid, stream, q, cache_k, cache_v, k_scale, k_min, v_scale, v_min, out, partial, H, Hk, cache_len, len, pos_dev, splits, scale_log2);
  }
  OB_LAUNCH_CHECK();
  if (splits > 1) {
    if (D == 128) decode_merge_kernel<128><<<B * H, 128, 0, stream>>>(partial, static_cast<__nv_bfloat16*>(out), splits);
    else decode_merge_kernel<64><<<B * H, 64, 0, stream>>>(partial, static_cast<__nv_bfloat16*>(out), splits);
    OB_LAUNCH_CHECK();
  }
}

size_t sample_smem_limit() {
  static size_t limit = [] {
    int dev = 0, bytes = 0;
    OB_CUDA_CHECK(cudaGetDevice(&dev));
    OB_CUDA_CHECK(cudaDeviceGetAttribute(&bytes, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    return (size_t)bytes;
  }();
  return limit;
}

void sample_tokens(const void* logits, bool logits_bf16, int64_t row_stride, int rows, int vocab,
                   int valid_vocab, float temperature, int top_k, float top_p,
                   const float* uniforms, int64_t* out_tokens, int64_t out_stride,
                   int64_t* next_input, int* step_dev, int* pos_dev, unsigned int* done,
                   float* workspace, cudaStream_t stream) {
  if (rows == 0) return;
  OB_CHECK(valid_vocab >= 1, "sampler needs at least one valid token");
  // Static shared memory of the kernel is about 9 KB; leave room for it.
  const size_t need = (size_t)vocab * sizeof(float);
  const bool use_smem = need + 10240 <= sample_smem_limit();
  OB_CHECK(use_smem || workspace != nullptr, "vocabulary too large for shared memory: pass a workspace");
  auto launch = [&](auto kernel, auto* typed) {
    if (use_smem) {
      ensure_dynamic_smem((const void*)kernel, need);
    }
    kernel<<<rows, kSampleThreads, use_smem ? need : 0, stream>>>(
        typed, row_stride, vocab, valid_vocab, temperature, top_k, top_p, uniforms, out_tokens,
        out_stride, next_input, step_dev, pos_dev, done, workspace, use_smem);
  };
  if (logits_bf16) launch(sample_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(logits));
  else launch(sample_kernel<float>, static_cast<const float*>(logits));
  OB_LAUNCH_CHECK();
}

}  // namespace ob
