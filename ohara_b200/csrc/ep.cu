// Expert-parallel dispatch / combine over NVLink peer memory. Every rank of the group owns
// E / world experts. The all-to-all of a mixture-of-experts layer is folded into the permutation
// kernels: the rank that owns a token writes the token's row straight into the expert-contiguous,
// tile-padded buffer of the rank that owns the expert (peer stores), and later reads the expert's
// output row straight from there while it applies the gate weights (peer loads). Nothing is packed
// into send buffers and no collective library call is made.
//
// Layout agreement: after the ranks have exchanged their per-expert counts, every rank computes the
// same plan. On the owner of expert e the rows of e form one segment that starts on a multiple of
// `tile` rows; inside the segment the sources follow each other in rank order.
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kMaxEP = 8;
constexpr int kMaxTopK = 16;

struct PtrTable {
  void* ptr[kMaxEP];
};

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// counts[E] of this rank -> row `rank` of the (world x E) table on every rank.
__global__ void ep_publish_counts_kernel(PtrTable tables, const int* __restrict__ counts, int experts,
                                         int rank, int world) {
  for (int i = threadIdx.x; i < experts; i += blockDim.x) {
    const int c = counts[i];
    for (int r = 0; r < world; ++r) static_cast<int*>(tables.ptr[r])[rank * experts + i] = c;
  }
}

// One CTA. From the full (world x E) count table: where this rank's pairs of expert e start on the
// owner (`pair_base`), and for the experts this rank owns the segment boundaries (`k_offsets`), the
// expert of every tile, and the padding rows to clear ([fill_begin, fill_end) per local expert).
__global__ void ep_plan_kernel(const int* __restrict__ table, int experts, int world, int rank,
                               int tile, int num_tiles, int capacity_rows,
                               int* __restrict__ pair_base,
                               int* __restrict__ k_offsets, int* __restrict__ tile_expert,
                               int* __restrict__ fill_begin, int* __restrict__ fill_end,
                               int* __restrict__ cursor, int* __restrict__ rows_used) {
  extern __shared__ int ends[];  // local experts
  const int local = experts / world;
  if (threadIdx.x == 0) {
    for (int r = 0; r < world; ++r) {
      int at = 0;
      for (int el = 0; el < local; ++el) {
        const int e = r * local + el;
        int total = 0, before = 0;
        for (int s = 0; s < world; ++s) {
          const int c = table[s * experts + e];
          if (s < rank) before += c;
          total += c;
        }
        pair_base[e] = at + before;
        const int padded = (total + tile - 1) / tile * tile;
        if (r == rank) {
          // Rows that do not fit the buffer are dropped (their pairs get no destination), so every
          // boundary is clamped to the capacity.
          k_offsets[el] = min(at, capacity_rows);
          fill_begin[el] = min(at + total, capacity_rows);
          fill_end[el] = min(at + padded, capacity_rows);
          ends[el] = min(at + padded, capacity_rows);
        }
        at += padded;
      }
      if (r == rank) {
        k_offsets[local] = min(at, capacity_rows);
        *rows_used = at;  // above the capacity: pairs were dropped
      }
    }
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  for (int t = threadIdx.x; t < num_tiles; t += blockDim.x) {
    const int begin = t * tile;
    int lo = 0, hi = local;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (ends[mid] > begin) hi = mid; else lo = mid + 1;
    }
    tile_expert[t] = lo < local ? lo : -1;
  }
}

// Pair j -> (owner rank of its expert, row in the owner's padded buffer).
__global__ void ep_place_kernel(const int* __restrict__ indices, const int* __restrict__ pair_base,
                                int* __restrict__ cursor, int* __restrict__ dest_rank,
                                int* __restrict__ dest_row, int64_t pairs, int local_experts,
                                int capacity_rows) {
  for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < pairs;
       j += (int64_t)gridDim.x * blockDim.x) {
    const int e = indices[j];
    const int row = pair_base[e] + atomicAdd(&cursor[e], 1);
    dest_rank[j] = e / local_experts;
    dest_row[j] = row < capacity_rows ? row : -1;  // beyond the buffer: the pair is dropped
  }
}

__global__ void ep_zero_fill_kernel(const int* __restrict__ fill_begin, const int* __restrict__ fill_end,
                                    __nv_bfloat16* __restrict__ buffer, int local_experts, int d,
                                    int capacity_rows) {
  const int lane = threadIdx.x & 31;
  const int warp_in_block = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  const int vecs = d >> 3;
  for (int el = blockIdx.y; el < local_experts; el += gridDim.y) {
    const int end = min(fill_end[el], capacity_rows);
    for (int row = fill_begin[el] + blockIdx.x * warps_per_block + warp_in_block; row < end;
         row += gridDim.x * warps_per_block) {
      uint4* out = reinterpret_cast<uint4*>(buffer + (int64_t)row * d);
      for (int v = lane; v < vecs; v += 32) out[v] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// buffers[dest_rank[j]][dest_row[j]] = scale_j * src[j / k]: one warp per *token*. The token's row
// is loaded once into registers (VPL 16-byte vectors per lane, all loads in flight together) and
// stored to its k destinations, remote for pairs whose expert lives on another rank; the
// destinations of a token are fetched by the first k lanes and broadcast. VPL = 0 is the generic
// form for row widths that are not a multiple of 256 elements.
template <int VPL>
__global__ void ep_push_rows_kernel(const __nv_bfloat16* __restrict__ src,
                                    const int* __restrict__ dest_rank, const int* __restrict__ dest_row,
                                    const float* __restrict__ scale, PtrTable buffers, int64_t pairs,
                                    int k, int d, int world, int capacity, int* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int vecs = d >> 3;
  const int64_t tokens = pairs / k;
  for (int64_t t = warp; t < tokens; t += warps) {
    const bf16x8* in = reinterpret_cast<const bf16x8*>(src + t * (int64_t)d);
    int my_row = -1, my_rank = 0;
    float my_scale = 1.f;
    if (lane < k) {
      my_row = dest_row[t * k + lane];
      my_rank = dest_rank[t * k + lane];
      if (scale != nullptr) my_scale = scale[t * k + lane];
      // A destination outside the peers' buffers would be a store into memory that is not ours
      // to write: record it in the status word and drop the pair instead.
      if (my_row >= 0 && (my_row >= capacity || my_rank < 0 || my_rank >= world)) {
        report_status(status, kBadArgument);
        my_row = -1;
      }
    }
    if constexpr (VPL > 0) {
      bf16x8 x[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) x[i] = in[lane + 32 * i];
      for (int i = 0; i < k; ++i) {
        const int row = __shfl_sync(0xffffffffu, my_row, i);
        const int rank = __shfl_sync(0xffffffffu, my_rank, i);
        const float sc = __shfl_sync(0xffffffffu, my_scale, i);
        if (row < 0) continue;
        bf16x8* out = reinterpret_cast<bf16x8*>(static_cast<__nv_bfloat16*>(buffers.ptr[rank]) +
                                                (int64_t)row * d);
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          bf16x8 y = x[v];
          if (scale != nullptr) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float2 f = __bfloat1622float2(y.v[c]);
              y.v[c] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
            }
          }
          out[lane + 32 * v] = y;
        }
      }
    } else {
      for (int i = 0; i < k; ++i) {
        const int row = __shfl_sync(0xffffffffu, my_row, i);
        const int rank = __shfl_sync(0xffffffffu, my_rank, i);
        const float sc = __shfl_sync(0xffffffffu, my_scale, i);
        if (row < 0) continue;
        bf16x8* out = reinterpret_cast<bf16x8*>(static_cast<__nv_bfloat16*>(buffers.ptr[rank]) +
                                                (int64_t)row * d);
        for (int v = lane; v < vecs; v += 32) {
          bf16x8 y = in[v];
          if (scale != nullptr) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float2 f = __bfloat1622float2(y.v[c]);
              y.v[c] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
            }
          }
          out[v] = y;
        }
      }
    }
  }
}

// out[t] = sum_i scale[t,i] * buffers[dest_rank][dest_row] (fp32 accumulation); with `other` also
// dot[t,i] = <row, other[t]>. One warp per token; rows are read through the peers' buffers.
__global__ void ep_pull_combine_kernel(PtrTable buffers, const int* __restrict__ dest_rank,
                                       const int* __restrict__ dest_row,
                                       const float* __restrict__ scale,
                                       const __nv_bfloat16* __restrict__ other,
                                       __nv_bfloat16* __restrict__ out, float* __restrict__ dot,
                                       int64_t tokens, int k, int d, int world, int capacity,
                                       int* status) {
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
      float oth[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (other != nullptr) {
        const bf16x8 o = reinterpret_cast<const bf16x8*>(other + t * (int64_t)d)[v];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(o.v[i]);
          oth[2 * i] = f.x;
          oth[2 * i + 1] = f.y;
        }
      }
#pragma unroll
      for (int i = 0; i < kMaxTopK; ++i) {
        if (i >= k) break;
        const int64_t j = t * k + i;
        const int row = dest_row[j];
        if (row < 0) continue;
        if (row >= capacity || dest_rank[j] < 0 || dest_rank[j] >= world) {
          if (v == lane && lane == 0) report_status(status, kBadArgument);  // skip, do not read
          continue;
        }
        const bf16x8 r = reinterpret_cast<const bf16x8*>(
            static_cast<const __nv_bfloat16*>(buffers.ptr[dest_rank[j]]) + (int64_t)row * d)[v];
        const float s = scale != nullptr ? scale[j] : 1.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float2 f = __bfloat1622float2(r.v[c]);
          acc[2 * c] += s * f.x;
          acc[2 * c + 1] += s * f.y;
          dots[i] += f.x * oth[2 * c] + f.y * oth[2 * c + 1];
        }
      }
      if (out != nullptr) {
        bf16x8 packed;
#pragma unroll
        for (int c = 0; c < 4; ++c) packed.v[c] = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
        reinterpret_cast<bf16x8*>(out + t * (int64_t)d)[v] = packed;
      }
    }
    if (dot != nullptr) {
#pragma unroll
      for (int i = 0; i < kMaxTopK; ++i) {
        if (i >= k) break;
        const float total = warp_sum(dots[i]);
        if (lane == 0) dot[t * k + i] = total;
      }
    }
  }
}

PtrTable make_table(const int64_t* bases, int world) {
  PtrTable table;
  for (int r = 0; r < kMaxEP; ++r) table.ptr[r] = r < world ? reinterpret_cast<void*>(bases[r]) : nullptr;
  return table;
}

}  // namespace

void ep_publish_counts(const int64_t* tables, const int* counts, int experts, int rank, int world,
                       cudaStream_t stream) {
  OB_CHECK(world >= 1 && world <= kMaxEP && experts % world == 0, "bad expert-parallel layout");
  ep_publish_counts_kernel<<<1, 256, 0, stream>>>(make_table(tables, world), counts, experts, rank, world);
  OB_LAUNCH_CHECK();
}

void ep_plan(const int* table, const int* indices, int experts, int world, int rank, int tile,
             int num_tiles, int capacity_rows, int64_t pairs, int* pair_base, int* k_offsets,
             int* tile_expert, int* fill_begin, int* fill_end, int* cursor, int* rows_used,
             int* dest_rank, int* dest_row, cudaStream_t stream) {
  const int local = experts / world;
  ep_plan_kernel<<<1, 256, local * sizeof(int), stream>>>(table, experts, world, rank, tile, num_tiles,
                                                          capacity_rows, pair_base, k_offsets, tile_expert,
                                                          fill_begin, fill_end, cursor, rows_used);
  OB_LAUNCH_CHECK();
  if (pairs == 0) return;
  const int blocks = (int)std::min<int64_t>((pairs + 255) / 256, device_sm_count() * 8);
  ep_place_kernel<<<blocks, 256, 0, stream>>>(indices, pair_base, cursor, dest_rank, dest_row, pairs,
                                              local, capacity_rows);
  OB_LAUNCH_CHECK();
}

void ep_zero_fill(const int* fill_begin, const int* fill_end, void* buffer, int local_experts, int d,
                  int capacity_rows, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "row width must be a multiple of 8");
  const dim3 grid(4, std::min(local_experts, 1024));
  ep_zero_fill_kernel<<<grid, 256, 0, stream>>>(fill_begin, fill_end, static_cast<__nv_bfloat16*>(buffer),
                                                local_experts, d, capacity_rows);
  OB_LAUNCH_CHECK();
}

void ep_push_rows(const void* src, const int* dest_rank, const int* dest_row, const float* scale,
                  const int64_t* buffers, int world, int64_t pairs, int k, int d, int capacity,
                  cudaStream_t stream) {
  OB_CHECK(d % 8 == 0 && world <= kMaxEP && k >= 1 && k <= 32 && pairs % k == 0,
           "bad push arguments");
  if (pairs == 0) return;
  const int64_t tokens = pairs / k;
  const int blocks = (int)std::min<int64_t>((tokens + 7) / 8, device_sm_count() * 16);
  const auto* in = static_cast<const __nv_bfloat16*>(src);
  const PtrTable table = make_table(buffers, world);
  const int vpl = (d % 256 == 0 && d <= 1024) ? d / 256 : 0;
  switch (vpl) {
    case 1: ep_push_rows_kernel<1><<<blocks, 256, 0, stream>>>(in, dest_rank, dest_row, scale, table, pairs, k, d, world, capacity, status_ptr()); break;
    case 2: ep_push_rows_kernel<2><<<blocks, 256, 0, stream>>>(in, dest_rank, dest_row, scale, table, pairs, k, d, world, capacity, status_ptr()); break;
    case 3: ep_push_rows_kernel<3><<<blocks, 256, 0, stream>>>(in, dest_rank, dest_row, scale, table, pairs, k, d, world, capacity, status_ptr()); break;
    case 4: ep_push_rows_kernel<4><<<blocks, 256, 0, stream>>>(in, dest_rank, dest_row, scale, table, pairs, k, d, world, capacity, status_ptr()); break;
    default: ep_push_rows_kernel<0><<<blocks, 256, 0, stream>>>(in, dest_rank, dest_row, scale, table, pairs, k, d, world, capacity, status_ptr()); break;
  }
  OB_LAUNCH_CHECK();
}

void ep_pull_combine(const int64_t* buffers, int world, const int* dest_rank, const int* dest_row,
                     const float* scale, const void* other, void* out, float* dot, int64_t tokens,
                     int k, int d, int capacity, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0 && world <= kMaxEP && k >= 1 && k <= kMaxTopK, "bad combine arguments");
  if (tokens == 0) return;
  const int blocks = (int)std::min<int64_t>((tokens + 7) / 8, device_sm_count() * 16);
  ep_pull_combine_kernel<<<blocks, 256, 0, stream>>>(
      make_table(buffers, world), dest_rank, dest_row, scale, static_cast<const __nv_bfloat16*>(other),
      static_cast<__nv_bfloat16*>(out), dot, tokens, k, d, world, capacity, status_ptr());
  OB_LAUNCH_CHECK();
}

}  // namespace ob
