// Companions of the GEMM's fused collectives (tensor / sequence parallel layers): publishing a
// ready flag to every peer, summing the receive slots that peers filled from their GEMM epilogues,
// and pulling the peers' staged rows into one local tensor. Waits are bounded; on expiry the kernel
// records kTimeoutPeerFlag in the status word and returns.
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kMaxTP = 8;

struct PadTable {
  unsigned int* ptr[kMaxTP];
};
struct BaseTable {
  const void* ptr[kMaxTP];
};

__device__ __forceinline__ void st_release_sys(unsigned int* addr, unsigned int value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* addr) {
  unsigned int value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(addr) : "memory");
  return value;
}

// Everything this rank wrote earlier on the stream (its staged rows, or its pushes into peers'
// receive slots) becomes visible to a peer that observes the flag.
__global__ void tp_signal_kernel(PadTable pads, int slot_base, int rank, int world,
                                 unsigned int epoch) {
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(pads.ptr[threadIdx.x] + slot_base + rank, epoch);
  }
}

// Every block waits until all `world` flags have reached `epoch`. Returns false on timeout.
__device__ bool wait_all_flags(const unsigned int* flags, int world, unsigned int epoch,
                               unsigned long long limit_ns, int* status) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < world) {
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (static_cast<int>(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
      if ((++spins & 0x3f) == 0 && global_timer_ns() - t0 > limit_ns) {
        failed = 1;
        if (blockIdx.x == 0) report_status(status, kTimeoutPeerFlag);
        break;
      }
    }
  }
  __syncthreads();
  return failed == 0;
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

// out (rows x cols) = sum over s of slots[s] (+ residual); slots is (world, rows, cols) bf16 in
// this rank's receive buffer. fp32 accumulation, bf16 result.
__global__ void __launch_bounds__(512)
tp_reduce_slots_kernel(const __nv_bfloat16* __restrict__ slots, const unsigned int* __restrict__ flags,
                       const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                       int64_t elems, int world, unsigned int epoch, unsigned long long limit_ns,
                       int* status) {
  if (!wait_all_flags(flags, world, epoch, limit_ns, status)) return;
  const int64_t vecs = elems >> 3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs;
       i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < world; ++s) {
      const bf16x8 v = reinterpret_cast<const bf16x8*>(slots + (int64_t)s * elems)[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v.v[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (residual != nullptr) {
      const bf16x8 v = reinterpret_cast<const bf16x8*>(residual)[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v.v[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<bf16x8*>(out)[i] = o;
  }
}

// out[r * bytes_per_rank ...] = bases[r][0 .. bytes_per_rank) for every rank r (16-byte copies,
// starting with the next rank so that the ranks do not all read the same peer at once).
__global__ void __launch_bounds__(512)
tp_gather_rows_kernel(BaseTable bases, const unsigned int* __restrict__ flags, uint4* __restrict__ out,
                      int64_t vecs_per_rank, int rank, int world, unsigned int epoch,
                      unsigned long long limit_ns, int* status) {
  if (!wait_all_flags(flags, world, epoch, limit_ns, status)) return;
  const int64_t total = vecs_per_rank * world;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int hop = (int)(i / vecs_per_rank);
    const int64_t v = i - (int64_t)hop * vecs_per_rank;
    const int src = (rank + 1 + hop) % world;
    out[(int64_t)src * vecs_per_rank + v] = static_cast<const uint4*>(bases.ptr[src])[v];
  }
}

}  // namespace

void tp_signal(const int64_t* flag_pads, int slot_base, int rank, int world, unsigned int epoch,
               cudaStream_t stream) {
  OB_CHECK(world >= 1 && world <= kMaxTP, "tensor-parallel degree above 8");
  PadTable pads;
  for (int r = 0; r < kMaxTP; ++r)
    pads.ptr[r] = r < world ? reinterpret_cast<unsigned int*>(flag_pads[r]) : nullptr;
  tp_signal_kernel<<<1, 32, 0, stream>>>(pads, slot_base, rank, world, epoch);
  OB_LAUNCH_CHECK();
}

void tp_reduce_slots(const void* slots, const unsigned int* flags, const void* residual, void* out,
                     int64_t rows, int64_t cols, int world, unsigned int epoch,
                     unsigned long long limit_ns, cudaStream_t stream) {
  const int64_t elems = rows * cols;
  OB_CHECK(elems % 8 == 0 && world >= 1 && world <= kMaxTP, "reduce: bad shape");
  if (elems == 0) return;
  const int blocks = (int)std::min<int64_t>((elems / 8 + 511) / 512, device_sm_count() * 4);
  tp_reduce_slots_kernel<<<blocks, 512, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(slots), flags, static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(out), elems, world, epoch, limit_ns, status_ptr());
  OB_LAUNCH_CHECK();
}

void tp_gather_rows(const int64_t* bases, const unsigned int* flags, void* out,
                    int64_t bytes_per_rank, int rank, int world, unsigned int epoch,
                    unsigned long long limit_ns, cudaStream_t stream) {
  OB_CHECK(bytes_per_rank % 16 == 0 && world >= 1 && world <= kMaxTP, "gather: bad shape");
  BaseTable table;
  for (int r = 0; r < kMaxTP; ++r)
    table.ptr[r] = r < world ? reinterpret_cast<const void*>(bases[r]) : nullptr;
  const int64_t vecs = bytes_per_rank / 16;
  if (vecs == 0) return;
  const int blocks = (int)std::min<int64_t>((vecs * world + 511) / 512, device_sm_count() * 4);
  tp_gather_rows_kernel<<<blocks, 512, 0, stream>>>(table, flags, static_cast<uint4*>(out), vecs, rank,
                                                    world, epoch, limit_ns, status_ptr());
  OB_LAUNCH_CHECK();
}

}  // namespace ob
