// Peer-memory (NVLink / NVSwitch) runtime: symmetric buffers shared between the GPUs of one node by
// CUDA IPC, a flag-based barrier, and the in-kernel collectives of the sharded optimizer.
//
// Every rank allocates the same buffers with cudaMalloc, exports IPC handles (exchanged by the
// host over the c10d store) and opens its peers' handles, so each kernel receives a table of
// `world` base pointers, one per rank, all addressing the same logical buffer. Collectives are
// plain loads/stores through those pointers:
//   * reduce-scatter : every rank reads its own region from all ranks' gradient buffers, sums in
//                      fp32, scales, and writes the fp32 result locally (bf16 -> fp32 cast fused);
//   * all-gather     : every rank pulls the other ranks' regions of the weight buffer.
// Ordering between ranks uses a signal pad per rank: a barrier writes this rank's epoch into its
// slot of every peer's pad (st.release.sys) and waits until every slot of its own pad has reached
// the epoch (ld.acquire.sys). The wait is bounded; when it runs out the kernel records
// kTimeoutPeerFlag in the status word and returns without touching peer memory.
#include "common.cuh"
#include "host_utils.h"

namespace ob {

constexpr int kMaxPeers = 16;

struct PeerTable {
  void* ptr[kMaxPeers];
};

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(addr) : "memory");
  return value;
}

// Barrier across ranks, executed by every block of the calling kernel. Block 0 publishes the epoch
// to all peers; every block waits on this rank's own pad. Returns false on timeout.
__device__ bool peer_barrier(const PeerTable& pads, int rank, int world, uint32_t epoch,
                             uint64_t limit_ns, int* status) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(pads.ptr[threadIdx.x]) + rank, epoch);
  }
  if (threadIdx.x < world) {
    const uint32_t* mine = static_cast<const uint32_t*>(pads.ptr[rank]) + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
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

__global__ void peer_barrier_kernel(PeerTable pads, int rank, int world, uint32_t epoch,
                                    uint64_t limit_ns, int* status) {
  peer_barrier(pads, rank, world, epoch, limit_ns, status);
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

// out[i] = scale * sum_r grads[r][rank * region + i], i in [0, region); bf16 in, fp32 out.
__global__ void __launch_bounds__(512)
reduce_scatter_mean_kernel(PeerTable grads, PeerTable pads, float* __restrict__ out, int64_t region,
                           int rank, int world, float scale, uint32_t epoch, uint64_t limit_ns,
                           int* status) {
  if (!peer_barrier(pads, rank, world, epoch, limit_ns, status)) return;
  const int64_t vecs = region >> 3;
  const int64_t base = (int64_t)rank * region;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs;
       i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
    for (int r = 0; r < world; ++r) {
      // Start with the next rank so that the ranks do not all hit the same peer at once.
      const int src = (rank + 1 + r) % world;
      const bf16x8 v =
          reinterpret_cast<const bf16x8*>(static_cast<const __nv_bfloat16*>(grads.ptr[src]) + base)[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v.v[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    float4* dst = reinterpret_cast<float4*>(out) + 2 * i;
    dst[0] = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
    dst[1] = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
  }
}

// local[r * region ...] = weights[r][r * region ...] for every r != rank (16-byte copies).
__global__ void __launch_bounds__(512)
all_gather_kernel(PeerTable weights, PeerTable pads, int64_t region_bytes, int rank, int world,
                  uint32_t epoch, uint64_t limit_ns, int* status) {
  if (!peer_barrier(pads, rank, world, epoch, limit_ns, status)) return;
  const int64_t vecs = region_bytes >> 4;
  const int64_t total = vecs * (world - 1);
  uint4* local = static_cast<uint4*>(weights.ptr[rank]);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int hop = (int)(i / vecs);
    const int64_t v = i - (int64_t)hop * vecs;
    const int src = (rank + 1 + hop) % world;
    const uint4* remote = static_cast<const uint4*>(weights.ptr[src]);
    local[(int64_t)src * vecs + v] = remote[(int64_t)src * vecs + v];
  }
}

// One-shot all-reduce for small tensors (decode-time tensor parallelism, scalars, norms): every
// rank has written its vector into its copy of a symmetric buffer; after the flag barrier each rank
// reads all `world` copies and sums them in fp32. One NVLink round trip, no ring, no chunking.
template <typename T>
__global__ void __launch_bounds__(512)
all_reduce_oneshot_kernel(PeerTable bufs, PeerTable pads, T* __restrict__ out, int64_t n, int rank,
                          int world, float scale, uint32_t epoch, uint64_t limit_ns, int* status) {
  if (!peer_barrier(pads, rank, world, epoch, limit_ns, status)) return;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    // Same summation order on every rank: the result must be bit-identical across the group
    // (replicated activations, clipping factors and sampled tokens depend on it).
    float acc = 0.f;
    for (int src = 0; src < world; ++src)
      acc += static_cast<float>(static_cast<const T*>(bufs.ptr[src])[i]);
    out[i] = static_cast<T>(acc * scale);
  }
}

// Graph-replayable variant for messages of a few hundred KB at most (decode-time tensor
// parallelism): one block copies the input into this rank's slot, signals, waits for the peers and
// sums all slots. The epoch lives in device memory and advances by one per launch, so a CUDA graph
// that contains the launch can be replayed; every rank must run the same number of launches. The
// two slots alternate by epoch parity: a slot is rewritten two calls after it was read, and a rank
// cannot be more than one call ahead of a peer (it waits for the peer's signal of the current
// call), so the peer has finished reading by then.
template <typename T>
__global__ void __launch_bounds__(1024)
all_reduce_small_kernel(PeerTable bufs, PeerTable pads, uint32_t* __restrict__ counter,
                        const T* __restrict__ in, T* __restrict__ out, int n, int64_t slot_elems,
                        int rank, int world, float scale, uint64_t limit_ns, int* status) {
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) epoch_s = *counter + 1;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const int64_t base = (int64_t)(epoch & 1) * slot_elems;
  T* mine = static_cast<T*>(bufs.ptr[rank]) + base;
  for (int i = threadIdx.x; i < n; i += blockDim.x) mine[i] = in[i];
  __threadfence_system();
  if (peer_barrier(pads, rank, world, epoch, limit_ns, status)) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float acc = 0.f;  // fixed order: bit-identical on every rank
      for (int src = 0; src < world; ++src)
        acc += static_cast<float>((static_cast<const T*>(bufs.ptr[src]) + base)[i]);
      out[i] = static_cast<T>(acc * scale);
    }
  }
  // Advance even after a timed-out wait so that the ranks stay in step once the cause is gone.
  if (threadIdx.x == 0) *counter = epoch;
}

}  // namespace

// ---- host API -------------------------------------------------------------------------------
void* peer_alloc(size_t bytes, char handle_out[64]) {
  void* ptr = nullptr;
  OB_CUDA_CHECK(cudaMalloc(&ptr, bytes));
  OB_CUDA_CHECK(cudaMemset(ptr, 0, bytes));
  cudaIpcMemHandle_t handle;
  OB_CUDA_CHECK(cudaIpcGetMemHandle(&handle, ptr));
  static_assert(sizeof(handle) == 64, "unexpected IPC handle size");
  memcpy(handle_out, &handle, 64);
  return ptr;
}

void* peer_open(const char handle_in[64]) {
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle_in, 64);
  void* ptr = nullptr;
  OB_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess));
  return ptr;
}

void peer_close(void* ptr) { cudaIpcCloseMemHandle(ptr); }
void peer_free(void* ptr) { cudaFree(ptr); }

static PeerTable make_table(const int64_t* ptrs, int world) {
  OB_CHECK(world >= 1 && world <= kMaxPeers, "peer table supports up to 16 ranks");
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return t;
}

void peer_barrier_launch(const int64_t* pads, int rank, int world, uint32_t epoch,
                         uint64_t limit_ns, cudaStream_t stream) {
  peer_barrier_kernel<<<1, 32, 0, stream>>>(make_table(pads, world), rank, world, epoch, limit_ns,
                                            status_ptr());
  OB_LAUNCH_CHECK();
}

void peer_reduce_scatter_mean(const int64_t* grads, const int64_t* pads, float* out, int64_t region,
                              int rank, int world, uint32_t epoch, uint64_t limit_ns,
                              cudaStream_t stream) {
  OB_CHECK(region % 8 == 0, "region must be a multiple of 8 elements");
  const int blocks = device_sm_count() * 2;
  reduce_scatter_mean_kernel<<<blocks, 512, 0, stream>>>(
      make_table(grads, world), make_table(pads, world), out, region, rank, world,
      1.0f / (float)world, epoch, limit_ns, status_ptr());
  OB_LAUNCH_CHECK();
}

void peer_all_gather(const int64_t* weights, const int64_t* pads, int64_t region_bytes, int rank,
                     int world, uint32_t epoch, uint64_t limit_ns, cudaStream_t stream) {
  OB_CHECK(region_bytes % 16 == 0, "region must be a multiple of 16 bytes");
  const int blocks = device_sm_count() * 2;
  all_gather_kernel<<<blocks, 512, 0, stream>>>(make_table(weights, world), make_table(pads, world),
                                                region_bytes, rank, world, epoch, limit_ns,
                                                status_ptr());
  OB_LAUNCH_CHECK();
}

void peer_all_reduce(const int64_t* bufs, const int64_t* pads, void* out, int64_t n, bool bf16,
                     float scale, int rank, int world, uint32_t epoch, uint64_t limit_ns,
                     cudaStream_t stream) {
  if (n == 0) return;
  const int blocks = (int)std::min<int64_t>((n + 511) / 512, device_sm_count() * 2);
  if (bf16)
    all_reduce_oneshot_kernel<__nv_bfloat16><<<blocks, 512, 0, stream>>>(
        make_table(bufs, world), make_table(pads, world), static_cast<__nv_bfloat16*>(out), n, rank,
        world, scale, epoch, limit_ns, status_ptr());
  else
    all_reduce_oneshot_kernel<float><<<blocks, 512, 0, stream>>>(
        make_table(bufs, world), make_table(pads, world), static_cast<float*>(out), n, rank, world,
        scale, epoch, limit_ns, status_ptr());
  OB_LAUNCH_CHECK();
}

void peer_all_reduce_small(const int64_t* bufs, const int64_t* pads, uint32_t* counter,
                           const void* in, void* out, int64_t n, int64_t slot_elems, bool bf16,
                           float scale, int rank, int world, uint64_t limit_ns,
                           cudaStream_t stream) {
  if (n == 0) return;
  OB_CHECK(n <= slot_elems && n < (1ll << 30), "peer_all_reduce_small: message exceeds the slot");
  if (bf16)
    all_reduce_small_kernel<__nv_bfloat16><<<1, 1024, 0, stream>>>(
        make_table(bufs, world), make_table(pads, world), counter,
        static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), (int)n,
        slot_elems, rank, world, scale, limit_ns, status_ptr());
  else
    all_reduce_small_kernel<float><<<1, 1024, 0, stream>>>(
        make_table(bufs, world), make_table(pads, world), counter, static_cast<const float*>(in),
        static_cast<float*>(out), (int)n, slot_elems, rank, world, scale, limit_ns, status_ptr());
  OB_LAUNCH_CHECK();
}

}  // namespace ob
