// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma
// with fp32 accumulators in TMEM (double buffered, so the epilogue of tile i overlaps the main loop
// of tile i+1), epilogue TMEM -> registers -> swizzled smem -> TMA store (or TMA reduce-add for
// split-K / gradient accumulation).
//
//   C[b] (M x N, row major) = alpha * A[b] (M x K) * B[b] (N x K)^T
//
// Each operand may be stored K-major (rows indexed by M/N, K contiguous) or MN-major (rows indexed
// by K, M/N contiguous); together these cover the NT / NN / TN products of a linear layer's forward,
// input-gradient and weight-gradient without materialising a transpose.
//
// Optional ragged modes for mixture-of-experts:
//   * m_tile_batch : per 128-row tile of A/C, which batch of B to use (grouped forward / dgrad;
//                    A and C are plain 2-D matrices whose row groups are padded to 128).
//   * k_offsets    : per output batch, the [begin, end) range of the shared K (token) dimension
//                    (grouped weight gradient; A and B are plain 2-D matrices).
//
// Optional fused collectives over NVLink peer memory (tensor / sequence parallel layers):
//   * gather-A (comm_mode 1): the rows of A are sharded over `world` ranks; the producer reads row
//     block r through a tensor map over rank r's buffer (a plain, non-multicast TMA load of peer
//     memory) after that rank's ready flag has reached `epoch`. This is all-gather -> GEMM in one
//     kernel: local rows are multiplied while remote rows are still arriving.
//   * push-C (comm_mode 2): the row block of C that rank r owns is stored straight into rank r's
//     receive slot for this rank (plain 16-byte peer stores from the epilogue registers); a small
//     reduction kernel on the owner sums the slots. This is GEMM -> reduce-scatter with the
//     transfer of tile i overlapping the math of tile i+1.
//   `rotate` shifts the order of the M tiles so that ranks start on different peers.
//
// Warp roles: four epilogue warps (TMEM lane quarter = warp index; eight in the PAIR variant, the
// second four draining the upper half of the columns), then the TMA producer warp, then the MMA
// issuer + TMEM allocator warp (192 threads, 320 in the PAIR variant).
//
// PAIR variant (plain and batched GEMMs with N > 128): two CTAs of a cluster share one 256 x 256
// output tile. Each loads its own 128 rows of A and one half (128 rows) of B per k-block, the
// leader CTA issues `tcgen05.mma.cta_group::2` (M = 256) which reads both CTAs' shared memory and
// writes 128 accumulator rows into each CTA's TMEM, and each CTA runs the epilogue of its rows.
// Per SM and k-block this moves 32 KB of operands instead of 48 KB: the single-CTA kernel is
// bound by operand delivery (L2 -> shared memory -> tensor core), not by the tensor pipe. The
// loads carry no cluster multicast; the pair is coupled only through mbarriers (the leader's
// "full" barrier counts the bytes of both producers, its commits arrive on both CTAs' "empty"
// and "accumulator ready" barriers, both epilogues arrive on the leader's "accumulator free").
#include "api.h"
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
// Epilogue warps: four cover the 128 TMEM lanes of a CTA (a warp reads lane quarter warp % 4);
// the CTA-pair kernel runs eight, the second four taking the upper half of the tile's columns, so
// that the drain of an accumulator takes half as long (at K = 768 the drain, not the main loop,
// bounded the tile rate with four).
template <bool WIDE>
struct Roles {
  static constexpr int kEpilogueWarps = WIDE ? 8 : 4;
  static constexpr int kProducerWarp = kEpilogueWarps;
  static constexpr int kMmaWarp = kEpilogueWarps + 1;
  static constexpr int kThreads = (kEpilogueWarps + 2) * 32;
};

struct GemmParams {
  int M, N, K;
  int batches;
  int a_mn, b_mn;
  int a_batched, b_batched;
  int splits;
  int reduce;
  float alpha;
  const int* m_tile_batch;
  int m_tile_rows;  // rows of A / C covered by one m_tile_batch entry (a multiple of the tile)
  const int* k_offsets;
  int* status;
  // Optional residual: C = alpha * A*B + beta * R, R bf16 with the geometry of C.
  const __nv_bfloat16* R;
  long long ldr;
  long long strideR;
  float beta;
  // Fused collective (see the header comment). comm_mode 0 = none.
  int comm_mode;
  int world, rank, rows_per_rank, rotate;
  unsigned int epoch;
  unsigned long long limit_ns;
  const CUtensorMap* a_maps;      // gather-A: `world` tensor maps in global memory
  const unsigned int* ready;      // gather-A: this rank's flag slots, one per source rank
  __nv_bfloat16* c_peer[8];       // push-C: destination of row block r (already offset to my slot)
  long long c_peer_ld;            // push-C: row pitch of the receive slots, in elements
};

__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* addr) {
  unsigned int value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(addr) : "memory");
  return value;
}

// Bounded wait until `*flag` has reached `epoch` (wrap-safe). On expiry the CTA is told to unwind
// and the status word records kTimeoutPeerFlag.
__device__ __forceinline__ bool wait_peer_flag(const unsigned int* flag, unsigned int epoch,
                                               unsigned long long limit_ns, const WaitCtx& ctx) {
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (static_cast<int>(ld_acquire_sys_u32(flag) - epoch) < 0) {
    if ((++spins & 0x3f) == 0) {
      if (*ctx.abort) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *ctx.abort = 1;
        report_status(ctx.status, kTimeoutPeerFlag);
        return false;
      }
    }
  }
  // Data published by the peer was written through the generic proxy; TMA reads it through the
  // async proxy.
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}

template <int BN, bool PAIR = false, bool WIDE = false>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;  // rows of B this CTA loads per k-block
  static constexpr int kBBytes = kBRows * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = Roles<WIDE>::kEpilogueWarps * 2 /*buffers*/ * 4096;
  static constexpr int kStages = PAIR ? (WIDE ? 5 : 6) : ((BN == 256) ? 4 : 6);
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

// beta * R[row, col0 .. col0+N) as floats (zeros when there is no residual or out of range).
template <int N>
__device__ __forceinline__ void load_residual(const GemmParams& p, int batch, int row, int col0,
                                              float (&out)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = 0.f;
  if (p.R == nullptr || row >= p.M) return;
  const __nv_bfloat16* src = p.R + (long long)batch * p.strideR + (long long)row * p.ldr + col0;
  if (col0 + N <= p.N && ((p.ldr & 7) == 0)) {
#pragma unroll
    for (int j = 0; j < N / 8; ++j) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + 8 * j);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h2[q]);
        out[8 * j + 2 * q] = f.x * p.beta;
        out[8 * j + 2 * q + 1] = f.y * p.beta;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (col0 + i < p.N) out[i] = __bfloat162float(src[i]) * p.beta;
  }
}

template <int BN, bool OUT_F32, bool PAIR, bool WIDE = false>
__global__ void __launch_bounds__(Roles<WIDE>::kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using L = SmemLayout<BN, PAIR, WIDE>;
  using R = Roles<WIDE>;
  constexpr int TM = PAIR ? 2 * BM : BM;  // rows of C per tile (per CTA pair when PAIR)
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + kStages * L::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + L::kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const WaitCtx wctx{abort_flag, p.status};
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles = (p.M + TM - 1) / TM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int tiles_per_batch = m_tiles * n_tiles * p.splits;
  const int total_tiles = tiles_per_batch * p.batches;
  // Tiles are dealt to CTAs (or CTA pairs) round robin.
  const uint32_t cta_rank = PAIR ? cluster_cta_rank() : 0u;
  const int first_tile = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    // epilogue warps (of both CTAs when PAIR)
    mbar_init(&tmem_empty[0], PAIR ? 2 * R::kEpilogueWarps : R::kEpilogueWarps);
    mbar_init(&tmem_empty[1], PAIR ? 2 * R::kEpilogueWarps : R::kEpilogueWarps);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == R::kProducerWarp && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  if (warp == R::kMmaWarp) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, 2 * BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 2 * BN);
      tmem_relinquish();
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  // Nothing may touch the peer's barriers before the peer has initialised them.
  if constexpr (PAIR) cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Decode a linear tile index. n fastest so CTAs running together share A rows through L2.
  auto decode = [&](int tile, int& batch, int& mt, int& nt, int& kb_begin, int& kb_count,
                    int& k_elem_begin) {
    batch = tile / tiles_per_batch;
    int r = tile - batch * tiles_per_batch;
    int split = r / (m_tiles * n_tiles);
    r -= split * (m_tiles * n_tiles);
    mt = r / n_tiles;
    nt = r - mt * n_tiles;
    if (p.rotate != 0) mt = (mt + p.rotate) % m_tiles;
    int k_lo = 0, k_hi = p.K;
    if (p.k_offsets != nullptr) {
      k_lo = p.k_offsets[batch];
      k_hi = p.k_offsets[batch + 1];
    }
    int kb_total = (k_hi - k_lo + BK - 1) / BK;
    int per = (kb_total + p.splits - 1) / p.splits;
    kb_begin = split * per;
    int kb_end = min(kb_begin + per, kb_total);
    kb_count = max(kb_end - kb_begin, 0);
    k_elem_begin = k_lo;
  };

  if (warp == R::kProducerWarp) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int ready_src = -1;  // source rank whose rows are known to have arrived
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
        int batch, mt, nt, kb_begin, kb_count, k0;
        decode(tile, batch, mt, nt, kb_begin, kb_count, k0);
        int b_batch = batch;
        if (p.m_tile_batch != nullptr) {
          b_batch = p.m_tile_batch[(mt * TM) / p.m_tile_rows];
          if (b_batch < 0) continue;  // padding tile: nothing to compute
        }
        const int za = p.a_batched ? batch : 0;
        const int zb = p.b_batched ? b_batch : 0;
        const CUtensorMap* mapA = &tmA;
        int a_row = mt * TM + (int)cta_rank * BM;
        const int b_row = nt * BN + (int)cta_rank * L::kBRows;
        if (p.comm_mode == 1) {
          const int src = a_row / p.rows_per_rank;
          if (src != ready_src) {
            if (src != p.rank && !wait_peer_flag(p.ready + src, p.epoch, p.limit_ns, wctx)) {
              ok = false;
              break;
            }
            ready_src = src;
          }
          mapA = p.a_maps + src;
          a_row -= src * p.rows_per_rank;
        }
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], phase ^ 1, wctx, kTimeoutEmptyBarrier)) {
            ok = false;
            break;
          }
          uint8_t* sa = stage_base + s * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          const int k = k0 + (kb_begin + kb) * BK;
          if constexpr (PAIR) {
            // The leader's barrier collects the bytes of both CTAs' loads.
            const uint32_t full_addr = map_to_cta(smem_u32(&full_bar[s]), 0);
            if (cta_rank == 0) mbar_expect_tx(&full_bar[s], 2 * L::kStageBytes);
            if (p.a_mn) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_3d_pair(sa + j * (BK * 128), &tmA, full_addr, a_row + j * 64, k, za);
            } else {
              tma_load_3d_pair(sa, &tmA, full_addr, k, a_row, za);
            }
            if (p.b_mn) {
#pragma unroll
              for (int j = 0; j < L::kBRows / 64; ++j)
                tma_load_3d_pair(sb + j * (BK * 128), &tmB, full_addr, b_row + j * 64, k, zb);
            } else {
              tma_load_3d_pair(sb, &tmB, full_addr, k, b_row, zb);
            }
            continue;
          }
          mbar_expect_tx(&full_bar[s], L::kStageBytes);
          if (p.a_mn) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sa + j * (BK * 128), &tmA, &full_bar[s], mt * BM + j * 64, k, za);
          } else {
            tma_load_3d(sa, mapA, &full_bar[s], k, a_row, za);
          }
          if (p.b_mn) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (BK * 128), &tmB, &full_bar[s], nt * BN + j * 64, k, zb);
          } else {
            tma_load_3d(sb, &tmB, &full_bar[s], k, nt * BN, zb);
          }
        }
      }
    }
  } else if (warp == R::kMmaWarp) {
    // ------------------------------- MMA issuer ----------------------------------------------
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc = make_idesc_bf16(TM, BN, p.a_mn != 0, p.b_mn != 0);
      // Descriptors of the operands in stage 0; stepping through k and stages only adds offsets.
      const SmemDesc desc_a = make_smem_desc_parts(smem_u32(stage_base), p.a_mn ? BK * 128 : 16, 1024);
      const SmemDesc desc_b = make_smem_desc_parts(smem_u32(stage_base + L::kABytes),
                                                   p.b_mn ? BK * 128 : 16, 1024);
      const uint32_t step_a = p.a_mn ? 2048 : 32;
      const uint32_t step_b = p.b_mn ? 2048 : 32;
      // This CTA's first non-padding tile at or after `tile`, and its number of k-blocks.
      auto next_tile = [&](int tile, int& kb_count) -> int {
        for (; tile < total_tiles; tile += tile_step) {
          int batch, mt, nt, kb_begin, k0;
          decode(tile, batch, mt, nt, kb_begin, kb_count, k0);
          if (p.m_tile_batch == nullptr || p.m_tile_batch[(mt * TM) / p.m_tile_rows] >= 0)
            return tile;
        }
        return total_tiles;
      };
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      int kb_count = 0;
      int tile = next_tile(first_tile, kb_count);
      while (tile < total_tiles && ok) {
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_phase = (tile_iter >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, wctx, kTimeoutTmemEmpty)) break;
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * BN;
        int next = -1, next_kb = 0;
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          if (!mbar_wait(&full_bar[s], phase, wctx, kTimeoutFullBarrier)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t stage_off = s * L::kStageBytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = smem_desc_at(desc_a, stage_off + k * step_a);
            const uint64_t db = smem_desc_at(desc_b, stage_off + k * step_b);
            if constexpr (PAIR)
              umma_bf16_ss_pair(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else
              umma_bf16_ss(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // Frees the stage (in both CTAs when PAIR) once these MMAs have read it.
          if constexpr (PAIR) {
            const uint32_t addr = smem_u32(&empty_bar[s]);
            tcgen05_commit_pair(map_to_cta(addr, 0));
            tcgen05_commit_pair(map_to_cta(addr, 1));
          } else {
            tcgen05_commit(&empty_bar[s]);
          }
          // Work out the next tile while the tensor pipe is busy with this one, so that the
          // integer divisions of the tile decode stay off the tile-to-tile critical path.
          if (kb == 0) next = next_tile(tile + tile_step, next_kb);
        }
        if (!ok) break;
        if constexpr (PAIR) {
          const uint32_t addr = smem_u32(&tmem_full[acc]);
          tcgen05_commit_pair(map_to_cta(addr, 0));
          tcgen05_commit_pair(map_to_cta(addr, 1));
        } else {
          tcgen05_commit(&tmem_full[acc]);
        }
        if (next < 0) next = next_tile(tile + tile_step, next_kb);
        ++tile_iter;
        tile = next;
        kb_count = next_kb;
      }
    }
  } else {
    // ------------------------------- Epilogue (warps 0 .. kEpilogueWarps-1) -------------------
    // Warp w drains TMEM lanes 32 * (w % 4) .. + 31 (rows of the tile) of the column range of its
    // group of four warps. Chunks of 128 bytes per row go TMEM -> registers -> swizzled staging
    // buffer -> TMA store; the TMEM load of chunk i+1 is issued before chunk i is written out, so
    // its latency hides behind the shared-memory stores and the TMA issue of chunk i.
    const int quarter = warp & 3;
    const int group = warp >> 2;
    constexpr int kGroups = R::kEpilogueWarps / 4;
    constexpr int kGroupCols = BN / kGroups;
    uint8_t* my_staging = staging + warp * 2 * 4096;
    uint32_t tile_iter = 0;
    uint32_t store_iter = 0;
    constexpr int kColsPerStore = OUT_F32 ? 32 : 64;
    const bool has_residual = p.R != nullptr;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step) {
      int batch, mt, nt, kb_begin, kb_count, k0;
      decode(tile, batch, mt, nt, kb_begin, kb_count, k0);
      if (p.m_tile_batch != nullptr && p.m_tile_batch[(mt * TM) / p.m_tile_rows] < 0) continue;
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_phase = (tile_iter >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, wctx, kTimeoutTmemFull)) break;
      tcgen05_fence_after();
      const bool skip_store = (kb_count == 0) && p.reduce;
      const bool have_acc = kb_count > 0;
      const uint32_t taddr_row =
          tmem_base + acc * BN + group * kGroupCols + (static_cast<uint32_t>(quarter * 32) << 16);
      const int row0 = mt * TM + (int)cta_rank * BM + quarter * 32;
      const int col_base = nt * BN + group * kGroupCols;
      // columns of this group that exist (uniform across the warp)
      const int cols_here = min(kGroupCols, p.N - col_base);
      const int chunks = cols_here > 0 ? (cols_here + kColsPerStore - 1) / kColsPerStore : 0;
      // Units of 32 columns: one TMEM load each; a 128-byte row segment of the output is one unit
      // of fp32 or two units of bf16.
      constexpr int kUnitsPerStore = OUT_F32 ? 1 : 2;
      constexpr int kWordsPerUnit = OUT_F32 ? 32 : 16;
      const int units = chunks * kUnitsPerStore;
      uint32_t v[32];
      if (units > 0 && have_acc) tmem_ld_32x32(taddr_row, v);
      bool released = false;
      uint8_t* buf = nullptr;
#pragma unroll 1
      for (int unit = 0; unit < units; ++unit) {
        const int c0 = unit * 32;
        const int col0 = col_base + c0;
        uint32_t packed[kWordsPerUnit];
        if (have_acc) {
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if constexpr (OUT_F32) {
          if (has_residual) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float res[8];
              load_residual<8>(p, batch, row0 + lane, col0 + 8 * j, res);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                packed[8 * j + i] =
                    __float_as_uint(__uint_as_float(v[8 * j + i]) * p.alpha + res[i]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              packed[i] = __float_as_uint(__uint_as_float(v[i]) * p.alpha);
          }
        } else {
          if (has_residual) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float res[8];
              load_residual<8>(p, batch, row0 + lane, col0 + 8 * j, res);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                packed[4 * j + i] =
                    pack_bf16(__uint_as_float(v[8 * j + 2 * i]) * p.alpha + res[2 * i],
                              __uint_as_float(v[8 * j + 2 * i + 1]) * p.alpha + res[2 * i + 1]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              packed[i] = pack_bf16(__uint_as_float(v[2 * i]) * p.alpha,
                                    __uint_as_float(v[2 * i + 1]) * p.alpha);
          }
        }
        // The values of this unit now live in `packed`: start the next unit's TMEM load, or,
        // after the last one, hand the accumulator back before the stores are even issued.
        if (unit + 1 < units) {
          if (have_acc) tmem_ld_32x32(taddr_row + c0 + 32, v);
        } else {
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR)
              mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));  // the leader's barrier
            else
              mbar_arrive(&tmem_empty[acc]);
          }
          released = true;
        }
        const int part = unit % kUnitsPerStore;  // which part of the 128-byte row segment
        if (part == 0) {
          buf = my_staging + (store_iter & 1) * 4096;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
        }
        uint8_t* my_row = buf + lane * 128;
        constexpr int kVecsPerUnit = kWordsPerUnit / 4;  // 16-byte pieces of this unit
#pragma unroll
        for (int j = 0; j < kVecsPerUnit; ++j) {
          const uint4 o = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2],
                                     packed[4 * j + 3]);
          const int piece = part * kVecsPerUnit + j;
          *reinterpret_cast<uint4*>(my_row + ((piece ^ (lane & 7)) << 4)) = o;
        }
        if (part + 1 < kUnitsPerStore && unit + 1 < units) continue;  // segment not complete yet
        const int seg_col0 = col0 - part * 32;  // first column of the 128-byte segment
        if (p.comm_mode == 2) {
          // Row block `owner` of C goes to that rank's receive slot. The 32 x 128-byte chunk is
          // read back from the staging buffer so that eight lanes store one whole 128-byte row
          // segment: full-line writes over NVLink instead of 16-byte fragments.
          __syncwarp();
          const int owner = row0 / p.rows_per_rank;
          __nv_bfloat16* slot = p.c_peer[owner] + (long long)(row0 - owner * p.rows_per_rank) * p.c_peer_ld;
          const int sub = lane & 7;
          const int col = seg_col0 + sub * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = (lane >> 3) + 4 * i;
            const uint4 w = *reinterpret_cast<const uint4*>(buf + r * 128 + ((sub ^ (r & 7)) << 4));
            if (row0 + r < p.M && col < p.N)
              *reinterpret_cast<uint4*>(slot + (long long)r * p.c_peer_ld + col) = w;
          }
          __syncwarp();
          ++store_iter;
          continue;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && !skip_store && row0 < p.M) {
          if (p.reduce)
            tma_reduce_add_3d(&tmC, buf, seg_col0, row0, batch);
          else
            tma_store_3d(&tmC, buf, seg_col0, row0, batch);
          tma_store_commit();
        }
        ++store_iter;
      }
      if (!released) {
        // no column of this group exists in this tile: nothing was read, release at once
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR)
            mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
          else
            mbar_arrive(&tmem_empty[acc]);
        }
      }
      ++tile_iter;
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ------------------------------- Teardown ---------------------------------------------------
  if (*abort_flag) {
    // Give copies that are still in flight time to land before shared memory is released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  // A CTA of a pair must outlive every access of its peer to its shared memory and barriers.
  if constexpr (PAIR) cluster_sync_all();
  if (warp == R::kMmaWarp) {
    tcgen05_fence_after();
    if constexpr (PAIR)
      tmem_dealloc_pair(tmem_base, 2 * BN);
    else
      tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, bool OUT_F32>
void launch_variant(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC,
                    const GemmParams& p, int grid, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  auto kernel = gemm_bf16_kernel<BN, OUT_F32, false>;
  ensure_dynamic_smem((const void*)kernel, L::kTotal);
  kernel<<<grid, Roles<false>::kThreads, L::kTotal, stream>>>(tA, tB, tC, p);
  OB_LAUNCH_CHECK();
}

// CTA-pair variant: clusters of two, at most `max_pairs` of them (0 = ask the driver how many can
// be resident, once per kernel).
template <bool OUT_F32, bool WIDE>
void launch_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC,
                 const GemmParams& p, long long total_tiles, int num_sms, cudaStream_t stream) {
  using L = SmemLayout<256, true, WIDE>;
  auto kernel = gemm_bf16_kernel<256, OUT_F32, true, WIDE>;
  static int resident_by_device[64] = {0};
  int dev = 0;
  OB_CUDA_CHECK(cudaGetDevice(&dev));
  int& resident_pairs = resident_by_device[dev & 63];
  ensure_dynamic_smem((const void*)kernel, L::kTotal);
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.blockDim = dim3(Roles<WIDE>::kThreads, 1, 1);
  config.dynamicSmemBytes = L::kTotal;
  config.stream = stream;
  config.attrs = attr;
  config.numAttrs = 1;
  if (resident_pairs == 0) {
    config.gridDim = dim3(2 * (num_sms / 2), 1, 1);
    int clusters = 0;
    OB_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&clusters, kernel, &config));
    resident_pairs = std::max(1, std::min(clusters, num_sms / 2));
  }
  const int pairs = (int)std::min<long long>(total_tiles, std::min(resident_pairs, num_sms / 2));
  config.gridDim = dim3(2 * pairs, 1, 1);
  OB_CUDA_CHECK(cudaLaunchKernelEx(&config, kernel, tA, tB, tC, p));
  count_launch();
}

// The pair kernel serves plain, batched and ragged (mixture-of-experts) products whose output is
// wide enough for a 256-column tile; the fused-collective modes stay on the single-CTA kernel.
bool pair_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("OHARA_GEMM_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  return enabled;
}

// Eight epilogue warps per CTA of a pair (the second four drain the upper column half) or four.
// Measured on one B200: equal within noise on the large training GEMMs, 17 % faster on the batched
// 768^3 Newton-Schulz products (few tiles per CTA: the drain of the last tile is exposed), 3 %
// slower on the ragged expert GEMMs (one pipeline stage fewer fits next to the wider staging
// buffer). Default: wide for plain / batched products, narrow for ragged ones;
// OHARA_GEMM_WIDE_EPILOGUE=0/1 forces one of them for A/B measurements.
bool wide_epilogue(const GemmParams& p) {
  static const int forced = [] {
    const char* e = std::getenv("OHARA_GEMM_WIDE_EPILOGUE");
    return e == nullptr ? -1 : (e[0] != '0' ? 1 : 0);
  }();
  if (forced >= 0) return forced == 1;
  return p.m_tile_batch == nullptr && p.k_offsets == nullptr;
}

}  // namespace

// Host entry point. Pointers are device pointers; `ld*` are row pitches in elements of the stored
// matrices; `stride*` are elements between consecutive batches (ignored when not batched).
void gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int batches, bool a_mn,
               bool b_mn, int64_t lda, int64_t ldb, int64_t ldc, int64_t strideA, int64_t strideB,
               int64_t strideC, bool a_batched, bool b_batched, int b_batches, bool out_f32,
               int splits, bool reduce, float alpha, const int* m_tile_batch,
               const int* k_offsets, int64_t a_rows, int64_t b_rows, int num_sms,
               const void* R, int64_t ldr, int64_t strideR, float beta, cudaStream_t stream,
               int m_tile_rows) {
  gemm_bf16_comm(A, B, C, M, N, K, batches, a_mn, b_mn, lda, ldb, ldc, strideA, strideB, strideC,
                 a_batched, b_batched, b_batches, out_f32, splits, reduce, alpha, m_tile_batch,
                 k_offsets, a_rows, b_rows, num_sms, R, ldr, strideR, beta, nullptr, stream,
                 m_tile_rows);
}

void gemm_bf16_comm(const void* A, const void* B, void* C, int M, int N, int K, int batches,
                    bool a_mn, bool b_mn, int64_t lda, int64_t ldb, int64_t ldc, int64_t strideA,
                    int64_t strideB, int64_t strideC, bool a_batched, bool b_batched, int b_batches,
                    bool out_f32, int splits, bool reduce, float alpha, const int* m_tile_batch,
                    const int* k_offsets, int64_t a_rows, int64_t b_rows, int num_sms,
                    const void* R, int64_t ldr, int64_t strideR, float beta, const GemmComm* comm,
                    cudaStream_t stream, int m_tile_rows) {
  OB_CHECK(M > 0 && N > 0 && K >= 0 && batches > 0, "gemm_bf16: bad problem size");
  OB_CHECK(m_tile_rows >= BM && m_tile_rows % BM == 0, "gemm_bf16: m_tile_rows must be a multiple of 128");
  OB_CHECK(!reduce || out_f32, "gemm_bf16: reduce-add epilogue needs an fp32 output");
  OB_CHECK(splits >= 1 && (splits == 1 || reduce), "gemm_bf16: split-K needs the reduce epilogue");
  const int BN = (N > 128) ? 256 : 128;
  // Ragged modes qualify when an m_tile_batch entry never covers less than a 256-row pair tile.
  const bool pair = pair_enabled() && BN == 256 && M > 128 &&
                    (m_tile_batch == nullptr || m_tile_rows % (2 * BM) == 0) &&
                    (comm == nullptr || comm->mode == 0);

  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.batches = batches;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  p.a_batched = a_batched;
  p.b_batched = b_batched;
  p.splits = splits;
  p.reduce = reduce;
  p.alpha = alpha;
  p.m_tile_batch = m_tile_batch;
  p.m_tile_rows = m_tile_rows;
  p.k_offsets = k_offsets;
  p.status = status_ptr();
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ldr = ldr;
  p.strideR = strideR;
  p.beta = beta;
  OB_CHECK(R == nullptr || !reduce, "gemm_bf16: a residual cannot be combined with the reduce epilogue");
  p.comm_mode = 0;
  p.world = 1;
  p.rank = 0;
  p.rows_per_rank = M;
  p.rotate = 0;
  p.epoch = 0;
  p.limit_ns = 0;
  p.a_maps = nullptr;
  p.ready = nullptr;
  for (auto& dst : p.c_peer) dst = nullptr;
  p.c_peer_ld = 0;
  if (comm != nullptr && comm->mode != 0) {
    OB_CHECK(comm->world >= 1 && comm->world <= 8 && comm->rank >= 0 && comm->rank < comm->world,
             "fused collective: bad rank / world");
    OB_CHECK(batches == 1 && splits == 1 && !reduce && m_tile_batch == nullptr && k_offsets == nullptr,
             "fused collective: plain 2-D GEMM only");
    OB_CHECK(M % comm->world == 0 && (M / comm->world) % BM == 0,
             "fused collective: rows per rank must be a multiple of 128");
    p.comm_mode = comm->mode;
    p.world = comm->world;
    p.rank = comm->rank;
    p.rows_per_rank = M / comm->world;
    const int tiles_per_rank = p.rows_per_rank / BM;
    p.epoch = comm->epoch;
    p.limit_ns = comm->limit_ns;
    if (comm->mode == 1) {
      OB_CHECK(!a_mn && comm->a_maps != nullptr && comm->ready != nullptr,
               "gather-A needs a K-major A, peer tensor maps and ready flags");
      p.a_maps = static_cast<const CUtensorMap*>(comm->a_maps);
      p.ready = comm->ready;
      p.rotate = comm->rank * tiles_per_rank;  // own rows first: they are already here
    } else {
      OB_CHECK(!out_f32 && N % 8 == 0 && R == nullptr, "push-C needs a bf16 output, N % 8 == 0");
      for (int r = 0; r < comm->world; ++r) {
        OB_CHECK(comm->c_peer[r] != nullptr, "push-C: missing destination");
        p.c_peer[r] = static_cast<__nv_bfloat16*>(comm->c_peer[r]);
      }
      p.c_peer_ld = comm->c_peer_ld;
      p.rotate = ((comm->rank + 1) % comm->world) * tiles_per_rank;  // own rows last
    }
  }

  // Stored shapes: K-major operand is (rows = M or N, inner = K); MN-major is (rows = K, inner =
  // M or N). `a_rows` / `b_rows` give the number of stored rows (the full token count in the
  // ragged weight-gradient mode, where K is per batch).
  CUtensorMap tA, tB, tC;
  const uint64_t a_inner = a_mn ? (uint64_t)M : (uint64_t)K;
  const uint64_t b_inner = b_mn ? (uint64_t)N : (uint64_t)K;
  const int a_nb = a_batched ? batches : 1;
  const int b_nb = b_batched ? b_batches : 1;
  make_tmap_3d(&tA, A, TmapDtype::BF16, a_inner, (uint64_t)a_rows, (uint64_t)a_nb, lda, strideA, 64,
               a_mn ? BK : BM, TmapSwizzle::B128);
  make_tmap_3d(&tB, B, TmapDtype::BF16, b_inner, (uint64_t)b_rows, (uint64_t)b_nb, ldb, strideB, 64,
               b_mn ? BK : (pair ? BN / 2 : BN), TmapSwizzle::B128);
  make_tmap_3d(&tC, C, out_f32 ? TmapDtype::F32 : TmapDtype::BF16, (uint64_t)N, (uint64_t)M,
               (uint64_t)batches, ldc, strideC, out_f32 ? 32 : 64, 32, TmapSwizzle::B128);

  const int tile_m = pair ? 2 * BM : BM;
  const int m_tiles = (M + tile_m - 1) / tile_m;
  const int n_tiles = (N + BN - 1) / BN;
  const long long total = (long long)m_tiles * n_tiles * splits * batches;
  const int grid = (int)std::min<long long>(total, num_sms);
  if (pair) {
    if (out_f32)
      wide_epilogue(p) ? launch_pair<true, true>(tA, tB, tC, p, total, num_sms, stream)
                      : launch_pair<true, false>(tA, tB, tC, p, total, num_sms, stream);
    else
      wide_epilogue(p) ? launch_pair<false, true>(tA, tB, tC, p, total, num_sms, stream)
                      : launch_pair<false, false>(tA, tB, tC, p, total, num_sms, stream);
  } else if (BN == 256) {
    if (out_f32)
      launch_variant<256, true>(tA, tB, tC, p, grid, stream);
    else
      launch_variant<256, false>(tA, tB, tC, p, grid, stream);
  } else {
    if (out_f32)
      launch_variant<128, true>(tA, tB, tC, p, grid, stream);
    else
      launch_variant<128, false>(tA, tB, tC, p, grid, stream);
  }
}

void make_peer_row_maps(const int64_t* bases, int world, int64_t rows, int64_t K, int64_t ld,
                        void* out) {
  CUtensorMap* maps = static_cast<CUtensorMap*>(out);
  for (int r = 0; r < world; ++r)
    make_tmap_3d(&maps[r], reinterpret_cast<const void*>(bases[r]), TmapDtype::BF16, (uint64_t)K,
                 (uint64_t)rows, 1, ld, 0, 64, BM, TmapSwizzle::B128);
}

}  // namespace ob
