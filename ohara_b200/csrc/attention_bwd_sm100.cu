// Flash-attention backward for sm_100a (causal or full, grouped-query heads).
//
// One CTA owns one 128-key tile of one (batch, kv-head) and walks over every 64-query tile (of
// every query head in the group) that can see it. All five products run on tcgen05.mma with
// M = 128; the score-shaped ones are computed *transposed* so that a thread (= TMEM lane) owns a
// key row and the per-query statistics (log-sum-exp and delta = rowsum(dO*O)) are plain broadcast
// reads:
//     S^T  = K  Q^T          (128 keys x 64 queries)      dP^T = V dO^T
//     P^T  = exp2(S^T*c - lse),  dS^T = P^T o (dP^T - delta)               (registers)
//     dV  += P^T dO          dK += dS^T Q                 (accumulate in TMEM over all q tiles)
//     dQ^T = K^T dS^T        (head_dim x 64) -> registers -> red.global.add.f32 (fp32 buffer)
// dK and dV are written once at the end (no atomics, GQA groups are summed inside the CTA); dQ is
// accumulated across key tiles in an fp32 buffer: a thread of the drain owns one head_dim index,
// so the 32 lanes of a warp add 128 contiguous bytes of one query row per instruction.
//
// The softmax scale of dS is applied once at the end instead of per element: dK is multiplied in
// the epilogue, and the dQ accumulators hold the unscaled sum (the caller scales while converting).
//
// Warp roles (576 threads): 0-15 softmax / drain / epilogue (four threads per key row: warp w owns
// TMEM lanes 32*(w%4).. and queries 16*(w/4).. of a tile; the element-wise work is bound by
// instruction latency, so it is spread over four warps per scheduler), 16 TMA producer (its lanes
// also stage the per-query statistics of each tile), 17 MMA issuer. The softmax warps never synchronise with one
// another inside the loop: P^T / dS^T are double buffered in shared memory and dQ^T in TMEM, and
// every hand-off is an mbarrier between a warp and the MMA issuer.
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kKeys = 128;
constexpr int kQRows = 64;
constexpr int kQStages = 3;  // (Q, dO) tiles in flight: covers the load latency of two tiles ahead
constexpr int kThreads = 576;  // 16 softmax warps, TMA producer (warp 16), MMA issuer (warp 17)
constexpr int kSoftmaxThreads = 512;
constexpr int kProducerWarp = 16;
constexpr int kMmaWarp = 17;
constexpr int kSliceCols = 16;  // queries of a tile handled by one thread
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  int B, T, S, H, Hk;
  int causal;
  float scale;       // softmax scale
  float scale_log2;  // scale * log2(e)
  const float* lse;    // (B, H, T) natural log
  const float* delta;  // (B, H, T)
  float* dq;           // (B, T, H, D) fp32 accumulators (unscaled), zero-initialised by the caller
  int* status;
};

template <int D>
struct BwdSmem {
  static constexpr int kKVBytes = kKeys * D * 2;   // K or V tile
  static constexpr int kQBytes = kQRows * D * 2;   // Q or dO tile
  static constexpr int kPBytes = kKeys * kQRows * 2;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kKVBytes;
  static constexpr int kQ = kV + kKVBytes;          // kQStages stages of (Q, dO)
  static constexpr int kP = kQ + 2 * kQStages * kQBytes;   // 2 buffers of P^T
  static constexpr int kdS = kP + 2 * kPBytes;             // 2 buffers of dS^T
  static constexpr int kStats = kdS + 2 * kPBytes;  // kQStages x (64 lse*log2e + 64 delta) floats
  static constexpr int kBars = kStats + kQStages * 128 * 4;
  static constexpr int kNeeded = kBars + 256 + 1024;
  static constexpr int kTotal = kNeeded > 120 * 1024 ? kNeeded : 120 * 1024;
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmdK,
                 const __grid_constant__ CUtensorMap tmdV, const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int kDSub = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem + L::kK;
  uint8_t* sV = smem + L::kV;
  uint8_t* sQdO = smem + L::kQ;  // stage s: Q at s*2*kQBytes, dO right after it
  uint8_t* sP = smem + L::kP;
  uint8_t* sdS = smem + L::kdS;
  float* sStats = reinterpret_cast<float*>(smem + L::kStats);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* kv_full = bars;        // 1
  uint64_t* qdo_full = bars + 1;               // kQStages
  uint64_t* qdo_empty = bars + 1 + kQStages;   // kQStages
  uint64_t* s_full = bars + 1 + 2 * kQStages;  // 1
  uint64_t* sd_empty = s_full + 1;   // 1 (one arrival per softmax warp)
  // ps_full and mma_done alternate between two barriers by tile parity. Their waiters have
  // already enabled the *next* completion when they start to wait (the softmax warps arrive on
  // ps_full before they wait for mma_done of the previous tile; the MMA issuer commits the next
  // scores before it waits for ps_full), so a single barrier could complete twice before a
  // delayed waiter looks, and a parity wait cannot tell that from "not yet".
  uint64_t* ps_full = s_full + 2;    // 2 (one arrival per softmax warp)
  uint64_t* mma_done = s_full + 4;   // 2
  uint64_t* grp_bar = s_full + 6;    // 1 (all softmax threads): bounded barrier among them
  uint64_t* stat_full = s_full + 7;  // kQStages (one arrival per lane of the producer warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_full + kQStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Block -> (batch, kv head, key tile) with the key tile fastest: the CTAs that run at the same
  // time then belong to a handful of (batch, head) pairs and share their Q / dO tiles and dQ
  // accumulators through L2 (with the key tile slowest, every resident CTA streamed its own
  // head's tensors and the kernel was bound by HBM). Within a head the low key tiles, which have
  // the most work under a causal mask, come first.
  int bid = blockIdx.x;
  const int k_tiles_total = (p.S + kKeys - 1) / kKeys;
  const int kt = bid % k_tiles_total;
  bid /= k_tiles_total;
  const int hk = bid % p.Hk;
  const int b = bid / p.Hk;
  const int kv0 = kt * kKeys;
  const int group = p.H / p.Hk;
  const int offset = p.S - p.T;
  const int q_tiles = (p.T + kQRows - 1) / kQRows;
  int qt_begin = 0;
  if (p.causal) qt_begin = max(0, kv0 - offset) / kQRows;
  const int tiles_per_head = max(q_tiles - qt_begin, 0);
  const int n_iters = tiles_per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&stat_full[i], 32);
    }
    mbar_init(s_full, 1);
    mbar_init(sd_empty, kSoftmaxThreads / 32);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ps_full[i], kSoftmaxThreads / 32);
      mbar_init(&mma_done[i], 1);
    }
    mbar_init(grp_bar, kSoftmaxThreads);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmdO);
    prefetch_tmap(&tmdK);
    prefetch_tmap(&tmdV);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base;          // 64 columns
  const uint32_t tm_dP = tmem_base + 64;    // 64 columns
  const uint32_t tm_dV = tmem_base + 128;   // D columns
  const uint32_t tm_dK = tmem_base + 256;   // D columns
  // dQ^T (lane = head_dim index) is double buffered by iteration parity, 2 x 64 columns: the MMAs of
  // tile it+1 write one buffer while the softmax warps still drain the other.
  const uint32_t tm_dQ = tmem_base + 384;

  auto iter_coords = [&](int it, int& h, int& tq0) {
    const int g = it / tiles_per_head;
    const int qt = qt_begin + (it - g * tiles_per_head);
    h = hk * group + g;
    tq0 = qt * kQRows;
  };

  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ---------------------------------------------
    // Lane 0 issues the tile loads; all 32 lanes fetch the 64 log-sum-exp and 64 delta values of
    // the tile (four each) into the stage's statistics slot and arrive on its barrier.
    if (n_iters > 0) {
      if (lane == 0) {
        mbar_expect_tx(kv_full, 2 * L::kKVBytes);
#pragma unroll
        for (int s = 0; s < kDSub; ++s) {
          tma_load_4d(sK + s * 16384, &tmK, kv_full, s * 64, hk, kv0, b);
          tma_load_4d(sV + s * 16384, &tmV, kv_full, s * 64, hk, kv0, b);
        }
      }
      for (int it = 0; it < n_iters; ++it) {
        const int st = it % kQStages;
        const uint32_t ph = (it / kQStages) & 1;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, wctx, kTimeoutEmptyBarrier)) break;
        int h, tq0;
        iter_coords(it, h, tq0);
        if (lane == 0) {
          uint8_t* q_dst = sQdO + st * 2 * L::kQBytes;
          uint8_t* do_dst = q_dst + L::kQBytes;
          mbar_expect_tx(&qdo_full[st], 2 * L::kQBytes);
#pragma unroll
          for (int s = 0; s < kDSub; ++s) {
            tma_load_4d(q_dst + s * 8192, &tmQ, &qdo_full[st], s * 64, h, tq0, b);
            tma_load_4d(do_dst + s * 8192, &tmdO, &qdo_full[st], s * 64, h, tq0, b);
          }
        }
        const size_t base = ((size_t)b * p.H + h) * p.T;
        float* stats = sStats + st * 128;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int qi = lane + 32 * j;
          const int tq = tq0 + qi;
          const bool valid = tq < p.T;
          // Out-of-range queries get +inf / 0: their probabilities come out as exactly zero.
          stats[qi] = valid ? p.lse[base + tq] * kLog2e : INFINITY;
          stats[64 + qi] = valid ? p.delta[base + tq] : 0.f;
        }
        mbar_arrive(&stat_full[st]);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer -----------------------------------------------
    if (lane == 0 && n_iters > 0) {
      const uint32_t idesc_st = make_idesc_bf16(128, 64, false, false);  // S^T, dP^T
      const uint32_t idesc_dv = make_idesc_bf16(128, D, false, true);    // dV, dK
      const uint32_t idesc_dq = make_idesc_bf16(128, 64, true, true);    // dQ^T
      // Descriptors of every operand at offset 0 of its buffer; the loops below only add offsets.
      const SmemDesc dK_k = make_smem_desc_parts(smem_u32(sK), 16, 1024);    // K, K-major (S^T)
      const SmemDesc dV_k = make_smem_desc_parts(smem_u32(sV), 16, 1024);    // V, K-major (dP^T)
      const SmemDesc dK_mn = make_smem_desc_parts(smem_u32(sK), D == 128 ? 16384 : 0, 1024);  // K^T
      const SmemDesc dQ_k = make_smem_desc_parts(smem_u32(sQdO), 16, 1024);  // Q / dO, K-major
      const SmemDesc dQ_mn = make_smem_desc_parts(smem_u32(sQdO), 8192, 1024);  // Q / dO as B, MN-major
      const SmemDesc dP_k = make_smem_desc_parts(smem_u32(sP), 16, 1024);    // P^T, K-major A
      const SmemDesc dS_k = make_smem_desc_parts(smem_u32(sdS), 16, 1024);   // dS^T, K-major A / B
      auto issue_scores = [&](int it) -> bool {
        const int st = it % kQStages;
        const uint32_t ph = (it / kQStages) & 1;
        if (!mbar_wait(&qdo_full[st], ph, wctx, kTimeoutFullBarrier)) return false;
        tcgen05_fence_after();
        const uint32_t q_off = st * 2 * L::kQBytes;
        const uint32_t do_off = q_off + L::kQBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offA = (k / 4) * 16384 + (k % 4) * 32;
          const uint32_t offB = (k / 4) * 8192 + (k % 4) * 32;
          if (k == 0)
            umma_bf16_ss_c<0>(tm_S, smem_desc_at(dK_k, offA), smem_desc_at(dQ_k, q_off + offB), idesc_st);
          else
            umma_bf16_ss_c<1>(tm_S, smem_desc_at(dK_k, offA), smem_desc_at(dQ_k, q_off + offB), idesc_st);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offA = (k / 4) * 16384 + (k % 4) * 32;
          const uint32_t offB = (k / 4) * 8192 + (k % 4) * 32;
          if (k == 0)
            umma_bf16_ss_c<0>(tm_dP, smem_desc_at(dV_k, offA), smem_desc_at(dQ_k, do_off + offB), idesc_st);
          else
            umma_bf16_ss_c<1>(tm_dP, smem_desc_at(dV_k, offA), smem_desc_at(dQ_k, do_off + offB), idesc_st);
        }
        tcgen05_commit(s_full);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, wctx, kTimeoutFullBarrier);
      if (ok) ok = issue_scores(0);
      for (int it = 0; it < n_iters && ok; ++it) {
        const int st = it % kQStages;
        if (it + 1 < n_iters) {
          if (!mbar_wait(sd_empty, it & 1, wctx, kTimeoutSoftmax)) break;
          if (!issue_scores(it + 1)) break;
        }
        if (!mbar_wait(&ps_full[it & 1], (it >> 1) & 1, wctx, kTimeoutSoftmax)) break;
        tcgen05_fence_after();
        const uint32_t q_off = st * 2 * L::kQBytes;
        const uint32_t do_off = q_off + L::kQBytes;
        const uint32_t p_off = (it & 1) * L::kPBytes;
        // dV += P^T dO ; dK += dS^T Q   (contraction over the 64 queries)
        if (it == 0) {
          umma_bf16_ss_c<0>(tm_dV, smem_desc_at(dP_k, p_off), smem_desc_at(dQ_mn, do_off), idesc_dv);
          umma_bf16_ss_c<0>(tm_dK, smem_desc_at(dS_k, p_off), smem_desc_at(dQ_mn, q_off), idesc_dv);
        } else {
          umma_bf16_ss_c<1>(tm_dV, smem_desc_at(dP_k, p_off), smem_desc_at(dQ_mn, do_off), idesc_dv);
          umma_bf16_ss_c<1>(tm_dK, smem_desc_at(dS_k, p_off), smem_desc_at(dQ_mn, q_off), idesc_dv);
        }
#pragma unroll
        for (int k = 1; k < kQRows / 16; ++k) {
          umma_bf16_ss_c<1>(tm_dV, smem_desc_at(dP_k, p_off + k * 32),
                            smem_desc_at(dQ_mn, do_off + k * 2048), idesc_dv);
          umma_bf16_ss_c<1>(tm_dK, smem_desc_at(dS_k, p_off + k * 32),
                            smem_desc_at(dQ_mn, q_off + k * 2048), idesc_dv);
        }
        // dQ^T = K^T dS^T (contraction over the 128 keys). For D = 64 the second 64 rows of the
        // M = 128 operand alias the first (leading offset 0) and are never read back.
        const uint32_t tm_dQ_it = tm_dQ + (it & 1) * 64;
#pragma unroll
        for (int k = 0; k < kKeys / 16; ++k) {
          if (k == 0)
            umma_bf16_ss_c<0>(tm_dQ_it, smem_desc_at(dK_mn, k * 2048),
                              smem_desc_at(dS_k, p_off + k * 2048), idesc_dq);
          else
            umma_bf16_ss_c<1>(tm_dQ_it, smem_desc_at(dK_mn, k * 2048),
                              smem_desc_at(dS_k, p_off + k * 2048), idesc_dq);
        }
        tcgen05_commit(&mma_done[it & 1]);
        tcgen05_commit(&qdo_empty[st]);
      }
    }
  } else {
    // ------------------------------ Softmax / drain / epilogue -------------------------------
    // Four threads per key row: warp w takes queries 16*(w/4) .. +15 of each 64-query tile. A warp
    // may only touch the TMEM lanes of its quarter (w % 4), which is what makes this split
    // possible: the four warps of a quarter address the same lanes, different columns.
    const int quarter = warp & 3;
    const int slice = warp >> 2;
    const int row = quarter * 32 + lane;  // key row within the tile == TMEM lane
    const int key = kv0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t col0 = slice * kSliceCols;
    bool ok = true;
    uint32_t grp_phase = 0;
    // Barrier among the softmax threads, built on an mbarrier so that it cannot outlive the wait
    // limit if some warp has already abandoned the tile.
    auto group_sync = [&]() -> bool {
      mbar_arrive(grp_bar);
      const bool done = mbar_wait(grp_bar, grp_phase & 1, wctx, kTimeoutSoftmax);
      ++grp_phase;
      return done;
    };

    // Adds dQ^T of iteration `it` (TMEM lane = head_dim index, column = query) to the fp32
    // gradient. The lanes of a warp hold 32 consecutive head_dim indices of the same query, so
    // each reduction instruction covers 128 contiguous bytes.
    const size_t q_stride = (size_t)p.H * D;
    auto drain_dq = [&](int it) {
      if (row >= D) return;
      int h, tq0;
      iter_coords(it, h, tq0);
      uint32_t v[16];
      tmem_ld_32x16(tm_dQ + (it & 1) * 64 + lane_addr + col0, v);
      tmem_ld_wait();
      const int tq_first = tq0 + (int)col0;
      float* dst = p.dq + (((size_t)b * p.T + tq_first) * p.H + h) * D + row;
      if (tq_first + kSliceCols <= p.T) {
#pragma unroll
        for (int i = 0; i < kSliceCols; ++i) {
          atomicAdd(dst, __uint_as_float(v[i]));
          dst += q_stride;
        }
      } else {
#pragma unroll
        for (int i = 0; i < kSliceCols; ++i) {
          if (tq_first + i < p.T) atomicAdd(dst, __uint_as_float(v[i]));
          dst += q_stride;
        }
      }
    };

    for (int it = 0; it < n_iters; ++it) {
      int h, tq0;
      iter_coords(it, h, tq0);
      const int st = it % kQStages;
      const float* stats = sStats + st * 128 + col0;
      if (!mbar_wait(&stat_full[st], (it / kQStages) & 1, wctx, kTimeoutFullBarrier)) {
        ok = false;
        break;
      }
      if (!mbar_wait(s_full, it & 1, wctx, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tcgen05_fence_after();
      uint32_t vs[16], vd[16];
      tmem_ld_32x16(tm_S + lane_addr + col0, vs);
      tmem_ld_32x16(tm_dP + lane_addr + col0, vd);
      float lse2[16], dlt[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float4 a = reinterpret_cast<const float4*>(stats)[c];
        const float4 d = reinterpret_cast<const float4*>(stats + 64)[c];
        lse2[4 * c + 0] = a.x, lse2[4 * c + 1] = a.y, lse2[4 * c + 2] = a.z, lse2[4 * c + 3] = a.w;
        dlt[4 * c + 0] = d.x, dlt[4 * c + 1] = d.y, dlt[4 * c + 2] = d.z, dlt[4 * c + 3] = d.w;
      }
      tmem_ld_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sd_empty);

      float pr[16], ds[16];
      const bool need_mask = (p.causal && (kv0 + kKeys - 1 > tq0 + offset)) ||
                             (kv0 + kKeys > p.S) || (tq0 + kQRows > p.T);
#pragma unroll
      for (int i = 0; i < kSliceCols; ++i) {
        float pv = fast_exp2(fmaf(__uint_as_float(vs[i]), p.scale_log2, -lse2[i]));
        if (need_mask) {
          const int tq = tq0 + (int)col0 + i;
          const bool visible = (key < p.S) && (tq < p.T) && (!p.causal || key <= tq + offset);
          pv = visible ? pv : 0.f;
        }
        pr[i] = pv;
        ds[i] = pv * (__uint_as_float(vd[i]) - dlt[i]);
      }

      // Buffer (it & 1) of P^T / dS^T was last read by the MMAs of tile it-2, whose completion
      // this warp has already observed when it drained dQ^T of that tile.
      uint8_t* prow = sP + (it & 1) * L::kPBytes + row * 128;
      uint8_t* dsrow = sdS + (it & 1) * L::kPBytes + row * 128;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint4 o, d;
        o.x = pack_bf16(pr[8 * c + 0], pr[8 * c + 1]);
        o.y = pack_bf16(pr[8 * c + 2], pr[8 * c + 3]);
        o.z = pack_bf16(pr[8 * c + 4], pr[8 * c + 5]);
        o.w = pack_bf16(pr[8 * c + 6], pr[8 * c + 7]);
        d.x = pack_bf16(ds[8 * c + 0], ds[8 * c + 1]);
        d.y = pack_bf16(ds[8 * c + 2], ds[8 * c + 3]);
        d.z = pack_bf16(ds[8 * c + 4], ds[8 * c + 5]);
        d.w = pack_bf16(ds[8 * c + 6], ds[8 * c + 7]);
        const int sw = (((slice * 2 + c) ^ (row & 7)) << 4);
        *reinterpret_cast<uint4*>(prow + sw) = o;
        *reinterpret_cast<uint4*>(dsrow + sw) = d;
      }
      fence_proxy_async_smem();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ps_full[it & 1]);
      // The MMAs of this tile may start as soon as every warp has arrived. Meanwhile move dQ^T of
      // the previous tile out of its TMEM buffer: tile it+1 overwrites that buffer, and its MMAs
      // need this warp's arrival on ps_full of tile it+1, which comes after this drain.
      if (it > 0) {
        if (!mbar_wait(&mma_done[(it - 1) & 1], ((it - 1) >> 1) & 1, wctx, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        drain_dq(it - 1);
        tcgen05_fence_before();
      }
    }

    if (ok && n_iters > 0) {
      ok = mbar_wait(&mma_done[(n_iters - 1) & 1], ((n_iters - 1) >> 1) & 1, wctx,
                     kTimeoutTmemFull);
      if (ok) {
        tcgen05_fence_after();
        drain_dq(n_iters - 1);
      }
    }
    // ---- epilogue: dK, dV (TMEM fp32) -> bf16 -> swizzled smem (over K / V tiles) -> TMA store --
    if (ok) {
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t tm_src = which == 0 ? tm_dK : tm_dV;
        uint8_t* dst = (which == 0 ? sK : sV) + row * 128;
#pragma unroll
        const float out_scale = which == 0 ? p.scale : 1.f;  // dS was left unscaled
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          if ((c & 3) != slice) continue;  // the warps of a row quartet split the column chunks
          uint32_t v[32];
          if (n_iters > 0) {
            tmem_ld_32x32(tm_src + lane_addr + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[8 * q4 + 0]) * out_scale,
                            __uint_as_float(v[8 * q4 + 1]) * out_scale);
            o.y = pack_bf16(__uint_as_float(v[8 * q4 + 2]) * out_scale,
                            __uint_as_float(v[8 * q4 + 3]) * out_scale);
            o.z = pack_bf16(__uint_as_float(v[8 * q4 + 4]) * out_scale,
                            __uint_as_float(v[8 * q4 + 5]) * out_scale);
            o.w = pack_bf16(__uint_as_float(v[8 * q4 + 6]) * out_scale,
                            __uint_as_float(v[8 * q4 + 7]) * out_scale);
            const int chunk = c * 4 + q4;
            *reinterpret_cast<uint4*>(dst + (chunk >> 3) * 16384 + (((chunk & 7) ^ (row & 7)) << 4)) = o;
          }
        }
      }
      fence_proxy_async_smem();
      ok = group_sync();  // all warps of every row quartet have written their chunks
      if (ok && slice == 0 && lane == 0 && kv0 + quarter * 32 < p.S) {
#pragma unroll
        for (int s2 = 0; s2 < kDSub; ++s2) {
          tma_store_4d(&tmdK, sK + s2 * 16384 + quarter * 32 * 128, s2 * 64, hk, kv0 + quarter * 32, b);
          tma_store_4d(&tmdV, sV + s2 * 16384 + quarter * 32 * 128, s2 * 64, hk, kv0 + quarter * 32, b);
        }
        tma_store_commit();
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  if (*abort_flag) {
    const uint64_t w0 = global_timer_ns();
    while (global_timer_ns() - w0 < 1000000ull) __nanosleep(1000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, t] = sum_d O[b, t, h, d] * dO[b, t, h, d]. D / 8 lanes share a (b, t, h) row, each
// with one 16-byte load of O and of dO, so a warp covers 256 / D rows per pass (D in {64, 128}).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                  const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                  int B, int T, int H, int D, int64_t do_tok_stride,
                                  int64_t do_batch_stride) {
  const int lanes_per_row = D >> 3;
  const int rows_per_warp = 32 / lanes_per_row;
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes_per_row;
  const int col = (lane % lanes_per_row) * 8;
  const int64_t rows = (int64_t)B * T * H;
  const int64_t first = ((int64_t)blockIdx.x * warps + (threadIdx.x >> 5)) * rows_per_warp;
  const int64_t step = (int64_t)gridDim.x * warps * rows_per_warp;
  for (int64_t r0 = first; r0 < rows; r0 += step) {
    const int64_t r = r0 + sub;
    float acc = 0.f;
    int h = 0, t = 0, b = 0;
    if (r < rows) {
      h = (int)(r % H);
      const int64_t bt = r / H;
      t = (int)(bt % T);
      b = (int)(bt / T);
      const uint4 a = *reinterpret_cast<const uint4*>(o + r * D + col);
      const uint4 g = *reinterpret_cast<const uint4*>(
          d_o + (int64_t)b * do_batch_stride + (int64_t)t * do_tok_stride + (int64_t)h * D + col);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(a2[i]);
        const float2 y = __bfloat1622float2(g2[i]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
    for (int s = lanes_per_row >> 1; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (r < rows && (lane % lanes_per_row) == 0) delta[((size_t)b * H + h) * T + t] = acc;
  }
}

template <int D>
void launch_bwd(const void* q, const void* k, const void* v, const void* d_o, float* dq, void* dk,
                void* dv, const float* lse, const float* delta, int B, int T, int S, int H, int Hk,
                bool causal, float scale, const int64_t* strides, cudaStream_t stream) {
  using L = BwdSmem<D>;
  CUtensorMap tQ, tK, tV, tdO, tdK, tdV;
  auto make4 = [&](CUtensorMap* tm, const void* base, TmapDtype dt, int heads, int len,
                   int64_t tok_stride, int64_t batch_stride, uint32_t box_inner, uint32_t box_rows,
                   TmapSwizzle sw) {
    const uint64_t esz = dt == TmapDtype::F32 ? 4 : 2;
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)len, (uint64_t)B};
    uint64_t st[3] = {(uint64_t)D * esz, (uint64_t)tok_stride * esz, (uint64_t)batch_stride * esz};
    uint32_t box[4] = {box_inner, 1, box_rows, 1};
    make_tmap(tm, base, dt, 4, dims, st, box, sw);
  };
  make4(&tQ, q, TmapDtype::BF16, H, T, strides[0], strides[1], 64, kQRows, TmapSwizzle::B128);
  make4(&tK, k, TmapDtype::BF16, Hk, S, strides[2], strides[3], 64, kKeys, TmapSwizzle::B128);
  make4(&tV, v, TmapDtype::BF16, Hk, S, strides[4], strides[5], 64, kKeys, TmapSwizzle::B128);
  make4(&tdO, d_o, TmapDtype::BF16, H, T, strides[6], strides[7], 64, kQRows, TmapSwizzle::B128);
  make4(&tdK, dk, TmapDtype::BF16, Hk, S, strides[8], strides[9], 64, 32, TmapSwizzle::B128);
  make4(&tdV, dv, TmapDtype::BF16, Hk, S, strides[10], strides[11], 64, 32, TmapSwizzle::B128);
  BwdParams p;
  p.B = B;
  p.T = T;
  p.S = S;
  p.H = H;
  p.Hk = Hk;
  p.causal = causal ? 1 : 0;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.lse = lse;
  p.delta = delta;
  p.dq = dq;
  p.status = status_ptr();
  auto kernel = flash_bwd_kernel<D>;
  ensure_dynamic_smem((const void*)kernel, L::kTotal);
  const int k_tiles = (S + kKeys - 1) / kKeys;
  const long long grid = (long long)k_tiles * B * Hk;
  kernel<<<(unsigned)grid, kThreads, L::kTotal, stream>>>(tQ, tK, tV, tdO, tdK, tdV, p);
  OB_LAUNCH_CHECK();
}

}  // namespace

void attn_delta(const void* o, const void* d_o, float* delta, int B, int T, int H, int D,
                int64_t do_tok_stride, int64_t do_batch_stride, cudaStream_t stream) {
  const int threads = 256;
  const int64_t rows = (int64_t)B * T * H;
  const int rows_per_block = (threads / 32) * (256 / D);
  const int blocks = (int)std::min<int64_t>((rows + rows_per_block - 1) / rows_per_block,
                                            (int64_t)device_sm_count() * 16);
  attn_delta_kernel<<<std::max(blocks, 1), threads, 0, stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, B, T, H, D, do_tok_stride,
      do_batch_stride);
  OB_LAUNCH_CHECK();
}

// strides = {q_tok, q_batch, k_tok, k_batch, v_tok, v_batch, do_tok, do_batch, dk_tok, dk_batch,
// dv_tok, dv_batch} in elements (the (heads, D) block of every tensor is contiguous).
// dq: zero-initialised fp32 (B, T, H, D), receives the gradient without the softmax scale;
// dk, dv: bf16 (B, S, Hk, D) with the given token / batch strides, so that they may be column
// slices of a wider buffer (the gradient of a fused q|k|v projection).
void flash_attn_bwd(const void* q, const void* k, const void* v, const void* d_o, float* dq,
                    void* dk, void* dv, const float* lse, const float* delta, int B, int T, int S,
                    int H, int Hk, int D, bool causal, float scale, const int64_t* strides,
                    cudaStream_t stream) {
  OB_CHECK(D == 64 || D == 128, "flash attention supports head_dim 64 or 128");
  OB_CHECK(H % Hk == 0, "query heads must be a multiple of KV heads");
  if (D == 128)
    launch_bwd<128>(q, k, v, d_o, dq, dk, dv, lse, delta, B, T, S, H, Hk, causal, scale, strides,
                    stream);
  else
    launch_bwd<64>(q, k, v, d_o, dq, dk, dv, lse, delta, B, T, S, H, Hk, causal, scale, strides,
                   stream);
}

}  // namespace ob

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (see noalloc.h for who needs it and the contract).
// ------------------------------------------------------------------------------------------------
#include <cstdio>
#include <cstring>
#include <mutex>

#include "api.h"
#include "noalloc.h"

namespace ob {
namespace {

constexpr size_t kNoallocDqBytes = (size_t)OB_NOALLOC_MAX_DQ_ELEMS * sizeof(float);
constexpr size_t kNoallocDeltaBytes = (size_t)OB_NOALLOC_MAX_ROWS * sizeof(float);

// Scratch that the regular entry point would allocate: [fp32 dQ accumulators | fp32 delta].
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoallocDqBytes + kNoallocDeltaBytes];

std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_base[64] = {nullptr};  // device address of the array, per device

int noalloc_fail(int code, const char* message, char* err, size_t err_len) {
  if (err != nullptr && err_len > 0) {
    std::strncpy(err, message, err_len - 1);
    err[err_len - 1] = '\0';
  }
  return code;
}

template <int D>
cudaError_t noalloc_launch(const void* q, const void* k, const void* v, const void* d_o, float* dq32,
                           void* dk, void* dv, const float* lse, const float* delta, int B, int T,
                           int S, int H, int Hk, bool causal, float scale, int* status,
                           cudaStream_t stream) {
  using L = BwdSmem<D>;
  CUtensorMap tQ, tK, tV, tdO, tdK, tdV;
  auto make4 = [&](CUtensorMap* tm, const void* base, TmapDtype dt, int heads, int len,
                   uint32_t box_inner, uint32_t box_rows, TmapSwizzle sw) {
    const uint64_t esz = dt == TmapDtype::F32 ? 4 : 2;
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)len, (uint64_t)B};
    uint64_t st[3] = {(uint64_t)D * esz, (uint64_t)heads * D * esz, (uint64_t)len * heads * D * esz};
    uint32_t box[4] = {box_inner, 1, box_rows, 1};
    make_tmap(tm, base, dt, 4, dims, st, box, sw);
  };
  make4(&tQ, q, TmapDtype::BF16, H, T, 64, kQRows, TmapSwizzle::B128);
  make4(&tK, k, TmapDtype::BF16, Hk, S, 64, kKeys, TmapSwizzle::B128);
  make4(&tV, v, TmapDtype::BF16, Hk, S, 64, kKeys, TmapSwizzle::B128);
  make4(&tdO, d_o, TmapDtype::BF16, H, T, 64, kQRows, TmapSwizzle::B128);
  make4(&tdK, dk, TmapDtype::BF16, Hk, S, 64, 32, TmapSwizzle::B128);
  make4(&tdV, dv, TmapDtype::BF16, Hk, S, 64, 32, TmapSwizzle::B128);
  BwdParams p;
  p.B = B;
  p.T = T;
  p.S = S;
  p.H = H;
  p.Hk = Hk;
  p.causal = causal ? 1 : 0;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.lse = lse;
  p.delta = delta;
  p.dq = dq32;
  p.status = status;
  auto kernel = flash_bwd_kernel<D>;
  // Recorded per device only once the driver has accepted it, so a failed first call is retried.
  cudaError_t rc = try_ensure_dynamic_smem((const void*)kernel, L::kTotal);
  if (rc != cudaSuccess) return rc;
  const int k_tiles = (S + kKeys - 1) / kKeys;
  const long long grid = (long long)k_tiles * B * Hk;
  kernel<<<(unsigned)grid, kThreads, L::kTotal, stream>>>(tQ, tK, tV, tdO, tdK, tdV, p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace
}  // namespace ob

extern "C" int ob_flash_attn_bwd_noalloc(const void* q, const void* k, const void* v,
                                         const void* out, const void* dout, const float* lse,
                                         void* dq, void* dk, void* dv, int B, int T, int S, int H,
                                         int Hk, int D, int causal, float scale, void* stream_ptr,
                                         int* status, char* err, size_t err_len) {
  using namespace ob;
  char msg[256];
  if (!q || !k || !v || !out || !dout || !lse || !dq || !dk || !dv)
    return noalloc_fail(-1, "ob_flash_attn_bwd_noalloc: null tensor pointer", err, err_len);
  if (B < 1 || T < 1 || S < 1 || H < 1 || Hk < 1 || H % Hk != 0 || (D != 64 && D != 128))
    return noalloc_fail(-1, "ob_flash_attn_bwd_noalloc: bad shape (need D in {64,128}, H % Hk == 0)",
                        err, err_len);
  if (causal && S < T)
    return noalloc_fail(-1, "ob_flash_attn_bwd_noalloc: causal attention needs S >= T", err, err_len);
  const long long dq_elems = (long long)B * T * H * D;
  const long long rows = (long long)B * H * T;
  if (dq_elems > OB_NOALLOC_MAX_DQ_ELEMS || rows > OB_NOALLOC_MAX_ROWS) {
    std::snprintf(msg, sizeof(msg),
                  "ob_flash_attn_bwd_noalloc: problem needs %lld dQ elements and %lld rows but the "
                  "built-in scratch holds at most %lld and %lld; use the allocating entry point",
                  dq_elems, rows, (long long)OB_NOALLOC_MAX_DQ_ELEMS, (long long)OB_NOALLOC_MAX_ROWS);
    return noalloc_fail(-2, msg, err, err_len);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess || dev < 0 || dev >= 64)
    return noalloc_fail(-3, "ob_flash_attn_bwd_noalloc: cannot query the current device", err, err_len);

  // One-time set-up for this device: resolve the device address of the static array.
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_base[dev] == nullptr) {
      void* ptr = nullptr;
      rc = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (rc != cudaSuccess || ptr == nullptr) {
        std::snprintf(msg, sizeof(msg), "ob_flash_attn_bwd_noalloc: cudaGetSymbolAddress failed: %s",
                      cudaGetErrorString(rc));
        return noalloc_fail(-3, msg, err, err_len);
      }
      g_noalloc_base[dev] = static_cast<unsigned char*>(ptr);
    }
    base = g_noalloc_base[dev];
  }
  float* dq32 = reinterpret_cast<float*>(base);
  float* delta = reinterpret_cast<float*>(base + kNoallocDqBytes);

  try {
    // The accumulators keep whatever the previous call left: clear what this call will add into.
    rc = cudaMemsetAsync(dq32, 0, (size_t)dq_elems * sizeof(float), stream);
    if (rc != cudaSuccess) throw std::runtime_error(cudaGetErrorString(rc));
    attn_delta(out, dout, delta, B, T, H, D, (int64_t)H * D, (int64_t)T * H * D, stream);
    rc = (D == 128) ? noalloc_launch<128>(q, k, v, dout, dq32, dk, dv, lse, delta, B, T, S, H, Hk,
                                          causal != 0, scale, status, stream)
                    : noalloc_launch<64>(q, k, v, dout, dq32, dk, dv, lse, delta, B, T, S, H, Hk,
                                         causal != 0, scale, status, stream);
    if (rc != cudaSuccess) throw std::runtime_error(cudaGetErrorString(rc));
    cast_f32_bf16(dq32, dq, dq_elems, stream, scale);
  } catch (const std::exception& e) {
    std::snprintf(msg, sizeof(msg), "ob_flash_attn_bwd_noalloc: %s", e.what());
    return noalloc_fail(-3, msg, err, err_len);
  }
  return 0;
}
