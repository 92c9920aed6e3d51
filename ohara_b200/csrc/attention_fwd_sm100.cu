// Causal / full flash-attention forward for sm_100a with grouped-query heads.
//
// One CTA per (batch, head, 128-query tile). Q, K and V tiles arrive by TMA straight from the
// (batch, seq, heads, head_dim) projection layout; S = Q K^T and O += P V run on tcgen05.mma with
// S (double buffered) and O accumulating in TMEM. Eight softmax warps, two threads per query row:
// warps 0-3 exponentiate key columns 0-63 of a tile, warps 4-7 columns 64-127 (the element-wise
// work is bound by instruction latency, so it is spread over two warps per scheduler). Both
// threads of a row scan all 128 scores for the row maximum, so they agree on it without talking to
// each other; each keeps a partial row sum, and the two are added once, in the epilogue. P goes as
// bf16 into swizzled shared memory (double buffered; the A operand of the second MMA), and O is
// rescaled in TMEM only when the running max moved by more than 2^8 (lazy rescaling; the final
// division by the row sum makes this exact). While the softmax of tile j runs, the MMA warp has
// already issued S for tile j+1.
//
// Warp roles (320 threads): 0-7 softmax + epilogue, 8 TMA producer, 9 MMA issuer / TMEM owner.
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

constexpr int kBlockQ = 128;
constexpr int kBlockKV = 128;
constexpr int kThreads = 320;
constexpr int kSoftmaxWarps = 8;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

struct FwdParams {
  int B, T, S, H, Hk;
  int causal;
  float scale_log2;
  float* lse;  // (B, H, T) natural-log log-sum-exp of the scaled scores
  int* status;
};

template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = 128 * D * 2;  // Q, K, V tiles
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kTileBytes;
  static constexpr int kV = kK + 2 * kTileBytes;
  static constexpr int kP = kV + 2 * kTileBytes;   // 2 buffers of P
  static constexpr int kSums = kP + 2 * kPBytes;   // 2 x 128 partial row sums (epilogue exchange)
  static constexpr int kBars = kSums + 256 * 4;
  // At least 120 KB so two CTAs never share an SM (each allocates all 512 TMEM columns).
  static constexpr int kTotal = (kBars + 256 + 1024) > 120 * 1024 ? (kBars + 256 + 1024) : 120 * 1024;
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                 const FwdParams p) {
  using L = FwdSmem<D>;
  constexpr int kDSub = D / 64;  // 64-element (128-byte) sub-tiles along head_dim
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem + L::kQ;
  uint8_t* sK = smem + L::kK;
  uint8_t* sV = smem + L::kV;
  uint8_t* sP = smem + L::kP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* s_empty = bars + 11;    // 2
  // p_full and pv_done alternate between two barriers by tile parity: their waiters have already
  // enabled the next completion when they start to wait, so a single barrier could complete twice
  // before a delayed waiter looks, which a parity wait cannot tell from "not yet".
  uint64_t* p_full = bars + 13;     // 2
  uint64_t* pv_done = bars + 15;    // 2
  uint64_t* grp_bar = bars + 17;    // 1 (all softmax threads, epilogue only)
  float* sSums = reinterpret_cast<float*>(smem + L::kSums);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Heaviest (latest) query tiles first so the tail of the grid is made of short CTAs.
  const int q_tiles = (p.T + kBlockQ - 1) / kBlockQ;
  int bid = blockIdx.x;
  const int h = bid % p.H;
  bid /= p.H;
  const int b = bid % p.B;
  const int qt = q_tiles - 1 - bid / p.B;
  const int hk = h / (p.H / p.Hk);
  const int t0 = qt * kBlockQ;
  const int offset = p.S - p.T;  // key index visible to query i is <= i + offset
  int n_kv = (p.S + kBlockKV - 1) / kBlockKV;
  if (p.causal) {
    const int last_key = min(t0 + kBlockQ - 1, p.T - 1) + offset;
    n_kv = min(n_kv, last_key / kBlockKV + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], kSoftmaxWarps);
      mbar_init(&p_full[i], kSoftmaxWarps);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(grp_bar, kSoftmaxWarps * 32);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_O = tmem_base + 256;

  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ---------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, L::kTileBytes);
#pragma unroll
      for (int s = 0; s < kDSub; ++s) tma_load_4d(sQ + s * 16384, &tmQ, q_full, s * 64, h, t0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, wctx, kTimeoutEmptyBarrier)) break;
        mbar_expect_tx(&k_full[st], L::kTileBytes);
#pragma unroll
        for (int s = 0; s < kDSub; ++s)
          tma_load_4d(sK + st * L::kTileBytes + s * 16384, &tmK, &k_full[st], s * 64, hk,
                      j * kBlockKV, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, wctx, kTimeoutEmptyBarrier)) break;
        mbar_expect_tx(&v_full[st], L::kTileBytes);
#pragma unroll
        for (int s = 0; s < kDSub; ++s)
          tma_load_4d(sV + st * L::kTileBytes + s * 16384, &tmV, &v_full[st], s * 64, hk,
                      j * kBlockKV, b);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer -----------------------------------------------
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      const uint32_t idesc_o = make_idesc_bf16(128, D, false, true);
      // Descriptors at offset 0 of each buffer; the issue loops only add offsets.
      const SmemDesc dQ = make_smem_desc_parts(smem_u32(sQ), 16, 1024);
      const SmemDesc dK = make_smem_desc_parts(smem_u32(sK), 16, 1024);
      const SmemDesc dP = make_smem_desc_parts(smem_u32(sP), 16, 1024);
      const SmemDesc dV = make_smem_desc_parts(smem_u32(sV), 16384, 1024);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, wctx, kTimeoutFullBarrier)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, wctx, kTimeoutSoftmax)) return false;
        tcgen05_fence_after();
        const uint32_t k_off = st * L::kTileBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * 16384 + (k % 4) * 32;
          if (k == 0)
            umma_bf16_ss_c<0>(tmem_S[st], smem_desc_at(dQ, off), smem_desc_at(dK, k_off + off), idesc_s);
          else
            umma_bf16_ss_c<1>(tmem_S[st], smem_desc_at(dQ, off), smem_desc_at(dK, k_off + off), idesc_s);
        }
        tcgen05_commit(&s_full[st]);
        tcgen05_commit(&k_empty[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, wctx, kTimeoutFullBarrier);
      if (ok && n_kv > 0) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          if (!issue_s(j + 1)) break;
        }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1, wctx, kTimeoutSoftmax)) break;
        if (!mbar_wait(&v_full[st], ph, wctx, kTimeoutFullBarrier)) break;
        tcgen05_fence_after();
        const uint32_t v_off = st * L::kTileBytes;
        const uint32_t p_off = (j & 1) * L::kPBytes;
        umma_bf16_ss(tmem_O, smem_desc_at(dP, p_off), smem_desc_at(dV, v_off), idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 1; k < kBlockKV / 16; ++k)
          umma_bf16_ss_c<1>(tmem_O, smem_desc_at(dP, p_off + (k / 4) * 16384 + (k % 4) * 32),
                            smem_desc_at(dV, v_off + k * 2048), idesc_o);
        tcgen05_commit(&pv_done[j & 1]);
        tcgen05_commit(&v_empty[st]);
      }
    }
  } else {
    // ------------------------------ Softmax + epilogue (warps 0..3) --------------------------
    const int quarter = warp & 3;  // TMEM lane quarter this warp may touch
    const int half = warp >> 2;    // which 64 key columns of a tile (and which half of head_dim)
    const int row = quarter * 32 + lane;  // query row within the tile == TMEM lane
    const int t = t0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float m_run = -INFINITY;  // running max, log2 domain, possibly stale (lazy rescale)
    float l_run = 0.f;        // partial row sum over this thread's columns
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, wctx, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const int kv0 = j * kBlockKV;
      const bool need_mask =
          (p.causal && (kv0 + kBlockKV - 1 > t0 + offset)) || (kv0 + kBlockKV > p.S);
      const int limit = p.causal ? min(t + offset, p.S - 1) : (p.S - 1);  // last visible key
      // Own 64 columns stay in registers; the other 64 are only scanned for the row maximum.
      uint32_t own[64], other[64];
      tmem_ld_32x32(tmem_S[st] + lane_addr + half * 64, reinterpret_cast<uint32_t(&)[32]>(own[0]));
      tmem_ld_32x32(tmem_S[st] + lane_addr + half * 64 + 32,
                    reinterpret_cast<uint32_t(&)[32]>(own[32]));
      tmem_ld_32x32(tmem_S[st] + lane_addr + (half ^ 1) * 64,
                    reinterpret_cast<uint32_t(&)[32]>(other[0]));
      tmem_ld_32x32(tmem_S[st] + lane_addr + (half ^ 1) * 64 + 32,
                    reinterpret_cast<uint32_t(&)[32]>(other[32]));
      tmem_ld_wait();
      // S buffer is free for the MMA of tile j+2.
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[st]);

      float s[64];
      float mx = -INFINITY;
      const int own0 = kv0 + half * 64, other0 = kv0 + (half ^ 1) * 64;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          s[i] = (own0 + i > limit) ? -INFINITY : __uint_as_float(own[i]);
          mx = fmaxf(mx, s[i]);
          if (other0 + i <= limit) mx = fmaxf(mx, __uint_as_float(other[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          s[i] = __uint_as_float(own[i]);
          mx = fmaxf(mx, fmaxf(s[i], __uint_as_float(other[i])));
        }
      }
      const float m_new = mx * p.scale_log2;
      // Lazy rescale: keep the stale max unless it is too far behind (or not set yet).
      const bool grow = (m_new > m_run + kRescaleThreshold) || (m_run == -INFINITY);
      float alpha = 1.f;
      float m_use = m_run;
      if (grow && m_new > -INFINITY) {
        alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
        m_use = m_new;
      }
      if (m_use == -INFINITY) m_use = 0.f;  // fully masked so far: every p below is 0
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        s[i] = fast_exp2(fmaf(s[i], p.scale_log2, -m_use));
        sum += s[i];
      }
      l_run = l_run * alpha + sum;
      m_run = (grow && m_new > -INFINITY) ? m_new : m_run;

      // O may only be rescaled between two PV products. Both threads of a row take the same
      // decision (same maximum) and each rescales its half of head_dim.
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, wctx, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[16];
          const uint32_t addr = tmem_O + lane_addr + half * (D / 2) + c * 16;
          tmem_ld_32x16(addr, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x16(addr, v);
        }
        tmem_st_wait();
      }
      // P buffer (j & 1) was last read by the PV product of tile j-2.
      if (j > 1) {
        if (!mbar_wait(&pv_done[j & 1], ((j - 2) >> 1) & 1, wctx, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
      }
      // Write P (bf16) as a K-major, 128B-swizzled A operand: this thread's 64 columns are one of
      // the two 64-column sub-tiles.
      uint8_t* prow = sP + (j & 1) * L::kPBytes + half * 16384 + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 o;
        o.x = pack_bf16(s[8 * c + 0], s[8 * c + 1]);
        o.y = pack_bf16(s[8 * c + 2], s[8 * c + 3]);
        o.z = pack_bf16(s[8 * c + 4], s[8 * c + 5]);
        o.w = pack_bf16(s[8 * c + 6], s[8 * c + 7]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = o;
      }
      fence_proxy_async_smem();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[j & 1]);
    }

    // ---- epilogue: O / l -> bf16 -> swizzled smem (reusing P buffer 0) -> TMA store ------------
    if (ok && n_kv > 0)
      ok = mbar_wait(&pv_done[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, wctx, kTimeoutTmemFull);
    // The two partial sums of a row meet in shared memory; the barrier is an mbarrier so that it
    // cannot outlive the wait limit if a warp has already given up.
    sSums[half * 128 + row] = l_run;
    mbar_arrive(grp_bar);
    if (!mbar_wait(grp_bar, 0, wctx, kTimeoutSoftmax)) ok = false;
    if (ok) {
      tcgen05_fence_after();
      const float l_total = l_run + sSums[(half ^ 1) * 128 + row];
      const float inv_l = (l_total > 0.f) ? 1.f / l_total : 0.f;
      uint8_t* orow = sP + row * 128;
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c = half * (D / 64) + cc;  // 32-column chunk of head_dim
        uint32_t v[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tmem_O + lane_addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(v[8 * q4 + 0]) * inv_l, __uint_as_float(v[8 * q4 + 1]) * inv_l);
          o.y = pack_bf16(__uint_as_float(v[8 * q4 + 2]) * inv_l, __uint_as_float(v[8 * q4 + 3]) * inv_l);
          o.z = pack_bf16(__uint_as_float(v[8 * q4 + 4]) * inv_l, __uint_as_float(v[8 * q4 + 5]) * inv_l);
          o.w = pack_bf16(__uint_as_float(v[8 * q4 + 6]) * inv_l, __uint_as_float(v[8 * q4 + 7]) * inv_l);
          const int chunk = c * 4 + q4;  // 16-byte chunk index along head_dim
          *reinterpret_cast<uint4*>(orow + (chunk >> 3) * 16384 + (((chunk & 7) ^ (row & 7)) << 4)) = o;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(grp_bar);
      if (!mbar_wait(grp_bar, 1, wctx, kTimeoutSoftmax)) ok = false;
      if (ok && half == 0 && lane == 0 && t0 + quarter * 32 < p.T) {
#pragma unroll
        for (int s2 = 0; s2 < kDSub; ++s2)
          tma_store_4d(&tmO, sP + s2 * 16384 + quarter * 32 * 128, s2 * 64, h, t0 + quarter * 32, b);
        tma_store_commit();
        tma_store_wait_all<0>();
      }
      if (half == 0 && t < p.T && p.lse != nullptr) {
        const float lse2 = (l_total > 0.f) ? (m_run + log2f(l_total)) : -INFINITY;
        p.lse[((size_t)b * p.H + h) * p.T + t] = lse2 * (1.f / kLog2e);
      }
    }
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

template <int D>
void launch_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T,
                int S, int H, int Hk, bool causal, float scale, int64_t q_tok_stride,
                int64_t k_tok_stride, int64_t v_tok_stride, int64_t q_batch_stride,
                int64_t k_batch_stride, int64_t v_batch_stride, cudaStream_t stream) {
  using L = FwdSmem<D>;
  CUtensorMap tQ, tK, tV, tO;
  auto make4 = [&](CUtensorMap* tm, const void* base, int heads, int len, int64_t tok_stride,
                   int64_t batch_stride, uint32_t box_rows) {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)len, (uint64_t)B};
    uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)tok_stride * 2, (uint64_t)batch_stride * 2};
    uint32_t box[4] = {64, 1, box_rows, 1};
    make_tmap(tm, base, TmapDtype::BF16, 4, dims, strides, box, TmapSwizzle::B128);
  };
  make4(&tQ, q, H, T, q_tok_stride, q_batch_stride, 128);
  make4(&tK, k, Hk, S, k_tok_stride, k_batch_stride, 128);
  make4(&tV, v, Hk, S, v_tok_stride, v_batch_stride, 128);
  make4(&tO, o, H, T, (int64_t)H * D, (int64_t)T * H * D, 32);
  FwdParams p;
  p.B = B;
  p.T = T;
  p.S = S;
  p.H = H;
  p.Hk = Hk;
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * kLog2e;
  p.lse = lse;
  p.status = status_ptr();
  auto kernel = flash_fwd_kernel<D>;
  ensure_dynamic_smem((const void*)kernel, L::kTotal);
  const int q_tiles = (T + kBlockQ - 1) / kBlockQ;
  const long long grid = (long long)q_tiles * B * H;
  kernel<<<(unsigned)grid, kThreads, L::kTotal, stream>>>(tQ, tK, tV, tO, p);
  OB_LAUNCH_CHECK();
}

}  // namespace

// q: (B, T, H, D), k/v: (B, S, Hk, D) with contiguous (heads, D); o: contiguous (B, T, H, D).
void flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T,
                    int S, int H, int Hk, int D, bool causal, float scale, int64_t q_tok_stride,
                    int64_t k_tok_stride, int64_t v_tok_stride, int64_t q_batch_stride,
                    int64_t k_batch_stride, int64_t v_batch_stride, cudaStream_t stream) {
  OB_CHECK(D == 64 || D == 128, "flash attention supports head_dim 64 or 128");
  OB_CHECK(H % Hk == 0, "query heads must be a multiple of KV heads");
  OB_CHECK(!causal || S >= T, "causal attention needs at least as many keys as queries");
  if (D == 128)
    launch_fwd<128>(q, k, v, o, lse, B, T, S, H, Hk, causal, scale, q_tok_stride, k_tok_stride,
                    v_tok_stride, q_batch_stride, k_batch_stride, v_batch_stride, stream);
  else
    launch_fwd<64>(q, k, v, o, lse, B, T, S, H, Hk, causal, scale, q_tok_stride, k_tok_stride,
                   v_tok_stride, q_batch_stride, k_batch_stride, v_batch_stride, stream);
}

}  // namespace ob
