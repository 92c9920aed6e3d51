// Bandwidth-bound kernels: RMSNorm, RoPE, SwiGLU, casts, embedding, fused optimizers' elementwise
// parts. All use 16-byte vector accesses and fp32 math; tensors are bf16 unless noted.
#include "common.cuh"
#include "host_utils.h"

namespace ob {

namespace {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
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
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * w, optionally with a fused residual add
// (x = x + delta is written back to `x_out` and normalised). One warp per row.
// ------------------------------------------------------------------------------------------------
template <bool HAS_DELTA>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ delta,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ x_out, float* __restrict__ rstd_out,
                                   int rows, int d, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vecs = d >> 3;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * d);
    const bf16x8* dr = HAS_DELTA ? reinterpret_cast<const bf16x8*>(delta + (size_t)row * d) : nullptr;
    bf16x8* xo = HAS_DELTA ? reinterpret_cast<bf16x8*>(x_out + (size_t)row * d) : nullptr;
    float ss = 0.f;
    for (int v = lane; v < vecs; v += 32) {
      float f[8];
      unpack8(xr[v], f);
      if (HAS_DELTA) {
        float g[8];
        unpack8(dr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
        bf16x8 packed = pack8(f);
        xo[v] = packed;
        unpack8(packed, f);  // normalise exactly what later kernels will read
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)d + eps);
    if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
    const bf16x8* src = HAS_DELTA ? reinterpret_cast<const bf16x8*>(xo) : xr;
    bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)row * d);
    for (int v = lane; v < vecs; v += 32) {
      float f[8];
      unpack8(src[v], f);
      const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v];
      const float4 w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
      const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * ww[i];
      yr[v] = pack8(f);
    }
  }
}

// Register-resident forward for rows of at most VPL * 256 elements: a warp handles two rows per
// pass, issues every load of both rows before it touches the data and keeps the values in
// registers between the sum of squares and the scaling (the generic kernel above reads a row
// twice and has one row's loads in flight per warp).
template <int VPL, bool HAS_DELTA>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                       const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                       __nv_bfloat16* __restrict__ x_out, float* __restrict__ rstd_out, int rows,
                       int d, float eps) {
  const int lane = threadIdx.x & 31;
  const int vecs = d >> 3;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * 2; row0 < rows;
       row0 += warps * 2) {
    bf16x8 raw[2][VPL], extra[2][VPL];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = row0 + r;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int v = lane + 32 * j;
        if (row < rows && v < vecs) {
          raw[r][j] = reinterpret_cast<const bf16x8*>(x + (size_t)row * d)[v];
          if (HAS_DELTA) extra[r][j] = reinterpret_cast<const bf16x8*>(delta + (size_t)row * d)[v];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = row0 + r;
      if (row >= rows) break;  // uniform across the warp
      float f[VPL][8];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int v = lane + 32 * j;
        if (v < vecs) {
          unpack8(raw[r][j], f[j]);
          if (HAS_DELTA) {
            float g[8];
            unpack8(extra[r][j], g);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[j][i] += g[i];
            const bf16x8 packed = pack8(f[j]);
            reinterpret_cast<bf16x8*>(x_out + (size_t)row * d)[v] = packed;
            unpack8(packed, f[j]);  // normalise exactly what later kernels will read
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += f[j][i] * f[j][i];
        }
      }
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / (float)d + eps);
      if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int v = lane + 32 * j;
        if (v < vecs) {
          const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v];
          const float4 w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
          const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = f[j][i] * rstd * ww[i];
          reinterpret_cast<bf16x8*>(y + (size_t)row * d)[v] = pack8(o);
        }
      }
    }
  }
}

// RMSNorm backward. dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres), dw += sum_rows(dy*xhat).
// One warp per row; every lane owns the same VPL 8-element column groups for all of its rows, so
// x, dy and the dw partial sums stay in registers. Per-warp partials are combined through shared
// memory and flushed with one atomicAdd per column per CTA.
template <int VPL, bool HAS_DRES>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw, int rows, int d) {
  extern __shared__ float dw_smem[];  // d floats
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_smem[i] = 0.f;
  __syncthreads();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vecs = d >> 3;
  float wreg[VPL][8];
  float acc[VPL][8];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane + 32 * j;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc[j][i] = 0.f;
      wreg[j][i] = (v < vecs) ? w[8 * v + i] : 0.f;
    }
  }
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)row * d);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * d);
    const float r = rstd[row];
    float g[VPL][8], xh[VPL][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int v = lane + 32 * j;
      if (v < vecs) {
        unpack8(dyr[v], g[j]);
        unpack8(xr[v], xh[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[j][i] *= r;
          dot += g[j][i] * wreg[j][i] * xh[j][i];
        }
      }
    }
    dot = warp_sum(dot) / (float)d;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + (size_t)row * d);
    const bf16x8* drr =
        HAS_DRES ? reinterpret_cast<const bf16x8*>(dres + (size_t)row * d) : nullptr;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int v = lane + 32 * j;
      if (v < vecs) {
        float o[8];
        float extra[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (HAS_DRES) unpack8(drr[v], extra);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o[i] = r * (g[j][i] * wreg[j][i] - xh[j][i] * dot) + extra[i];
          acc[j][i] += g[j][i] * xh[j][i];
        }
        dxr[v] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane + 32 * j;
    if (v < vecs) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&dw_smem[8 * v + i], acc[j][i]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(&dw[i], dw_smem[i]);
}

// ------------------------------------------------------------------------------------------------
// RoPE on interleaved pairs for q (B,T,H,D) and k (B,T,Hk,D) in one launch. cos/sin are (T, D/2)
// fp32 rows for the positions being processed. `sign` = -1 rotates by -theta (the backward pass).
// ------------------------------------------------------------------------------------------------
// One warp per token. When D / 8 divides 32 (every head_dim that is a power of two up to 256) a
// lane keeps the same position inside the head for every vector it touches, so it loads its
// cos / sin values once per token (FIXED); other head sizes reload them per vector.
template <bool FIXED>
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                            __nv_bfloat16* __restrict__ qo, __nv_bfloat16* __restrict__ ko,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int B,
                            int T, int H, int Hk, int D, float sign, int64_t q_row_stride,
                            int64_t k_row_stride, int64_t qo_row_stride, int64_t ko_row_stride) {
  const int vec_per_head = D >> 3;
  const int lane = threadIdx.x & 31;
  const int q_vecs = H * vec_per_head;
  const int all_vecs = q_vecs + Hk * vec_per_head;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int tokens = B * T;
  for (int bt = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; bt < tokens; bt += warps) {
    const int t = bt % T;
    const float* cos_row = cos_t + (size_t)t * (D >> 1);
    const float* sin_row = sin_t + (size_t)t * (D >> 1);
    float cc[4], ssn[4];
    int c = FIXED ? (lane & (vec_per_head - 1)) : 0;
    if (FIXED) {
      const float4 cs = *reinterpret_cast<const float4*>(cos_row + c * 4);
      const float4 sn = *reinterpret_cast<const float4*>(sin_row + c * 4);
      cc[0] = cs.x, cc[1] = cs.y, cc[2] = cs.z, cc[3] = cs.w;
      ssn[0] = sn.x * sign, ssn[1] = sn.y * sign, ssn[2] = sn.z * sign, ssn[3] = sn.w * sign;
    }
    const __nv_bfloat16* q_src = q + bt * q_row_stride;
    const __nv_bfloat16* k_src = k + bt * k_row_stride;
    __nv_bfloat16* q_dst = qo + bt * qo_row_stride;
    __nv_bfloat16* k_dst = ko + bt * ko_row_stride;
    for (int v = lane; v < all_vecs; v += 32) {
      const bool is_q = v < q_vecs;
      const int local = is_q ? v : v - q_vecs;
      const int head = local / vec_per_head;
      if (!FIXED) {
        c = local - head * vec_per_head;
        const float4 cs = *reinterpret_cast<const float4*>(cos_row + c * 4);
        const float4 sn = *reinterpret_cast<const float4*>(sin_row + c * 4);
        cc[0] = cs.x, cc[1] = cs.y, cc[2] = cs.z, cc[3] = cs.w;
        ssn[0] = sn.x * sign, ssn[1] = sn.y * sign, ssn[2] = sn.z * sign, ssn[3] = sn.w * sign;
      }
      const int off = head * D + c * 8;
      const __nv_bfloat16* src = (is_q ? q_src : k_src) + off;
      __nv_bfloat16* dst = (is_q ? q_dst : k_dst) + off;
      float f[8], o[8];
      unpack8(*reinterpret_cast<const bf16x8*>(src), f);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o[2 * i] = f[2 * i] * cc[i] - f[2 * i + 1] * ssn[i];
        o[2 * i + 1] = f[2 * i] * ssn[i] + f[2 * i + 1] * cc[i];
      }
      *reinterpret_cast<bf16x8*>(dst) = pack8(o);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// SwiGLU: a = silu(g) * u and its backward. g/u/dg/du may be column slices of a wider matrix, so
// each takes a row pitch.
// ------------------------------------------------------------------------------------------------
// A block walks over pairs of rows and its threads over the 8-element column groups: no index
// division in the loop, and the loads of two rows are in flight before either is consumed. Rows
// narrower than the block (fewer than blockDim.x column groups) share it: ``tpr`` threads per row,
// blockDim.x / tpr row pairs per pass, so that no thread idles on the narrow expert layers.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g,
                                  const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ a,
                                  int64_t rows, int h, int tpr, int64_t g_pitch, int64_t u_pitch,
                                  int64_t a_pitch) {
  const int vecs = h >> 3;
  const int sub = threadIdx.x / tpr, v0 = threadIdx.x - sub * tpr, rpb = blockDim.x / tpr;
  for (int64_t r = ((int64_t)blockIdx.x * rpb + sub) * 2; r < rows;
       r += (int64_t)gridDim.x * rpb * 2) {
    const bool two = r + 1 < rows;
    for (int v = v0; v < vecs; v += tpr) {
      const int c = v * 8;
      bf16x8 g_raw[2], u_raw[2];
      g_raw[0] = *reinterpret_cast<const bf16x8*>(g + r * g_pitch + c);
      u_raw[0] = *reinterpret_cast<const bf16x8*>(u + r * u_pitch + c);
      if (two) {
        g_raw[1] = *reinterpret_cast<const bf16x8*>(g + (r + 1) * g_pitch + c);
        u_raw[1] = *reinterpret_cast<const bf16x8*>(u + (r + 1) * u_pitch + c);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (j == 1 && !two) break;
        float gf[8], uf[8], o[8];
        unpack8(g_raw[j], gf);
        unpack8(u_raw[j], uf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = gf[i] / (1.f + __expf(-gf[i])) * uf[i];
        *reinterpret_cast<bf16x8*>(a + (r + j) * a_pitch + c) = pack8(o);
      }
    }
  }
}

__global__ void __launch_bounds__(256, 6)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ da, const __nv_bfloat16* __restrict__ g,
                  const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ dg,
                  __nv_bfloat16* __restrict__ du, int64_t rows, int h, int tpr,
                  int64_t da_pitch, int64_t g_pitch, int64_t u_pitch, int64_t dg_pitch,
                  int64_t du_pitch) {
  // One row per pass and thread group (three loads in flight per thread): the two-row form of the
  // forward kernel needs 95 registers here and loses more to occupancy than it gains. ``tpr``
  // threads share a row, as in the forward kernel.
  const int vecs = h >> 3;
  const int sub = threadIdx.x / tpr, v0 = threadIdx.x - sub * tpr, rpb = blockDim.x / tpr;
  for (int64_t r = (int64_t)blockIdx.x * rpb + sub; r < rows; r += (int64_t)gridDim.x * rpb) {
    for (int v = v0; v < vecs; v += tpr) {
      const int c = v * 8;
      const bf16x8 d_raw = *reinterpret_cast<const bf16x8*>(da + r * da_pitch + c);
      const bf16x8 g_raw = *reinterpret_cast<const bf16x8*>(g + r * g_pitch + c);
      const bf16x8 u_raw = *reinterpret_cast<const bf16x8*>(u + r * u_pitch + c);
      float df[8], gf[8], uf[8], og[8], ou[8];
      unpack8(d_raw, df);
      unpack8(g_raw, gf);
      unpack8(u_raw, uf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float sig = __fdividef(1.f, 1.f + __expf(-gf[i]));
        const float silu = gf[i] * sig;
        ou[i] = df[i] * silu;
        og[i] = df[i] * uf[i] * (sig + silu * (1.f - sig));
      }
      *reinterpret_cast<bf16x8*>(dg + r * dg_pitch + c) = pack8(og);
      *reinterpret_cast<bf16x8*>(du + r * du_pitch + c) = pack8(ou);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Casts and embedding
// ------------------------------------------------------------------------------------------------
__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                     int64_t n, float scale) {
  const int64_t vecs = n >> 3;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < vecs;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(in)[2 * idx];
    const float4 b = reinterpret_cast<const float4*>(in)[2 * idx + 1];
    const float f[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                        b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    reinterpret_cast<bf16x8*>(out)[idx] = pack8(f);
  }
  if (blockIdx.x == 0) {
    for (int64_t i = (vecs << 3) + threadIdx.x; i < n; i += blockDim.x)
      out[i] = __float2bfloat16_rn(in[i] * scale);
  }
}

__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const float* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int64_t tokens, int d,
                                     int vocab) {
  const int vecs = d >> 3;
  const int64_t total = tokens * vecs;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vecs;
    const int c = (int)(idx - t * vecs);
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const float4* src = reinterpret_cast<const float4*>(table + id * d) + 2 * c;
    const float4 a = src[0], b = src[1];
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    reinterpret_cast<bf16x8*>(out + t * d)[c] = pack8(f);
  }
}

__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, int64_t tokens, int d, int vocab) {
  const int vecs = d >> 3;
  const int64_t total = tokens * vecs;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vecs;
    const int c = (int)(idx - t * vecs);
    const int64_t id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(dout + t * d)[c], f);
    float4* dst = reinterpret_cast<float4*>(dtable + id * d) + 2 * c;
    atomicAdd(dst, make_float4(f[0], f[1], f[2], f[3]));
    atomicAdd(dst + 1, make_float4(f[4], f[5], f[6], f[7]));
  }
}

// ------------------------------------------------------------------------------------------------
// AdamW on an fp32 master tensor; optionally refreshes the bf16 compute copy in the same pass.
// Matches torch.optim.AdamW: decoupled decay, bias-corrected moments, eps added after the sqrt.
// ------------------------------------------------------------------------------------------------
template <typename GradT>
__global__ void adamw_kernel(float* __restrict__ p, const GradT* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ shadow, int64_t n, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2,
                             float grad_scale) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float grad = static_cast<float>(g[i]) * grad_scale;
    float param = p[i] * (1.f - lr * wd);
    const float mi = m[i] + (1.f - beta1) * (grad - m[i]);
    const float vi = v[i] + (1.f - beta2) * (grad * grad - v[i]);
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi / bc2) + eps;
    param -= (lr / bc1) * mi / denom;
    p[i] = param;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(param);
  }
}

inline int grid_for(int64_t work_items, int threads, int max_blocks_per_sm = 8) {
  const int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)device_sm_count() * max_blocks_per_sm;
  return (int)std::max<int64_t>(1, std::min<int64_t>(blocks, cap));
}

// Threads that share one row of ``vecs`` 16-byte groups: the smallest of 32, 64, 128, ... that
// covers the row, capped at the block size.
inline int threads_per_row(int vecs, int threads) {
  int tpr = 32;
  while (tpr < vecs && tpr < threads) tpr <<= 1;
  return tpr;
}

}  // namespace

void rmsnorm_fwd(const void* x, const void* delta, const float* w, void* y, void* x_out, float* rstd,
                 int rows, int d, float eps, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "rmsnorm: width must be a multiple of 8");
  const int threads = 256;
  const int vpl = (d / 8 + 31) / 32;
  if (vpl <= 4) {
    const int blocks = grid_for((int64_t)((rows + 1) / 2) * 32, threads, 8);
    const auto* xp = (const __nv_bfloat16*)x;
    const auto* dp = (const __nv_bfloat16*)delta;
    auto* yp = (__nv_bfloat16*)y;
    auto* xo = (__nv_bfloat16*)x_out;
#define OB_NORM_FWD(V)                                                                          \
  if (delta != nullptr)                                                                         \
    rmsnorm_fwd_reg_kernel<V, true><<<blocks, threads, 0, stream>>>(xp, dp, w, yp, xo, rstd,    \
                                                                    rows, d, eps);              \
  else                                                                                          \
    rmsnorm_fwd_reg_kernel<V, false><<<blocks, threads, 0, stream>>>(xp, nullptr, w, yp,        \
                                                                     nullptr, rstd, rows, d, eps)
    if (vpl <= 1) { OB_NORM_FWD(1); }
    else if (vpl == 2) { OB_NORM_FWD(2); }
    else if (vpl == 3) { OB_NORM_FWD(3); }
    else { OB_NORM_FWD(4); }
#undef OB_NORM_FWD
    OB_LAUNCH_CHECK();
    return;
  }
  const int blocks = grid_for((int64_t)rows * 32, threads, 8);
  if (delta != nullptr)
    rmsnorm_fwd_kernel<true><<<blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)delta, w, (__nv_bfloat16*)y,
        (__nv_bfloat16*)x_out, rstd, rows, d, eps);
  else
    rmsnorm_fwd_kernel<false><<<blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, nullptr, w, (__nv_bfloat16*)y, nullptr, rstd, rows, d, eps);
  OB_LAUNCH_CHECK();
}

template <int VPL>
void launch_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd,
                        const void* dres, void* dx, float* dw, int rows, int d,
                        cudaStream_t stream) {
  const int threads = 256;
  // Two blocks per SM is what the register budget keeps resident; a larger grid only adds a tail
  // wave and more contention on the weight-gradient atomics (measured: 0.142 ms at 2, 0.149 at 4,
  // 0.180 at 3 blocks per SM for 65536 x 768).
  const int blocks = std::min((rows + 7) / 8, device_sm_count() * 2);
  if (dres != nullptr)
    rmsnorm_bwd_kernel<VPL, true><<<std::max(blocks, 1), threads, d * sizeof(float), stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w, rstd, (const __nv_bfloat16*)dres,
        (__nv_bfloat16*)dx, dw, rows, d);
  else
    rmsnorm_bwd_kernel<VPL, false><<<std::max(blocks, 1), threads, d * sizeof(float), stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w, rstd, nullptr, (__nv_bfloat16*)dx, dw,
        rows, d);
  OB_LAUNCH_CHECK();
}

void rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, const void* dres,
                 void* dx, float* dw, int rows, int d, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "rmsnorm: width must be a multiple of 8");
  OB_CHECK(d <= 8192, "rmsnorm backward supports widths up to 8192");
  const int vpl = (d / 8 + 31) / 32;
  if (vpl <= 1) launch_rmsnorm_bwd<1>(dy, x, w, rstd, dres, dx, dw, rows, d, stream);
  else if (vpl <= 2) launch_rmsnorm_bwd<2>(dy, x, w, rstd, dres, dx, dw, rows, d, stream);
  else if (vpl <= 3) launch_rmsnorm_bwd<3>(dy, x, w, rstd, dres, dx, dw, rows, d, stream);
  else if (vpl <= 4) launch_rmsnorm_bwd<4>(dy, x, w, rstd, dres, dx, dw, rows, d, stream);
  else if (vpl <= 8) launch_rmsnorm_bwd<8>(dy, x, w, rstd, dres, dx, dw, rows, d, stream);
  else if (vpl <= 16) launch_rmsnorm_bwd<16>(dy, x, w, rstd, dres, dx, dw, rows, d, stream);
  else launch_rmsnorm_bwd<32>(dy, x, w, rstd, dres, dx, dw, rows, d, stream);
}

void rope_qk(const void* q, const void* k, void* qo, void* ko, const float* cos_t,
             const float* sin_t, int B, int T, int H, int Hk, int D, bool inverse,
             int64_t q_row_stride, int64_t k_row_stride, int64_t qo_row_stride,
             int64_t ko_row_stride, cudaStream_t stream) {
  OB_CHECK(D % 8 == 0, "rope: head_dim must be a multiple of 8");
  OB_CHECK((int64_t)B * T < (1ll << 31), "rope: too many tokens");
  const int threads = 256;
  const int blocks = grid_for((int64_t)B * T * 32, threads);
  const int vec_per_head = D / 8;
  const bool fixed = vec_per_head <= 32 && (32 % vec_per_head) == 0;
  auto kernel = fixed ? rope_kernel<true> : rope_kernel<false>;
  kernel<<<blocks, threads, 0, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (__nv_bfloat16*)qo, (__nv_bfloat16*)ko,
      cos_t, sin_t, B, T, H, Hk, D, inverse ? -1.f : 1.f, q_row_stride, k_row_stride,
      qo_row_stride, ko_row_stride);
  OB_LAUNCH_CHECK();
}

void swiglu_fwd(const void* g, const void* u, void* a, int64_t rows, int h, int64_t g_pitch,
                int64_t u_pitch, int64_t a_pitch, cudaStream_t stream) {
  OB_CHECK(h % 8 == 0, "swiglu: width must be a multiple of 8");
  const int threads = 256;
  const int tpr = threads_per_row(h >> 3, threads);
  swiglu_fwd_kernel<<<grid_for((rows + 1) / 2 * tpr, threads), threads, 0, stream>>>(
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)a, rows, h, tpr, g_pitch,
      u_pitch, a_pitch);
  OB_LAUNCH_CHECK();
}

void swiglu_bwd(const void* da, const void* g, const void* u, void* dg, void* du, int64_t rows,
                int h, int64_t da_pitch, int64_t g_pitch, int64_t u_pitch, int64_t dg_pitch,
                int64_t du_pitch, cudaStream_t stream) {
  OB_CHECK(h % 8 == 0, "swiglu: width must be a multiple of 8");
  const int threads = 256;
  const int tpr = threads_per_row(h >> 3, threads);
  swiglu_bwd_kernel<<<grid_for(rows * tpr, threads), threads, 0, stream>>>(
      (const __nv_bfloat16*)da, (const __nv_bfloat16*)g, (const __nv_bfloat16*)u,
      (__nv_bfloat16*)dg, (__nv_bfloat16*)du, rows, h, tpr, da_pitch, g_pitch, u_pitch, dg_pitch,
      du_pitch);
  OB_LAUNCH_CHECK();
}

void cast_f32_bf16(const float* in, void* out, int64_t n, cudaStream_t stream, float scale) {
  if (n == 0) return;
  const int threads = 256;
  cast_f32_bf16_kernel<<<grid_for((n + 7) / 8, threads), threads, 0, stream>>>(
      in, (__nv_bfloat16*)out, n, scale);
  OB_LAUNCH_CHECK();
}

void embedding_fwd(const int64_t* ids, const float* table, void* out, int64_t tokens, int d,
                   int vocab, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "embedding: width must be a multiple of 8");
  const int threads = 256;
  embedding_fwd_kernel<<<grid_for(tokens * (d / 8), threads), threads, 0, stream>>>(
      ids, table, (__nv_bfloat16*)out, tokens, d, vocab);
  OB_LAUNCH_CHECK();
}

void embedding_bwd(const int64_t* ids, const void* dout, float* dtable, int64_t tokens, int d,
                   int vocab, cudaStream_t stream) {
  OB_CHECK(d % 8 == 0, "embedding: width must be a multiple of 8");
  const int threads = 256;
  embedding_bwd_kernel<<<grid_for(tokens * (d / 8), threads), threads, 0, stream>>>(
      ids, (const __nv_bfloat16*)dout, dtable, tokens, d, vocab);
  OB_LAUNCH_CHECK();
}

void adamw_step(float* p, const void* g, bool grad_is_bf16, float* m, float* v, void* shadow,
                int64_t n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                float bc2, float grad_scale, cudaStream_t stream) {
  if (n == 0) return;
  const int threads = 256;
  const int blocks = grid_for(n, threads);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        p, (const __nv_bfloat16*)g, m, v, (__nv_bfloat16*)shadow, n, lr, beta1, beta2, eps, wd, bc1,
        bc2, grad_scale);
  else
    adamw_kernel<float><<<blocks, threads, 0, stream>>>(p, (const float*)g, m, v,
                                                        (__nv_bfloat16*)shadow, n, lr, beta1, beta2,
                                                        eps, wd, bc1, bc2, grad_scale);
  OB_LAUNCH_CHECK();
}

}  // namespace ob
