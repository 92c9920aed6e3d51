// Python bindings: thin, checked wrappers that take torch tensors, launch on the current stream and
// never synchronise. Kernel launchers themselves are torch-free (raw pointers + geometry).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"

// cpu_scan.cpp: the linear recurrence on host tensors
namespace ob_cpu {
torch::Tensor pscan_cpu_fwd(const torch::Tensor& a, const torch::Tensor& x);
std::vector<torch::Tensor> pscan_cpu_bwd(const torch::Tensor& a, const torch::Tensor& h,
                                         const torch::Tensor& dh);
}  // namespace ob_cpu

namespace {

using torch::Tensor;

cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}
void check_bf16(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bfloat16");
}
void check_f32(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, " must be float32");
}
void check_rowmajor(const Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() >= 2 && t.stride(-1) == 1, name, " must have a contiguous last dimension");
}

// c[b] = alpha * op(a[b]) * op(b[b])^T with the conventions of ob::gemm_bf16. `a`, `b` are the
// *stored* matrices: (rows, inner) or (batch, rows, inner) with unit inner stride.
void gemm(const Tensor& a, const Tensor& b, Tensor& c, int64_t M, int64_t N, int64_t K, bool a_mn,
          bool b_mn, int64_t splits, bool reduce, double alpha,
          const c10::optional<Tensor>& m_tile_batch, const c10::optional<Tensor>& k_offsets,
          const c10::optional<Tensor>& residual, double beta, int64_t m_tile_rows) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  check_cuda(c, "c");
  check_rowmajor(a, "a");
  check_rowmajor(b, "b");
  check_rowmajor(c, "c");
  const bool out_f32 = c.scalar_type() == torch::kFloat32;
  TORCH_CHECK(out_f32 || c.scalar_type() == torch::kBFloat16, "c must be bf16 or fp32");
  const c10::cuda::CUDAGuard guard(a.device());
  const bool a_batched = a.dim() == 3;
  const bool b_batched = b.dim() == 3;
  const bool c_batched = c.dim() == 3;
  const int64_t batches = c_batched ? c.size(0) : 1;
  if (a_batched) TORCH_CHECK(a.size(0) == batches, "a batch count mismatch");
  const int64_t b_batches = b_batched ? b.size(0) : 1;
  if (b_batched && !m_tile_batch.has_value())
    TORCH_CHECK(b_batches == batches, "b batch count mismatch");
  TORCH_CHECK(c.size(-2) == M && c.size(-1) == N, "c has the wrong shape");
  const int64_t a_rows = a.size(-2), b_rows = b.size(-2);
  if (!k_offsets.has_value()) {
    TORCH_CHECK(a_mn ? (a_rows == K && a.size(-1) == M) : (a_rows == M && a.size(-1) == K),
                "a does not match (M, K) with the requested major");
    TORCH_CHECK(b_mn ? (b_rows == K && b.size(-1) == N) : (b_rows == N && b.size(-1) == K),
                "b does not match (N, K) with the requested major");
  }
  auto aligned = [](const Tensor& t) {
    bool ok = (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0);
    for (int i = 0; i + 1 < t.dim(); ++i) ok = ok && ((t.stride(i) * t.element_size()) % 16 == 0);
    return ok;
  };
  TORCH_CHECK(aligned(a) && aligned(b) && aligned(c),
              "gemm operands need 16-byte aligned base addresses and row pitches");
  const int* mtb = nullptr;
  const int* koff = nullptr;
  if (m_tile_batch.has_value()) {
    TORCH_CHECK(m_tile_batch->scalar_type() == torch::kInt32 && m_tile_batch->is_cuda());
    TORCH_CHECK(m_tile_rows >= 128 && m_tile_rows % 128 == 0, "m_tile_rows must be a multiple of 128");
    TORCH_CHECK(m_tile_batch->numel() >= (M + m_tile_rows - 1) / m_tile_rows, "m_tile_batch is too short");
    mtb = m_tile_batch->data_ptr<int>();
  }
  if (k_offsets.has_value()) {
    TORCH_CHECK(k_offsets->scalar_type() == torch::kInt32 && k_offsets->is_cuda());
    TORCH_CHECK(k_offsets->numel() >= batches + 1, "k_offsets is too short");
    koff = k_offsets->data_ptr<int>();
  }
  const void* res_ptr = nullptr;
  int64_t ldr = 0, stride_r = 0;
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    check_rowmajor(*residual, "residual");
    TORCH_CHECK(residual->dim() == c.dim() && residual->size(-2) == M && residual->size(-1) == N,
                "residual must have the shape of c");
    TORCH_CHECK(!c_batched || residual->size(0) == batches, "residual batch count mismatch");
    res_ptr = residual->data_ptr();
    ldr = residual->stride(-2);
    stride_r = c_batched ? residual->stride(0) : 0;
  }
  ob::gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, (int)batches,
                a_mn, b_mn, a.stride(-2), b.stride(-2), c.stride(-2), a_batched ? a.stride(0) : 0,
                b_batched ? b.stride(0) : 0, c_batched ? c.stride(0) : 0, a_batched, b_batched,
                (int)b_batches, out_f32, (int)splits, reduce, (float)alpha, mtb, koff, a_rows,
                b_rows, ob::device_sm_count(), res_ptr, ldr, stride_r, (float)beta, current_stream(),
                (int)m_tile_rows);
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& delta, const Tensor& w,
                                double eps) {
  check_bf16(x, "x");
  check_f32(w, "weight");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t d = x.size(-1);
  const int64_t rows = x.numel() / d;
  TORCH_CHECK(w.numel() == d, "weight width mismatch");
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  Tensor x_out;
  const void* dptr = nullptr;
  void* xo = nullptr;
  if (delta.has_value()) {
    check_bf16(*delta, "delta");
    TORCH_CHECK(delta->is_contiguous() && delta->numel() == x.numel());
    x_out = torch::empty_like(x);
    dptr = delta->data_ptr();
    xo = x_out.data_ptr();
  }
  ob::rmsnorm_fwd(x.data_ptr(), dptr, w.data_ptr<float>(), y.data_ptr(), xo, rstd.data_ptr<float>(),
                  (int)rows, (int)d, (float)eps, current_stream());
  if (delta.has_value()) return {y, rstd, x_out};
  return {y, rstd};
}

std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w,
                                const Tensor& rstd, const c10::optional<Tensor>& dres) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  check_f32(w, "weight");
  check_f32(rstd, "rstd");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t d = x.size(-1);
  const int64_t rows = x.numel() / d;
  Tensor dx = torch::empty_like(x);
  Tensor dw = torch::zeros({d}, x.options().dtype(torch::kFloat32));
  const void* dr = nullptr;
  if (dres.has_value()) {
    check_bf16(*dres, "dres");
    TORCH_CHECK(dres->is_contiguous() && dres->numel() == x.numel());
    dr = dres->data_ptr();
  }
  ob::rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr<float>(), rstd.data_ptr<float>(), dr,
                  dx.data_ptr(), dw.data_ptr<float>(), (int)rows, (int)d, current_stream());
  return {dx, dw};
}

// q: (B, T, H, D), k: (B, T, Hk, D) with contiguous (H, D); row (token) stride may exceed H*D.
// Rotates q and k. Without `q_out` / `k_out` fresh contiguous tensors are returned; with them the
// results are written there (they may be column slices of a wider buffer, e.g. the gradient of a
// fused q|k|v projection).
std::vector<Tensor> rope(const Tensor& q, const Tensor& k, const Tensor& cos_t, const Tensor& sin_t,
                         bool inverse, const c10::optional<Tensor>& q_out,
                         const c10::optional<Tensor>& k_out) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_f32(cos_t, "cos");
  check_f32(sin_t, "sin");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4);
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), Hk = k.size(2);
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(0) >= T &&
                  cos_t.size(1) * 2 == D,
              "rope tables must be (>=T, D/2) fp32");
  auto token_strided = [&](const Tensor& t, int64_t heads) {
    return t.stride(3) == 1 && t.stride(2) == D && t.stride(0) == t.stride(1) * T &&
           t.stride(1) >= heads * D && (t.stride(1) % 8 == 0) &&
           (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0);
  };
  Tensor qq = token_strided(q, H) ? q : q.contiguous();
  Tensor kk = token_strided(k, Hk) ? k : k.contiguous();
  Tensor qo = q_out.has_value() ? *q_out : torch::empty({B, T, H, D}, q.options());
  Tensor ko = k_out.has_value() ? *k_out : torch::empty({B, T, Hk, D}, k.options());
  check_bf16(qo, "q_out");
  check_bf16(ko, "k_out");
  TORCH_CHECK(qo.dim() == 4 && ko.dim() == 4 && qo.sizes() == q.sizes() && ko.sizes() == k.sizes() &&
                  token_strided(qo, H) && token_strided(ko, Hk),
              "rope outputs must be (B, T, heads, D) with a constant token stride");
  ob::rope_qk(qq.data_ptr(), kk.data_ptr(), qo.data_ptr(), ko.data_ptr(), cos_t.data_ptr<float>(),
              sin_t.data_ptr<float>(), (int)B, (int)T, (int)H, (int)Hk, (int)D, inverse,
              qq.stride(1), kk.stride(1), qo.stride(1), ko.stride(1), current_stream());
  return {qo, ko};
}

bool pitched_2d(const Tensor& t) {
  return t.dim() == 2 && t.stride(1) == 1 && (t.stride(0) % 8 == 0) &&
         (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0);
}

Tensor swiglu_fwd(const Tensor& g, const Tensor& u) {
  check_bf16(g, "gate");
  check_bf16(u, "up");
  TORCH_CHECK(pitched_2d(g) && pitched_2d(u) && g.sizes() == u.sizes(),
              "swiglu expects 2-D bf16 operands with 16-byte aligned rows");
  const c10::cuda::CUDAGuard guard(g.device());
  Tensor a = torch::empty({g.size(0), g.size(1)}, g.options());
  ob::swiglu_fwd(g.data_ptr(), u.data_ptr(), a.data_ptr(), g.size(0), (int)g.size(1), g.stride(0),
                 u.stride(0), a.stride(0), current_stream());
  return a;
}

// Writes the two gradients into `dg` and `du`, which may be column slices of one buffer.
void swiglu_bwd(const Tensor& da, const Tensor& g, const Tensor& u, Tensor& dg, Tensor& du) {
  check_bf16(da, "da");
  check_bf16(g, "gate");
  check_bf16(u, "up");
  check_bf16(dg, "dg");
  check_bf16(du, "du");
  TORCH_CHECK(pitched_2d(da) && pitched_2d(g) && pitched_2d(u) && pitched_2d(dg) && pitched_2d(du));
  TORCH_CHECK(da.sizes() == g.sizes() && g.sizes() == u.sizes() && dg.sizes() == g.sizes() &&
              du.sizes() == g.sizes());
  const c10::cuda::CUDAGuard guard(g.device());
  ob::swiglu_bwd(da.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(), g.size(0),
                 (int)g.size(1), da.stride(0), g.stride(0), u.stride(0), dg.stride(0), du.stride(0),
                 current_stream());
}

void cast_bf16_into(const Tensor& src, Tensor& dst) {
  check_f32(src, "src");
  check_bf16(dst, "dst");
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel());
  const c10::cuda::CUDAGuard guard(src.device());
  ob::cast_f32_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), current_stream());
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& table) {
  check_cuda(ids, "ids");
  check_f32(table, "table");
  TORCH_CHECK(ids.scalar_type() == torch::kInt64 && ids.is_contiguous() && table.is_contiguous());
  const c10::cuda::CUDAGuard guard(table.device());
  auto shape = ids.sizes().vec();
  shape.push_back(table.size(1));
  Tensor out = torch::empty(shape, table.options().dtype(torch::kBFloat16));
  ob::embedding_fwd(ids.data_ptr<int64_t>(), table.data_ptr<float>(), out.data_ptr(), ids.numel(),
                    (int)table.size(1), (int)table.size(0), current_stream());
  return out;
}

void embedding_bwd(const Tensor& ids, const Tensor& dout, Tensor& dtable) {
  check_cuda(ids, "ids");
  check_bf16(dout, "dout");
  check_f32(dtable, "dtable");
  TORCH_CHECK(ids.is_contiguous() && dout.is_contiguous() && dtable.is_contiguous());
  const c10::cuda::CUDAGuard guard(dtable.device());
  ob::embedding_bwd(ids.data_ptr<int64_t>(), dout.data_ptr(), dtable.data_ptr<float>(), ids.numel(),
                    (int)dtable.size(1), (int)dtable.size(0), current_stream());
}

void adamw_step(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const c10::optional<Tensor>& shadow,
                double lr, double beta1, double beta2, double eps, double wd, int64_t step,
                double grad_scale) {
  check_f32(p, "param");
  check_f32(m, "exp_avg");
  check_f32(v, "exp_avg_sq");
  check_cuda(g, "grad");
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel());
  const bool g_bf16 = g.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(g_bf16 || g.scalar_type() == torch::kFloat32, "grad must be bf16 or fp32");
  void* sh = nullptr;
  if (shadow.has_value()) {
    check_bf16(*shadow, "shadow");
    TORCH_CHECK(shadow->is_contiguous() && shadow->numel() == p.numel());
    sh = shadow->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(p.device());
  const double bc1 = 1.0 - std::pow(beta1, (double)step);
  const double bc2 = 1.0 - std::pow(beta2, (double)step);
  ob::adamw_step(p.data_ptr<float>(), g.data_ptr(), g_bf16, m.data_ptr<float>(), v.data_ptr<float>(),
                 sh, p.numel(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd,
                 (float)bc1, (float)bc2, (float)grad_scale, current_stream());
}

// logits (rows, vocab) bf16 with pitch >= vocab; turned into gradients in place when write_grad.
std::vector<Tensor> cross_entropy_rows(Tensor& logits, const Tensor& targets,
                                       const c10::optional<Tensor>& scale, int64_t ignore_index,
                                       bool write_grad, bool want_correct) {
  check_bf16(logits, "logits");
  check_cuda(targets, "targets");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(targets.scalar_type() == torch::kInt64 && targets.is_contiguous() &&
              targets.numel() == logits.size(0));
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t rows = logits.size(0);
  auto fopt = logits.options().dtype(torch::kFloat32);
  Tensor loss = torch::empty({rows}, fopt);
  Tensor lse = torch::empty({rows}, fopt);
  Tensor correct;
  int* cptr = nullptr;
  if (want_correct) {
    correct = torch::empty({rows}, logits.options().dtype(torch::kInt32));
    cptr = correct.data_ptr<int>();
  }
  const float* sptr = nullptr;
  if (scale.has_value()) {
    check_f32(*scale, "scale");
    sptr = scale->data_ptr<float>();
  }
  ob::cross_entropy_rows(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(),
                         lse.data_ptr<float>(), cptr, sptr, rows, (int)logits.size(1),
                         logits.stride(0), ignore_index, write_grad, current_stream());
  if (want_correct) return {loss, lse, correct};
  return {loss, lse};
}

void scale_by_scalar(Tensor& x, const Tensor& scalar) {
  check_cuda(x, "x");
  check_f32(scalar, "scalar");
  TORCH_CHECK(x.is_contiguous() && scalar.numel() == 1);
  const bool bf16 = x.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(bf16 || x.scalar_type() == torch::kFloat32);
  const c10::cuda::CUDAGuard guard(x.device());
  ob::scale_by_scalar(x.data_ptr(), bf16, scalar.data_ptr<float>(), x.numel(), current_stream());
}

// (B, T, H, D) tensors whose (heads, D) block is contiguous; token and batch strides are free.
bool attn_layout_ok(const Tensor& t) {
  return t.dim() == 4 && t.stride(3) == 1 && t.stride(2) == t.size(3) &&
         (t.stride(1) * 2) % 16 == 0 && (t.stride(0) * 2) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0;
}

std::vector<Tensor> flash_attn_fwd(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in,
                                   bool causal, double scale) {
  check_bf16(q_in, "q");
  check_bf16(k_in, "k");
  check_bf16(v_in, "v");
  Tensor q = attn_layout_ok(q_in) ? q_in : q_in.contiguous();
  Tensor k = attn_layout_ok(k_in) ? k_in : k_in.contiguous();
  Tensor v = attn_layout_ok(v_in) ? v_in : v_in.contiguous();
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3);
  const int64_t S = k.size(1), Hk = k.size(2);
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && k.size(3) == D && v.sizes() == k.sizes(),
              "attention operand shapes do not match");
  Tensor o = torch::empty({B, T, H, D}, q.options());
  Tensor lse = torch::empty({B, H, T}, q.options().dtype(torch::kFloat32));
  ob::flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                     (int)B, (int)T, (int)S, (int)H, (int)Hk, (int)D, causal, (float)scale,
                     q.stride(1), k.stride(1), v.stride(1), q.stride(0), k.stride(0), v.stride(0),
                     current_stream());
  return {o, lse};
}

// With `dk_out` / `dv_out` the key / value gradients are written there (bf16 (B, S, Hk, D) whose
// (heads, D) block is contiguous: column slices of a wider buffer are fine).
std::vector<Tensor> flash_attn_bwd(const Tensor& dout_in, const Tensor& q_in, const Tensor& k_in,
                                   const Tensor& v_in, const Tensor& out, const Tensor& lse,
                                   bool causal, double scale, const c10::optional<Tensor>& dk_out,
                                   const c10::optional<Tensor>& dv_out) {
  check_bf16(dout_in, "dout");
  check_bf16(out, "out");
  check_f32(lse, "lse");
  Tensor q = attn_layout_ok(q_in) ? q_in : q_in.contiguous();
  Tensor k = attn_layout_ok(k_in) ? k_in : k_in.contiguous();
  Tensor v = attn_layout_ok(v_in) ? v_in : v_in.contiguous();
  Tensor d_o = attn_layout_ok(dout_in) ? dout_in : dout_in.contiguous();
  TORCH_CHECK(out.is_contiguous() && lse.is_contiguous());
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3);
  const int64_t S = k.size(1), Hk = k.size(2);
  Tensor delta = torch::empty({B, H, T}, lse.options());
  ob::attn_delta(out.data_ptr(), d_o.data_ptr(), delta.data_ptr<float>(), (int)B, (int)T, (int)H,
                 (int)D, d_o.stride(1), d_o.stride(0), current_stream());
  Tensor dq32 = torch::zeros({B, T, H, D}, q.options().dtype(torch::kFloat32));
  Tensor dk = dk_out.has_value() ? *dk_out : torch::empty({B, S, Hk, D}, k.options());
  Tensor dv = dv_out.has_value() ? *dv_out : torch::empty({B, S, Hk, D}, k.options());
  check_bf16(dk, "dk");
  check_bf16(dv, "dv");
  TORCH_CHECK(attn_layout_ok(dk) && attn_layout_ok(dv) && dk.sizes() == k.sizes() &&
                  dv.sizes() == k.sizes(),
              "dk / dv must be (B, S, Hk, D) bf16 with contiguous (heads, D) blocks");
  const int64_t strides[12] = {q.stride(1), q.stride(0), k.stride(1), k.stride(0),
                               v.stride(1), v.stride(0), d_o.stride(1), d_o.stride(0),
                               dk.stride(1), dk.stride(0), dv.stride(1), dv.stride(0)};
  ob::flash_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr(),
                     dq32.data_ptr<float>(), dk.data_ptr(), dv.data_ptr(), lse.data_ptr<float>(),
                     delta.data_ptr<float>(), (int)B, (int)T, (int)S, (int)H, (int)Hk, (int)D,
                     causal, (float)scale, strides, current_stream());
  Tensor dq = torch::empty({B, T, H, D}, q.options());
  ob::cast_f32_bf16(dq32.data_ptr<float>(), dq.data_ptr(), dq32.numel(), current_stream(),
                    (float)scale);
  return {dq, dk, dv};
}

// ---- Muon stages --------------------------------------------------------------------------------
ob::MuonTable muon_table(const std::vector<Tensor>& tensors, bool bf16) {
  TORCH_CHECK(!tensors.empty() && tensors.size() <= (size_t)ob::kMuonMaxPointers,
              "a Muon group takes 1..", ob::kMuonMaxPointers, " tensors here");
  ob::MuonTable table = {};
  for (size_t i = 0; i < tensors.size(); ++i) {
    const Tensor& t = tensors[i];
    TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.sizes() == tensors[0].sizes());
    TORCH_CHECK(t.scalar_type() == (bf16 ? torch::kBFloat16 : torch::kFloat32));
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, "Muon tensors must be 16-byte aligned");
    table.ptr[i] = t.data_ptr();
  }
  return table;
}

// momentum (B, r, c) fp32 updated in place; returns nothing: `u` (B, r, c) bf16 receives the
// normalised Nesterov direction, ready for the Newton-Schulz iteration.
void muon_prepare(const std::vector<Tensor>& grads, Tensor& momentum, Tensor& u, Tensor& norm2,
                  double mu) {
  check_f32(momentum, "momentum");
  check_bf16(u, "u");
  check_f32(norm2, "norm2");
  TORCH_CHECK(momentum.is_contiguous() && u.is_contiguous() && momentum.dim() == 3 &&
              u.sizes() == momentum.sizes());
  const c10::cuda::CUDAGuard guard(momentum.device());
  const int64_t batch = momentum.size(0), numel = momentum.size(1) * momentum.size(2);
  const int per_pointer = (int)(batch / (int64_t)grads.size());
  TORCH_CHECK((int64_t)grads.size() * per_pointer == batch && grads[0].numel() == per_pointer * numel);
  TORCH_CHECK(norm2.numel() == batch);
  const ob::MuonTable table = muon_table(grads, false);
  ob::muon_momentum(table, momentum.data_ptr<float>(), u.data_ptr(), norm2.data_ptr<float>(),
                    (int)batch, numel, (float)mu, per_pointer, current_stream());
  ob::muon_scale(u.data_ptr(), norm2.data_ptr<float>(), (int)batch, numel, current_stream());
}

Tensor muon_variance(const Tensor& x, bool by_row) {
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && x.dim() == 3);
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t batch = x.size(0), rows = x.size(1), cols = x.size(2);
  Tensor v = torch::empty({batch, by_row ? rows : 1, by_row ? 1 : cols},
                          x.options().dtype(torch::kFloat32));
  ob::muon_variance(x.data_ptr(), v.data_ptr<float>(), (int)batch, (int)rows, (int)cols, by_row,
                    current_stream());
  return v;
}

void muon_apply(const std::vector<Tensor>& params, const std::vector<Tensor>& shadows,
                const Tensor& x, const Tensor& factor, double lr, double wd, bool by_row) {
  check_bf16(x, "x");
  check_f32(factor, "factor");
  TORCH_CHECK(x.is_contiguous() && x.dim() == 3 && factor.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t batch = x.size(0), rows = x.size(1), cols = x.size(2);
  const int per_pointer = (int)(batch / (int64_t)params.size());
  TORCH_CHECK((int64_t)params.size() * per_pointer == batch &&
              params[0].numel() == per_pointer * rows * cols);
  TORCH_CHECK(factor.numel() == batch * (by_row ? rows : cols));
  const ob::MuonTable ptable = muon_table(params, false);
  ob::MuonTable stable = {};
  const bool has_shadow = !shadows.empty();
  if (has_shadow) {
    TORCH_CHECK(shadows.size() == params.size());
    stable = muon_table(shadows, true);
  }
  ob::muon_apply(ptable, has_shadow ? &stable : nullptr, x.data_ptr(), factor.data_ptr<float>(),
                 (int)batch, (int)rows, (int)cols, (float)lr, (float)wd, by_row, per_pointer,
                 current_stream());
}

// ---- linear recurrence scan ------------------------------------------------------------------------
Tensor pscan_fwd(const Tensor& a, const Tensor& x) {
  check_f32(a, "a");
  check_f32(x, "x");
  TORCH_CHECK(a.is_contiguous() && x.is_contiguous() && a.sizes() == x.sizes() && a.dim() >= 2,
              "pscan: contiguous (B, L, ...) tensors of equal shape");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor h = torch::empty_like(a);
  const int64_t batch = a.size(0), length = a.size(1);
  const int64_t channels = batch * length == 0 ? 0 : a.numel() / (batch * length);
  ob::pscan_forward(a.data_ptr<float>(), x.data_ptr<float>(), h.data_ptr<float>(), batch,
                    (int)length, channels, current_stream());
  return h;
}

std::vector<Tensor> pscan_bwd(const Tensor& a, const Tensor& h, const Tensor& dh) {
  check_f32(a, "a");
  check_f32(h, "h");
  check_f32(dh, "dh");
  TORCH_CHECK(a.is_contiguous() && h.is_contiguous() && dh.is_contiguous() &&
                  a.sizes() == h.sizes() && a.sizes() == dh.sizes() && a.dim() >= 2,
              "pscan: contiguous (B, L, ...) tensors of equal shape");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor da = torch::empty_like(a), dx = torch::empty_like(a);
  const int64_t batch = a.size(0), length = a.size(1);
  const int64_t channels = batch * length == 0 ? 0 : a.numel() / (batch * length);
  ob::pscan_backward(a.data_ptr<float>(), h.data_ptr<float>(), dh.data_ptr<float>(),
                     da.data_ptr<float>(), dx.data_ptr<float>(), batch, (int)length, channels,
                     current_stream());
  return {da, dx};
}

// ---- Sinkhorn -----------------------------------------------------------------------------------
Tensor sinkhorn_fwd(const Tensor& x, int64_t iters) {
  check_f32(x, "log_alpha");
  TORCH_CHECK(x.is_contiguous() && x.dim() >= 2 && x.size(-1) == x.size(-2));
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t n = x.size(-1);
  Tensor out = torch::empty_like(x);
  ob::sinkhorn_forward(x.data_ptr<float>(), out.data_ptr<float>(), x.numel() / (n * n), (int)n,
                       (int)iters, current_stream());
  return out;
}

Tensor sinkhorn_bwd(const Tensor& x, const Tensor& grad_out, int64_t iters) {
  check_f32(x, "log_alpha");
  check_f32(grad_out, "grad_out");
  TORCH_CHECK(x.is_contiguous() && grad_out.is_contiguous() && x.sizes() == grad_out.sizes());
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t n = x.size(-1);
  Tensor grad_in = torch::empty_like(x);
  const int64_t count = x.numel() / (n * n);
  const int64_t tape_floats = ob::sinkhorn_tape_floats((int)n, (int)iters);
  Tensor tape;
  if (tape_floats > 0) tape = torch::empty({count, tape_floats}, x.options());
  ob::sinkhorn_backward(x.data_ptr<float>(), grad_out.data_ptr<float>(), grad_in.data_ptr<float>(),
                        tape_floats > 0 ? tape.data_ptr<float>() : nullptr, count, (int)n,
                        (int)iters, current_stream());
  return grad_in;
}

bool sinkhorn_supported(int64_t n, int64_t iters) {
  return ob::sinkhorn_supported((int)n, (int)iters);
}

// ---- multicast reduction --------------------------------------------------------------------------
// out <- scale * sum over the ranks of the bytes at `multicast_ptr` (the multicast address of a
// symmetric buffer every rank has filled and fenced with a barrier before this call).
void multimem_sum(int64_t multicast_ptr, Tensor& out, double scale) {
  check_cuda(out, "out");
  const bool bf16 = out.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(bf16 || out.scalar_type() == torch::kFloat32, "out must be bfloat16 or float32");
  TORCH_CHECK(out.is_contiguous(), "out must be contiguous");
  TORCH_CHECK(multicast_ptr != 0, "no multicast address: the devices do not support multicast");
  const c10::cuda::CUDAGuard guard(out.device());
  ob::multimem_sum(reinterpret_cast<const void*>(multicast_ptr), out.data_ptr(),
                   out.numel() * out.element_size(), bf16, (float)scale, current_stream());
}

// ---- BitNet quantisers ---------------------------------------------------------------------------
// (q, dequant, rstd) of a 2-D bf16 tensor; `norm_weight` (fp32, width) fuses the RMS norm in, and
// rstd is then the per-row 1 / rms (an empty tensor otherwise).
std::vector<Tensor> bitnet_act_quant(const Tensor& x, const c10::optional<Tensor>& norm_weight,
                                     double eps) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(1) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0,
              "act_quant expects a contiguous, 16-byte aligned (rows, width % 8 == 0) tensor");
  TORCH_CHECK(x.size(0) < (1ll << 31), "act_quant: too many rows");
  const c10::cuda::CUDAGuard guard(x.device());
  const float* w = nullptr;
  if (norm_weight.has_value()) {
    check_f32(*norm_weight, "norm_weight");
    TORCH_CHECK(norm_weight->is_contiguous() && norm_weight->numel() == x.size(1) &&
                    reinterpret_cast<uintptr_t>(norm_weight->data_ptr()) % 16 == 0,
                "norm_weight must be a contiguous, 16-byte aligned vector of the row width");
    w = norm_weight->data_ptr<float>();
  }
  Tensor q = torch::empty_like(x);
  Tensor dequant = torch::empty({x.size(0)}, x.options().dtype(torch::kFloat32));
  Tensor rstd = torch::empty({w != nullptr ? x.size(0) : 0}, dequant.options());
  ob::bitnet_act_quant(x.data_ptr(), w, q.data_ptr(), dequant.data_ptr<float>(),
                       w != nullptr ? rstd.data_ptr<float>() : nullptr, (int)x.size(0),
                       (int)x.size(1), (float)eps, current_stream());
  return {q, dequant, rstd};
}

// (ternary bf16 of w's shape, scale (1,) fp32) of a contiguous fp32 or bf16 weight.
std::vector<Tensor> bitnet_weight_quant(const Tensor& w) {
  check_cuda(w, "w");
  const bool f32 = w.scalar_type() == torch::kFloat32;
  TORCH_CHECK(f32 || w.scalar_type() == torch::kBFloat16, "w must be float32 or bfloat16");
  TORCH_CHECK(w.is_contiguous(), "w must be contiguous");
  const c10::cuda::CUDAGuard guard(w.device());
  Tensor ternary = torch::empty(w.sizes(), w.options().dtype(torch::kBFloat16));
  Tensor scale = torch::empty({1}, w.options().dtype(torch::kFloat32));
  Tensor partials = torch::empty({ob::bitnet_partial_count()}, scale.options());
  ob::bitnet_weight_quant(w.data_ptr(), f32, w.numel(), ternary.data_ptr(), scale.data_ptr<float>(),
                          partials.data_ptr<float>(), current_stream());
  return {ternary, scale};
}

Tensor bitnet_scale_rows(const Tensor& acc, const Tensor& row_factor, const Tensor& weight_scale,
                         const c10::optional<Tensor>& bias) {
  check_f32(acc, "acc");
  check_f32(row_factor, "row_factor");
  check_f32(weight_scale, "weight_scale");
  TORCH_CHECK(acc.dim() == 2 && acc.is_contiguous() && acc.size(1) % 4 == 0 &&
                  reinterpret_cast<uintptr_t>(acc.data_ptr()) % 16 == 0,
              "scale_rows expects a contiguous, 16-byte aligned (rows, width % 4 == 0) tensor");
  TORCH_CHECK(row_factor.is_contiguous() && row_factor.numel() == acc.size(0) &&
                  weight_scale.numel() == 1,
              "one factor per row and one weight scale expected");
  const c10::cuda::CUDAGuard guard(acc.device());
  const float* b = nullptr;
  if (bias.has_value()) {
    check_f32(*bias, "bias");
    TORCH_CHECK(bias->is_contiguous() && bias->numel() == acc.size(1) &&
                    reinterpret_cast<uintptr_t>(bias->data_ptr()) % 16 == 0,
                "bias must be a contiguous, 16-byte aligned vector of the row width");
    b = bias->data_ptr<float>();
  }
  Tensor out = torch::empty(acc.sizes(), acc.options().dtype(torch::kBFloat16));
  ob::bitnet_scale_rows(acc.data_ptr<float>(), row_factor.data_ptr<float>(),
                        weight_scale.data_ptr<float>(), b, out.data_ptr(), acc.size(0),
                        (int)acc.size(1), current_stream());
  return out;
}

// ---- peer memory ---------------------------------------------------------------------------------
// Allocates `bytes` of device memory outside the caching allocator and returns (tensor view as
// uint8, IPC handle bytes). The memory lives until peer_free(tensor.data_ptr()).
std::pair<Tensor, py::bytes> peer_alloc(int64_t bytes, int64_t device_index) {
  const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index));
  char handle[64];
  void* ptr = ob::peer_alloc((size_t)bytes, handle);
  auto options = torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, device_index);
  Tensor view = torch::from_blob(ptr, {bytes}, options);
  return {view, py::bytes(handle, 64)};
}

// Opens a peer's handle; returns a uint8 view of the peer's memory addressable from this device.
Tensor peer_open(const std::string& handle, int64_t bytes, int64_t device_index) {
  TORCH_CHECK(handle.size() == 64, "IPC handle must be 64 bytes");
  const c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_index));
  void* ptr = ob::peer_open(handle.data());
  auto options = torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, device_index);
  return torch::from_blob(ptr, {bytes}, options);
}

void peer_close(int64_t ptr) { ob::peer_close(reinterpret_cast<void*>(ptr)); }
void peer_free(int64_t ptr) { ob::peer_free(reinterpret_cast<void*>(ptr)); }

void peer_barrier(const std::vector<int64_t>& pads, int64_t rank, int64_t epoch, double limit_s) {
  ob::peer_barrier_launch(pads.data(), (int)rank, (int)pads.size(), (uint32_t)epoch,
                          (uint64_t)(limit_s * 1e9), current_stream());
}

void peer_reduce_scatter_mean(const std::vector<int64_t>& grads, const std::vector<int64_t>& pads,
                              Tensor& out, int64_t region, int64_t rank, int64_t epoch,
                              double limit_s) {
  check_f32(out, "out");
  TORCH_CHECK(out.is_contiguous() && out.numel() >= region && grads.size() == pads.size());
  const c10::cuda::CUDAGuard guard(out.device());
  ob::peer_reduce_scatter_mean(grads.data(), pads.data(), out.data_ptr<float>(), region, (int)rank,
                               (int)grads.size(), (uint32_t)epoch, (uint64_t)(limit_s * 1e9),
                               current_stream());
}

void peer_all_gather(const std::vector<int64_t>& weights, const std::vector<int64_t>& pads,
                     int64_t region_bytes, int64_t rank, int64_t epoch, double limit_s) {
  TORCH_CHECK(weights.size() == pads.size());
  ob::peer_all_gather(weights.data(), pads.data(), region_bytes, (int)rank, (int)weights.size(),
                      (uint32_t)epoch, (uint64_t)(limit_s * 1e9), current_stream());
}

// y (M, N) = x (M, K) @ w (N, K)^T for at most 16 rows (decode); returns false when the shape is not
// supported and nothing was launched.
bool gemv(const Tensor& x, const Tensor& w, Tensor& y) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  check_bf16(y, "y");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && y.dim() == 2 && x.size(1) == w.size(1) &&
              y.size(0) == x.size(0) && y.size(1) == w.size(0));
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1);
  const int64_t M = x.size(0), N = w.size(0), K = x.size(1);
  auto aligned = [](const Tensor& t) {
    return reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && (t.stride(0) * 2) % 16 == 0;
  };
  if (!ob::gemv_supported((int)M, (int)N, (int)K) || !aligned(x) || !aligned(w)) return false;
  const c10::cuda::CUDAGuard guard(x.device());
  ob::gemv_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), (int)M, (int)N, (int)K, x.stride(0),
                w.stride(0), y.stride(0), current_stream());
  return true;
}

// -- mixture of experts ---------------------------------------------------------------------------
void check_i32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous(), name,
              " must be a contiguous int32 CUDA tensor");
}

// logits (N, E) fp32 -> indices (N, k) int32, weights (N, k) fp32, alpha (N) fp32 (empty when not
// requested), counts (E) int32 (accumulated into; the caller zeroes it).
std::vector<Tensor> route_topk(const Tensor& logits, const c10::optional<Tensor>& bias, int64_t k,
                               bool sigmoid_gate, bool normalize, bool want_alpha, Tensor& counts) {
  check_f32(logits, "logits");
  check_i32(counts, "counts");
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous());
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t n = logits.size(0), e = logits.size(1);
  TORCH_CHECK(counts.numel() == e, "counts must have one entry per expert");
  const float* bias_ptr = nullptr;
  if (bias.has_value()) {
    check_f32(*bias, "bias");
    TORCH_CHECK(bias->numel() == e && bias->is_contiguous());
    bias_ptr = bias->data_ptr<float>();
  }
  Tensor indices = torch::empty({n, k}, logits.options().dtype(torch::kInt32));
  Tensor weights = torch::empty({n, k}, logits.options());
  Tensor alpha = torch::empty({want_alpha ? n : 0}, logits.options());
  ob::route_topk(logits.data_ptr<float>(), bias_ptr, indices.data_ptr<int>(),
                 weights.data_ptr<float>(), want_alpha ? alpha.data_ptr<float>() : nullptr,
                 counts.data_ptr<int>(), (int)n, (int)e, (int)k, sigmoid_gate, normalize, want_alpha,
                 current_stream());
  return {indices, weights, alpha};
}

// indices (N, k) int32 + counts (E) -> dest_row (N*k), row_pair (padded_rows, -1 on padding rows),
// tile_expert (padded_rows / tile), k_offsets (E + 1). padded_rows is a static upper bound.
std::vector<Tensor> moe_plan(const Tensor& indices, const Tensor& counts, int64_t tile) {
  check_i32(indices, "indices");
  check_i32(counts, "counts");
  const c10::cuda::CUDAGuard guard(indices.device());
  const int64_t pairs = indices.numel(), experts = counts.numel();
  const int64_t padded_rows = (pairs + experts * (tile - 1)) / tile * tile + tile;
  const int64_t num_tiles = padded_rows / tile;
  auto opts = indices.options();
  Tensor dest_row = torch::empty({pairs}, opts);
  Tensor row_pair = torch::full({padded_rows}, -1, opts);
  Tensor tile_expert = torch::empty({num_tiles}, opts);
  Tensor k_offsets = torch::empty({experts + 1}, opts);
  Tensor scratch = torch::empty({2 * experts}, opts);  // segment starts, placement cursors
  ob::moe_plan(indices.data_ptr<int>(), counts.data_ptr<int>(), scratch.data_ptr<int>(),
               k_offsets.data_ptr<int>(), tile_expert.data_ptr<int>(),
               scratch.data_ptr<int>() + experts, dest_row.data_ptr<int>(),
               row_pair.data_ptr<int>(), pairs, (int)experts, (int)tile, (int)num_tiles,
               current_stream());
  return {dest_row, row_pair, tile_expert, k_offsets};
}

// dst[dest_row[j]] = scale[j] * src[j / k]. With `row_pair` (one entry per row of dst, negative for
// rows no pair maps to) those rows are zeroed; without it they are left untouched.
void moe_scatter_rows(const Tensor& src, const Tensor& dest_row, const c10::optional<Tensor>& scale,
                      const c10::optional<Tensor>& row_pair, Tensor& dst, int64_t k) {
  check_bf16(src, "src");
  check_bf16(dst, "dst");
  check_i32(dest_row, "dest_row");
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.dim() == 2 && dst.dim() == 2);
  TORCH_CHECK(src.size(1) == dst.size(1) && dest_row.numel() == src.size(0) * k);
  const float* scale_ptr = nullptr;
  if (scale.has_value()) {
    check_f32(*scale, "scale");
    TORCH_CHECK(scale->is_contiguous() && scale->numel() == dest_row.numel());
    scale_ptr = scale->data_ptr<float>();
  }
  const int* pair_ptr = nullptr;
  if (row_pair.has_value()) {
    check_i32(*row_pair, "row_pair");
    TORCH_CHECK(row_pair->numel() == dst.size(0), "row_pair must have one entry per row of dst");
    pair_ptr = row_pair->data_ptr<int>();
  }
  const c10::cuda::CUDAGuard guard(src.device());
  ob::moe_scatter_rows(src.data_ptr(), dest_row.data_ptr<int>(), scale_ptr, pair_ptr, dst.size(0),
                       dst.data_ptr(), dest_row.numel(), (int)k, (int)src.size(1), current_stream());
}

// out[t] = sum_i scale[t, i] * rows[dest_row[t*k + i]]; with `other` (tokens, d) also returns
// dot[t, i] = <rows[dest_row[t*k+i]], other[t]>.
std::vector<Tensor> moe_gather_combine(const Tensor& rows, const Tensor& dest_row,
                                       const c10::optional<Tensor>& scale,
                                       const c10::optional<Tensor>& other, int64_t k,
                                       bool want_out) {
  check_bf16(rows, "rows");
  check_i32(dest_row, "dest_row");
  TORCH_CHECK(rows.is_contiguous() && rows.dim() == 2 && dest_row.numel() % k == 0);
  const c10::cuda::CUDAGuard guard(rows.device());
  const int64_t tokens = dest_row.numel() / k, d = rows.size(1);
  const float* scale_ptr = nullptr;
  if (scale.has_value()) {
    check_f32(*scale, "scale");
    TORCH_CHECK(scale->is_contiguous() && scale->numel() == dest_row.numel());
    scale_ptr = scale->data_ptr<float>();
  }
  Tensor out, dot;
  const void* other_ptr = nullptr;
  if (other.has_value()) {
    check_bf16(*other, "other");
    TORCH_CHECK(other->is_contiguous() && other->numel() == tokens * d);
    other_ptr = other->data_ptr();
    dot = torch::empty({tokens, k}, rows.options().dtype(torch::kFloat32));
  }
  if (want_out) out = torch::empty({tokens, d}, rows.options());
  ob::moe_gather_combine(rows.data_ptr(), dest_row.data_ptr<int>(), scale_ptr, other_ptr,
                         want_out ? out.data_ptr() : nullptr,
                         other.has_value() ? dot.data_ptr<float>() : nullptr, tokens, (int)k, (int)d,
                         current_stream());
  return {out, dot};
}

// beta_sum[e] += rank-th largest of (logits[:, e] - alpha)
void qb_quantile(const Tensor& logits, const Tensor& alpha, Tensor& beta_sum, int64_t rank) {
  check_f32(logits, "logits");
  check_f32(alpha, "alpha");
  check_f32(beta_sum, "beta_sum");
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous() && alpha.is_contiguous());
  TORCH_CHECK(alpha.numel() == logits.size(0) && beta_sum.numel() == logits.size(1));
  const c10::cuda::CUDAGuard guard(logits.device());
  ob::qb_quantile(logits.data_ptr<float>(), alpha.data_ptr<float>(), beta_sum.data_ptr<float>(),
                  (int)logits.size(0), (int)logits.size(1), (int)rank, current_stream());
}

// -- serving --------------------------------------------------------------------------------------
const int* optional_i32(const c10::optional<Tensor>& t, const char* name) {
  if (!t.has_value()) return nullptr;
  check_i32(*t, name);
  return t->data_ptr<int>();
}
float* optional_f32(const c10::optional<Tensor>& t, const char* name) {
  if (!t.has_value()) return nullptr;
  check_f32(*t, name);
  TORCH_CHECK(t->is_contiguous(), name, " must be contiguous");
  return t->data_ptr<float>();
}

// q (B,T,H,D), k/v (B,T,Hk,D) bf16; cache_k/cache_v (Bmax, L, Hk, D) bf16 or int8 (then stats are
// four fp32 tensors (Bmax, L, Hk, 1)); cos/sin (positions, D/2) fp32 full tables. Returns rotated q.
Tensor rope_append(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& cache_k,
                   Tensor& cache_v, const std::vector<Tensor>& stats, const Tensor& cos_t,
                   const Tensor& sin_t, int64_t pos, const c10::optional<Tensor>& pos_dev) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_bf16(v, "v");
  check_f32(cos_t, "cos");
  check_f32(sin_t, "sin");
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && q.dim() == 4);
  TORCH_CHECK(cache_k.is_contiguous() && cache_v.is_contiguous() && cache_k.dim() == 4);
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous());
  const bool int8 = cache_k.scalar_type() == torch::kInt8;
  TORCH_CHECK(int8 || cache_k.scalar_type() == torch::kBFloat16, "cache must be bf16 or int8");
  TORCH_CHECK(cache_v.scalar_type() == cache_k.scalar_type());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), Hk = k.size(2);
  TORCH_CHECK(k.sizes() == v.sizes() && k.size(0) == B && k.size(1) == T && k.size(3) == D);
  TORCH_CHECK(cache_k.size(0) >= B && cache_k.size(2) == Hk && cache_k.size(3) == D,
              "cache shape does not match the new keys");
  TORCH_CHECK(cos_t.size(-1) == D / 2 && sin_t.sizes() == cos_t.sizes());
  float* st[4] = {nullptr, nullptr, nullptr, nullptr};
  if (int8) {
    TORCH_CHECK(stats.size() == 4, "an int8 cache needs key/value scale and minimum tensors");
    for (int i = 0; i < 4; ++i) {
      check_f32(stats[i], "cache statistics");
      TORCH_CHECK(stats[i].is_contiguous() && stats[i].numel() == cache_k.numel() / D);
      st[i] = stats[i].data_ptr<float>();
    }
  }
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor q_out = torch::empty_like(q);
  ob::rope_append(q.data_ptr(), k.data_ptr(), v.data_ptr(), q_out.data_ptr(), cache_k.data_ptr(),
                  cache_v.data_ptr(), st[0], st[1], st[2], st[3], cos_t.data_ptr<float>(),
                  sin_t.data_ptr<float>(), (int)B, (int)T, (int)H, (int)Hk, (int)D, (int)pos,
                  optional_i32(pos_dev, "pos_dev"), (int)cache_k.size(1), (int)cos_t.size(0), int8,
                  current_stream());
  return q_out;
}

// q (B, H, D) bf16 against the first `len` cache positions (or *pos_dev + 1). Returns (B, H, D).
Tensor decode_attention(const Tensor& q, const Tensor& cache_k, const Tensor& cache_v,
                        const std::vector<Tensor>& stats, int64_t len,
                        const c10::optional<Tensor>& pos_dev, double scale, int64_t splits) {
  check_bf16(q, "q");
  TORCH_CHECK(q.is_contiguous() && q.dim() == 3 && cache_k.is_contiguous() && cache_v.is_contiguous());
  const bool int8 = cache_k.scalar_type() == torch::kInt8;
  TORCH_CHECK(int8 || cache_k.scalar_type() == torch::kBFloat16, "cache must be bf16 or int8");
  const int64_t B = q.size(0), H = q.size(1), D = q.size(2), Hk = cache_k.size(2);
  TORCH_CHECK(cache_k.size(0) >= B && cache_k.size(3) == D && cache_v.sizes() == cache_k.sizes());
  TORCH_CHECK(pos_dev.has_value() || (len >= 1 && len <= cache_k.size(1)), "length out of range");
  const float* st[4] = {nullptr, nullptr, nullptr, nullptr};
  if (int8) {
    TORCH_CHECK(stats.size() == 4, "an int8 cache needs key/value scale and minimum tensors");
    for (int i = 0; i < 4; ++i) {
      check_f32(stats[i], "cache statistics");
      st[i] = stats[i].data_ptr<float>();
    }
  }
  const c10::cuda::CUDAGuard guard(q.device());
  if (splits <= 0) {
    const int64_t assumed = pos_dev.has_value() ? cache_k.size(1) : len;
    splits = ob::decode_attention_splits((int)B, (int)Hk, (int)assumed);
  }
  Tensor out = torch::empty_like(q);
  Tensor partial;
  if (splits > 1) partial = torch::empty({B * H * splits * (D + 2)}, q.options().dtype(torch::kFloat32));
  ob::decode_attention(q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(), st[0], st[1], st[2],
                       st[3], out.data_ptr(), splits > 1 ? partial.data_ptr<float>() : nullptr,
                       (int)B, (int)H, (int)Hk, (int)D, (int)cache_k.size(1), (int)len,
                       optional_i32(pos_dev, "pos_dev"), (int)splits, (float)scale, int8,
                       current_stream());
  return out;
}

// logits (rows, vocab) bf16 or fp32 (row stride may exceed vocab); uniforms (steps, rows) fp32 or
// none (greedy); out_tokens (rows, out_steps) int64. The int32 scalars `step` and `pos` live on
// the device and are advanced by the kernel when `counters` (three int32: step, pos, done) is given.
void sample_tokens(const Tensor& logits, int64_t valid_vocab, double temperature, int64_t top_k,
                   double top_p, const c10::optional<Tensor>& uniforms, Tensor& out_tokens,
                   const c10::optional<Tensor>& next_input, const c10::optional<Tensor>& counters,
                   const c10::optional<Tensor>& workspace) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  const bool bf16 = logits.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(bf16 || logits.scalar_type() == torch::kFloat32, "logits must be bf16 or fp32");
  TORCH_CHECK(out_tokens.is_cuda() && out_tokens.scalar_type() == torch::kInt64 &&
              out_tokens.dim() == 2 && out_tokens.size(0) == logits.size(0) &&
              out_tokens.stride(1) == 1);
  const c10::cuda::CUDAGuard guard(logits.device());
  int64_t* next_ptr = nullptr;
  if (next_input.has_value()) {
    TORCH_CHECK(next_input->is_cuda() && next_input->scalar_type() == torch::kInt64 &&
                next_input->is_contiguous() && next_input->numel() == logits.size(0));
    next_ptr = next_input->data_ptr<int64_t>();
  }
  int* step_ptr = nullptr;
  int* pos_ptr = nullptr;
  unsigned int* done_ptr = nullptr;
  if (counters.has_value()) {
    check_i32(*counters, "counters");
    TORCH_CHECK(counters->numel() == 3, "counters holds (step, position, done)");
    step_ptr = counters->data_ptr<int>();
    pos_ptr = step_ptr + 1;
    done_ptr = reinterpret_cast<unsigned int*>(step_ptr + 2);
  }
  const float* uni = nullptr;
  if (uniforms.has_value()) {
    check_f32(*uniforms, "uniforms");
    TORCH_CHECK(uniforms->is_contiguous() && uniforms->numel() % logits.size(0) == 0);
    uni = uniforms->data_ptr<float>();
  }
  ob::sample_tokens(logits.data_ptr(), bf16, logits.stride(0), (int)logits.size(0),
                    (int)logits.size(1), (int)std::min<int64_t>(valid_vocab, logits.size(1)),
                    (float)temperature, (int)top_k, (float)top_p, uni,
                    out_tokens.data_ptr<int64_t>(), out_tokens.stride(0), next_ptr, step_ptr, pos_ptr,
                    done_ptr, optional_f32(workspace, "workspace"), current_stream());
}

// -- expert parallelism ------------------------------------------------------------------------------
void ep_publish_counts(const std::vector<int64_t>& tables, const Tensor& counts, int64_t rank) {
  check_i32(counts, "counts");
  const c10::cuda::CUDAGuard guard(counts.device());
  ob::ep_publish_counts(tables.data(), counts.data_ptr<int>(), (int)counts.numel(), (int)rank,
                        (int)tables.size(), current_stream());
}

// From the exchanged (world, E) count table and this rank's int32 indices (N, k):
// (dest_rank (N*k), dest_row (N*k), tile_expert, k_offsets (E/world + 1), fill (2, E/world),
//  rows_used (1)). `capacity_rows` is the size of every rank's padded buffer.
std::vector<Tensor> ep_plan(const Tensor& table, const Tensor& indices, int64_t rank, int64_t world,
                            int64_t tile, int64_t capacity_rows) {
  check_i32(table, "table");
  check_i32(indices, "indices");
  const c10::cuda::CUDAGuard guard(indices.device());
  const int64_t experts = table.numel() / world, local = experts / world, pairs = indices.numel();
  TORCH_CHECK(experts * world == table.numel() && local * world == experts && capacity_rows % tile == 0);
  auto opts = indices.options();
  const int64_t num_tiles = capacity_rows / tile;
  Tensor dest_rank = torch::empty({pairs}, opts), dest_row = torch::empty({pairs}, opts);
  Tensor tile_expert = torch::empty({num_tiles}, opts), k_offsets = torch::empty({local + 1}, opts);
  Tensor fill = torch::empty({2, local}, opts), rows_used = torch::empty({1}, opts);
  Tensor scratch = torch::empty({2 * experts}, opts);  // pair bases, placement cursors
  ob::ep_plan(table.data_ptr<int>(), indices.data_ptr<int>(), (int)experts, (int)world, (int)rank,
              (int)tile, (int)num_tiles, (int)capacity_rows, pairs, scratch.data_ptr<int>(),
              k_offsets.data_ptr<int>(), tile_expert.data_ptr<int>(), fill.data_ptr<int>(),
              fill.data_ptr<int>() + local, scratch.data_ptr<int>() + experts,
              rows_used.data_ptr<int>(), dest_rank.data_ptr<int>(), dest_row.data_ptr<int>(),
              current_stream());
  return {dest_rank, dest_row, tile_expert, k_offsets, fill, rows_used};
}

void ep_zero_fill(const Tensor& fill, Tensor& buffer, int64_t d, int64_t capacity_rows) {
  check_i32(fill, "fill");
  check_bf16(buffer, "buffer");
  const c10::cuda::CUDAGuard guard(buffer.device());
  const int64_t local = fill.size(1);
  ob::ep_zero_fill(fill.data_ptr<int>(), fill.data_ptr<int>() + local, buffer.data_ptr(), (int)local,
                   (int)d, (int)capacity_rows, current_stream());
}

// `capacity_rows`: rows of every rank's buffer; a destination at or beyond it (or a rank outside the
// table) is recorded in the status word as a bad argument and skipped. -1 = unknown (no upper check).
void ep_push_rows(const Tensor& src, const Tensor& dest_rank, const Tensor& dest_row,
                  const c10::optional<Tensor>& scale, const std::vector<int64_t>& buffers, int64_t k,
                  int64_t capacity_rows) {
  check_bf16(src, "src");
  check_i32(dest_rank, "dest_rank");
  check_i32(dest_row, "dest_row");
  TORCH_CHECK(src.is_contiguous() && src.dim() == 2 && dest_row.numel() == src.size(0) * k);
  const float* scale_ptr = nullptr;
  if (scale.has_value()) {
    check_f32(*scale, "scale");
    TORCH_CHECK(scale->is_contiguous() && scale->numel() == dest_row.numel());
    scale_ptr = scale->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(src.device());
  ob::ep_push_rows(src.data_ptr(), dest_rank.data_ptr<int>(), dest_row.data_ptr<int>(), scale_ptr,
                   buffers.data(), (int)buffers.size(), dest_row.numel(), (int)k, (int)src.size(1),
                   capacity_rows < 0 ? 0x7fffffff : (int)capacity_rows, current_stream());
}

std::vector<Tensor> ep_pull_combine(const std::vector<int64_t>& buffers, const Tensor& dest_rank,
                                    const Tensor& dest_row, const c10::optional<Tensor>& scale,
                                    const c10::optional<Tensor>& other, int64_t k, int64_t d,
                                    bool want_out, int64_t capacity_rows) {
  check_i32(dest_rank, "dest_rank");
  check_i32(dest_row, "dest_row");
  const c10::cuda::CUDAGuard guard(dest_row.device());
  const int64_t tokens = dest_row.numel() / k;
  const float* scale_ptr = nullptr;
  if (scale.has_value()) {
    check_f32(*scale, "scale");
    TORCH_CHECK(scale->is_contiguous() && scale->numel() == dest_row.numel());
    scale_ptr = scale->data_ptr<float>();
  }
  auto bf16_opts = dest_row.options().dtype(torch::kBFloat16);
  Tensor out, dot;
  const void* other_ptr = nullptr;
  if (other.has_value()) {
    check_bf16(*other, "other");
    TORCH_CHECK(other->is_contiguous() && other->numel() == tokens * d);
    other_ptr = other->data_ptr();
    dot = torch::empty({tokens, k}, dest_row.options().dtype(torch::kFloat32));
  }
  if (want_out) out = torch::empty({tokens, d}, bf16_opts);
  ob::ep_pull_combine(buffers.data(), (int)buffers.size(), dest_rank.data_ptr<int>(),
                      dest_row.data_ptr<int>(), scale_ptr, other_ptr,
                      want_out ? out.data_ptr() : nullptr,
                      other.has_value() ? dot.data_ptr<float>() : nullptr, tokens, (int)k, (int)d,
                      capacity_rows < 0 ? 0x7fffffff : (int)capacity_rows, current_stream());
  return {out, dot};
}

// -- fused tensor-parallel collectives ---------------------------------------------------------------
// Tensor maps over `bases` (one (rows, K) K-major bf16 matrix of pitch `ld` per rank), uploaded to
// the device: the A operand of gemm_gather_a. Build once per buffer set and keep the tensor.
Tensor peer_row_maps(const std::vector<int64_t>& bases, int64_t rows, int64_t K, int64_t ld,
                     int64_t device_index) {
  const c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, (c10::DeviceIndex)device_index));
  Tensor host = torch::empty({(int64_t)bases.size() * 128}, torch::dtype(torch::kUInt8));
  ob::make_peer_row_maps(bases.data(), (int)bases.size(), rows, K, ld, host.data_ptr());
  return host.to(c10::Device(c10::kCUDA, (c10::DeviceIndex)device_index));
}

void check_2d_operand(const Tensor& t, const char* name) {
  check_bf16(t, name);
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1 && (t.stride(0) * 2) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              name, " must be a 2-D bf16 matrix with unit inner stride and 16-byte aligned rows");
}

// c (M, N) = [rows of all ranks] (M, K) @ op(b): the rows of A are read from the peers' staging
// buffers through `maps` once their ready flags (int32 at address `ready_addr`, one per rank) have
// reached `epoch`. `a_local` is this rank's staging buffer (rows M / world).
void gemm_gather_a(const Tensor& maps, const Tensor& a_local, const Tensor& b, Tensor& c, bool b_mn,
                   int64_t ready_addr, int64_t epoch, int64_t rank, int64_t world, double limit_s) {
  check_2d_operand(a_local, "a_local");
  check_2d_operand(b, "b");
  check_2d_operand(c, "c");
  TORCH_CHECK(maps.is_cuda() && maps.numel() == world * 128, "maps must hold one tensor map per rank");
  const int64_t rows = a_local.size(0), K = a_local.size(1), M = rows * world, N = c.size(1);
  TORCH_CHECK(c.size(0) == M && (b_mn ? (b.size(0) == K && b.size(1) == N)
                                      : (b.size(0) == N && b.size(1) == K)),
              "operand shapes do not match");
  const c10::cuda::CUDAGuard guard(c.device());
  ob::GemmComm comm;
  comm.mode = 1;
  comm.world = (int)world;
  comm.rank = (int)rank;
  comm.epoch = (unsigned int)epoch;
  comm.limit_ns = (unsigned long long)(limit_s * 1e9);
  comm.a_maps = maps.data_ptr();
  comm.ready = reinterpret_cast<const unsigned int*>(ready_addr);
  ob::gemm_bf16_comm(a_local.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, 1,
                     false, b_mn, a_local.stride(0), b.stride(0), c.stride(0), 0, 0, 0, false, false,
                     1, false, 1, false, 1.0f, nullptr, nullptr, rows, b.size(0),
                     ob::device_sm_count(), nullptr, 0, 0, 0.f, &comm, current_stream());
}

// Row block r of a (M, K) @ op(b) is stored into the buffer at address dests[r] (row pitch
// `dest_ld` elements): the receive slot that rank r keeps for this rank.
void gemm_push_c(const Tensor& a, const Tensor& b, bool b_mn, const std::vector<int64_t>& dests,
                 int64_t dest_ld, int64_t N, int64_t rank) {
  check_2d_operand(a, "a");
  check_2d_operand(b, "b");
  const int64_t M = a.size(0), K = a.size(1), world = (int64_t)dests.size();
  TORCH_CHECK(b_mn ? (b.size(0) == K && b.size(1) == N) : (b.size(0) == N && b.size(1) == K),
              "operand shapes do not match");
  TORCH_CHECK(world >= 1 && world <= 8 && dest_ld >= N && dest_ld % 8 == 0);
  const c10::cuda::CUDAGuard guard(a.device());
  ob::GemmComm comm;
  comm.mode = 2;
  comm.world = (int)world;
  comm.rank = (int)rank;
  for (int64_t r = 0; r < world; ++r) {
    TORCH_CHECK(dests[r] % 16 == 0, "receive slots must be 16-byte aligned");
    comm.c_peer[r] = reinterpret_cast<void*>(dests[r]);
  }
  comm.c_peer_ld = dest_ld;
  // The C tensor map is not used in this mode; describe this rank's own slot so that it is valid.
  ob::gemm_bf16_comm(a.data_ptr(), b.data_ptr(), reinterpret_cast<void*>(dests[rank]), (int)M, (int)N,
                     (int)K, 1, false, b_mn, a.stride(0), b.stride(0), dest_ld, 0, 0, 0, false, false,
                     1, false, 1, false, 1.0f, nullptr, nullptr, M, b.size(0), ob::device_sm_count(),
                     nullptr, 0, 0, 0.f, &comm, current_stream());
}

// Stream-ordered "wait until the int32 at `addr` is >= value" / "store value" on the current stream.
void stream_wait_value32(int64_t addr, int64_t value) {
  ob::stream_wait_value32(current_stream(), (uint64_t)addr, (uint32_t)value);
}
void stream_write_value32(int64_t addr, int64_t value) {
  ob::stream_write_value32(current_stream(), (uint64_t)addr, (uint32_t)value);
}

void tp_signal(const std::vector<int64_t>& pads, int64_t slot_base, int64_t rank, int64_t epoch) {
  ob::tp_signal(pads.data(), (int)slot_base, (int)rank, (int)pads.size(), (unsigned int)epoch,
                current_stream());
}

// out (rows, cols) = sum of the `world` slots of `slots` (world, rows, cols) (+ residual) once every
// flag at `flags_addr` has reached `epoch`.
Tensor tp_reduce_slots(const Tensor& slots, int64_t flags_addr, const c10::optional<Tensor>& residual,
                       int64_t epoch, double limit_s) {
  check_bf16(slots, "slots");
  TORCH_CHECK(slots.dim() == 3 && slots.is_contiguous());
  const c10::cuda::CUDAGuard guard(slots.device());
  Tensor out = torch::empty({slots.size(1), slots.size(2)}, slots.options());
  const void* res = nullptr;
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    TORCH_CHECK(residual->is_contiguous() && residual->numel() == out.numel());
    res = residual->data_ptr();
  }
  ob::tp_reduce_slots(slots.data_ptr(), reinterpret_cast<const unsigned int*>(flags_addr), res,
                      out.data_ptr(), slots.size(1), slots.size(2), (int)slots.size(0),
                      (unsigned int)epoch, (unsigned long long)(limit_s * 1e9), current_stream());
  return out;
}

// out (world * rows, cols) = the staged (rows, cols) blocks at `bases`, in rank order.
void tp_gather_rows(const std::vector<int64_t>& bases, int64_t flags_addr, Tensor& out, int64_t rank,
                    int64_t epoch, double limit_s) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous());
  const int64_t world = (int64_t)bases.size();
  const int64_t bytes = out.numel() * out.element_size();
  TORCH_CHECK(bytes % (16 * world) == 0, "gathered tensor must split into 16-byte aligned parts");
  const c10::cuda::CUDAGuard guard(out.device());
  ob::tp_gather_rows(bases.data(), reinterpret_cast<const unsigned int*>(flags_addr), out.data_ptr(),
                     bytes / world, (int)rank, (int)world, (unsigned int)epoch,
                     (unsigned long long)(limit_s * 1e9), current_stream());
}

// out = scale * sum over ranks of the symmetric buffers `bufs` (first out.numel() elements).
void peer_all_reduce(const std::vector<int64_t>& bufs, const std::vector<int64_t>& pads, Tensor& out,
                     double scale, int64_t rank, int64_t epoch, double limit_s) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && bufs.size() == pads.size());
  const bool bf16 = out.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(bf16 || out.scalar_type() == torch::kFloat32, "all-reduce supports bf16 and fp32");
  const c10::cuda::CUDAGuard guard(out.device());
  ob::peer_all_reduce(bufs.data(), pads.data(), out.data_ptr(), out.numel(), bf16, (float)scale,
                      (int)rank, (int)bufs.size(), (uint32_t)epoch, (uint64_t)(limit_s * 1e9),
                      current_stream());
}

// In-place small all-reduce whose epoch lives in `counter` (a 1-element int32 CUDA tensor), so the
// launch can be captured in a CUDA graph and replayed.
void peer_all_reduce_small(const std::vector<int64_t>& bufs, const std::vector<int64_t>& pads,
                           Tensor& counter, Tensor& tensor, int64_t slot_elems, double scale,
                           int64_t rank, double limit_s) {
  TORCH_CHECK(tensor.is_cuda() && tensor.is_contiguous() && bufs.size() == pads.size());
  TORCH_CHECK(counter.is_cuda() && counter.scalar_type() == torch::kInt32 && counter.numel() == 1);
  const bool bf16 = tensor.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(bf16 || tensor.scalar_type() == torch::kFloat32, "all-reduce supports bf16 and fp32");
  const c10::cuda::CUDAGuard guard(tensor.device());
  ob::peer_all_reduce_small(bufs.data(), pads.data(),
                            reinterpret_cast<uint32_t*>(counter.data_ptr<int32_t>()),
                            tensor.data_ptr(), tensor.data_ptr(), tensor.numel(), slot_elems, bf16,
                            (float)scale, (int)rank, (int)bufs.size(), (uint64_t)(limit_s * 1e9),
                            current_stream());
}

std::vector<int64_t> status(bool clear) {
  int out[4];
  ob::status_read(out, clear);
  return {out[0], out[1], out[2], out[3]};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "ohara_b200 sm_100a kernels";
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("c"), py::arg("M"), py::arg("N"),
        py::arg("K"), py::arg("a_mn"), py::arg("b_mn"), py::arg("splits") = 1,
        py::arg("reduce") = false, py::arg("alpha") = 1.0, py::arg("m_tile_batch") = py::none(),
        py::arg("k_offsets") = py::none(), py::arg("residual") = py::none(),
        py::arg("beta") = 1.0, py::arg("m_tile_rows") = 128);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope", &rope, py::arg("q"), py::arg("k"), py::arg("cos"), py::arg("sin"),
        py::arg("inverse"), py::arg("q_out") = py::none(), py::arg("k_out") = py::none());
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("cast_bf16_into", &cast_bf16_into);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("adamw_step", &adamw_step);
  m.def("cross_entropy_rows", &cross_entropy_rows);
  m.def("scale_by_scalar", &scale_by_scalar);
  m.def("flash_attn_fwd", &flash_attn_fwd);
  m.def("muon_prepare", &muon_prepare);
  m.def("muon_variance", &muon_variance);
  m.def("muon_apply", &muon_apply);
  m.def("pscan_fwd", &pscan_fwd);
  m.def("pscan_bwd", &pscan_bwd);
  m.def("pscan_cpu_fwd", &ob_cpu::pscan_cpu_fwd);
  m.def("pscan_cpu_bwd", &ob_cpu::pscan_cpu_bwd);
  m.def("sinkhorn_fwd", &sinkhorn_fwd);
  m.def("sinkhorn_bwd", &sinkhorn_bwd);
  m.def("sinkhorn_supported", &sinkhorn_supported);
  m.def("multimem_sum", &multimem_sum);
  m.def("bitnet_act_quant", &bitnet_act_quant);
  m.def("bitnet_weight_quant", &bitnet_weight_quant);
  m.def("bitnet_scale_rows", &bitnet_scale_rows);
  m.def("flash_attn_bwd", &flash_attn_bwd, py::arg("dout"), py::arg("q"), py::arg("k"),
        py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("causal"), py::arg("scale"),
        py::arg("dk_out") = py::none(), py::arg("dv_out") = py::none());
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_open", &peer_open);
  m.def("peer_close", &peer_close);
  m.def("peer_free", &peer_free);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_reduce_scatter_mean", &peer_reduce_scatter_mean);
  m.def("peer_all_gather", &peer_all_gather);
  m.def("peer_all_reduce", &peer_all_reduce);
  m.def("peer_all_reduce_small", &peer_all_reduce_small);
  m.def("gemv", &gemv);
  m.def("route_topk", &route_topk);
  m.def("moe_plan", &moe_plan);
  m.def("moe_scatter_rows", &moe_scatter_rows);
  m.def("moe_gather_combine", &moe_gather_combine);
  m.def("qb_quantile", &qb_quantile);
  m.def("rope_append", &rope_append);
  m.def("decode_attention", &decode_attention);
  m.def("sample_tokens", &sample_tokens);
  m.def("ep_publish_counts", &ep_publish_counts);
  m.def("ep_plan", &ep_plan);
  m.def("ep_zero_fill", &ep_zero_fill);
  m.def("ep_push_rows", &ep_push_rows, py::arg("src"), py::arg("dest_rank"), py::arg("dest_row"),
        py::arg("scale"), py::arg("buffers"), py::arg("k"), py::arg("capacity_rows") = -1);
  m.def("ep_pull_combine", &ep_pull_combine, py::arg("buffers"), py::arg("dest_rank"),
        py::arg("dest_row"), py::arg("scale"), py::arg("other"), py::arg("k"), py::arg("d"),
        py::arg("want_out"), py::arg("capacity_rows") = -1);
  m.def("peer_row_maps", &peer_row_maps);
  m.def("gemm_gather_a", &gemm_gather_a);
  m.def("gemm_push_c", &gemm_push_c);
  m.def("stream_wait_value32", &stream_wait_value32);
  m.def("stream_write_value32", &stream_write_value32);
  m.def("tp_signal", &tp_signal);
  m.def("tp_reduce_slots", &tp_reduce_slots);
  m.def("tp_gather_rows", &tp_gather_rows);
  m.def("status", &status);
  m.def("launch_count", []() { return (int64_t)ob::launch_count(); });
}
