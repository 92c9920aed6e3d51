// Python bindings: thin, checked wrappers that take torch tensors, launch on the current stream and
// never synchronise. Kernel launchers themselves are torch-free (raw pointers + geometry).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"

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
          const c10::optional<Tensor>& residual, double beta) {
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
    TORCH_CHECK(m_tile_batch->numel() >= (M + 127) / 128, "m_tile_batch is too short");
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
                b_rows, ob::device_sm_count(), res_ptr, ldr, stride_r, (float)beta, current_stream());
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
std::vector<Tensor> rope(const Tensor& q, const Tensor& k, const Tensor& cos_t, const Tensor& sin_t,
                         bool inverse) {
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
  Tensor qo = torch::empty({B, T, H, D}, q.options());
  Tensor ko = torch::empty({B, T, Hk, D}, k.options());
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

std::vector<Tensor> flash_attn_bwd(const Tensor& dout_in, const Tensor& q_in, const Tensor& k_in,
                                   const Tensor& v_in, const Tensor& out, const Tensor& lse,
                                   bool causal, double scale) {
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
  Tensor dk = torch::empty({B, S, Hk, D}, k.options());
  Tensor dv = torch::empty({B, S, Hk, D}, k.options());
  const int64_t strides[8] = {q.stride(1), q.stride(0), k.stride(1), k.stride(0),
                              v.stride(1), v.stride(0), d_o.stride(1), d_o.stride(0)};
  ob::flash_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr(),
                     dq32.data_ptr<float>(), dk.data_ptr(), dv.data_ptr(), lse.data_ptr<float>(),
                     delta.data_ptr<float>(), (int)B, (int)T, (int)S, (int)H, (int)Hk, (int)D,
                     causal, (float)scale, strides, current_stream());
  return {dq32.to(torch::kBFloat16), dk, dv};
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
        py::arg("beta") = 1.0);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope", &rope);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("cast_bf16_into", &cast_bf16_into);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("adamw_step", &adamw_step);
  m.def("cross_entropy_rows", &cross_entropy_rows);
  m.def("scale_by_scalar", &scale_by_scalar);
  m.def("flash_attn_fwd", &flash_attn_fwd);
  m.def("flash_attn_bwd", &flash_attn_bwd);
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_open", &peer_open);
  m.def("peer_close", &peer_close);
  m.def("peer_free", &peer_free);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_reduce_scatter_mean", &peer_reduce_scatter_mean);
  m.def("peer_all_gather", &peer_all_gather);
  m.def("status", &status);
  m.def("launch_count", []() { return (int64_t)ob::launch_count(); });
}
