// First-order linear recurrence h[t] = a[t] * h[t-1] + x[t] (h[-1] = 0) along dim 1 of contiguous
// (B, L, C) fp32 tensors in host memory: the selective scan of Mamba and the RG-LRU on CPU tensors
// (reference: ohara/modules/pscan.py:63-258, an up/down sweep of whole-tensor PyTorch operations).
//
// The scan is bound by memory traffic, so it is written as one pass: a task owns a block of
// adjacent channels of one batch row, keeps the running state of the block in registers / L1 and
// walks the sequence once (read a, read x, write h). The channel loop is unit-stride and
// vectorises (the task bodies are compiled for AVX-512, AVX2 and the baseline, chosen at load
// time); tasks are spread over as many threads as PyTorch's intra-op setting allows (plain
// std::thread: a call moves tens of megabytes, against which starting the threads is free, and
// the extension then does not depend on which OpenMP runtime PyTorch was built with). The backward pass is the same
// recurrence in reverse time with the coefficient of the next step:
//     g[t] = dh[t] + a[t+1] * g[t+1],   dx[t] = g[t],   da[t] = g[t] * h[t-1].
#include <ATen/Parallel.h>
#include <torch/extension.h>

#include <algorithm>
#include <thread>
#include <vector>

#if defined(__GNUC__) && defined(__x86_64__)
#define OB_CPU_CLONES __attribute__((target_clones("avx512f", "avx2", "default")))
#else
#define OB_CPU_CLONES
#endif

namespace ob_cpu {

namespace {

constexpr int64_t kBlock = 1024;  // channels per task: 4 KB of state, one page of each tensor per step

void check(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.device().is_cpu() && t.scalar_type() == torch::kFloat32 && t.is_contiguous() &&
                  t.dim() >= 2,
              "cpu scan: ", name, " must be a contiguous float32 CPU tensor of shape (B, L, ...)");
}

// Runs body(task) for task in [0, tasks) on up to at::get_num_threads() threads.
template <typename Body>
void for_each_task(int64_t tasks, int64_t elements, const Body& body) {
  int64_t threads = std::min<int64_t>(at::get_num_threads(), tasks);
  if (elements < (1 << 16) || at::in_parallel_region()) threads = 1;
  if (threads <= 1) {
    for (int64_t task = 0; task < tasks; ++task) body(task);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(threads - 1);
  auto share = [&](int64_t worker) {
    for (int64_t task = worker; task < tasks; task += threads) body(task);
  };
  for (int64_t worker = 1; worker < threads; ++worker) pool.emplace_back(share, worker);
  share(0);
  for (auto& thread : pool) thread.join();
}

// One block of `width` <= kBlock channels of one batch row; pointers are at (row, t = 0, c0).
OB_CPU_CLONES void forward_block(const float* __restrict__ a, const float* __restrict__ x,
                                 float* __restrict__ h, int64_t length,
                                 int64_t channels, int64_t width) {
  float state[kBlock];
  for (int64_t c = 0; c < width; ++c) state[c] = 0.f;
  for (int64_t t = 0; t < length; ++t) {
    const float* __restrict__ at_ = a + t * channels;
    const float* __restrict__ xt = x + t * channels;
    float* __restrict__ ht = h + t * channels;
    for (int64_t c = 0; c < width; ++c) {
      state[c] = at_[c] * state[c] + xt[c];
      ht[c] = state[c];
    }
  }
}

OB_CPU_CLONES void backward_block(const float* __restrict__ a, const float* __restrict__ h,
                                  const float* __restrict__ dh, float* __restrict__ da,
                                  float* __restrict__ dx, int64_t length, int64_t channels,
                                  int64_t width) {
  float carry[kBlock];  // a[t+1] * g[t+1]
  for (int64_t c = 0; c < width; ++c) carry[c] = 0.f;
  for (int64_t t = length - 1; t > 0; --t) {
    const float* at_ = a + t * channels;
    const float* gt = dh + t * channels;
    const float* hprev = h + (t - 1) * channels;
    float* dat = da + t * channels;
    float* dxt = dx + t * channels;
    for (int64_t c = 0; c < width; ++c) {
      const float g = gt[c] + carry[c];
      dxt[c] = g;
      dat[c] = g * hprev[c];
      carry[c] = at_[c] * g;
    }
  }
  if (length > 0) {
    for (int64_t c = 0; c < width; ++c) {
      dx[c] = dh[c] + carry[c];
      da[c] = 0.f;  // h[-1] = 0
    }
  }
}

}  // namespace

torch::Tensor pscan_cpu_fwd(const torch::Tensor& a, const torch::Tensor& x) {
  check(a, "a");
  check(x, "x");
  TORCH_CHECK(a.sizes() == x.sizes(), "cpu scan: a and x must have the same shape");
  torch::Tensor h = torch::empty_like(x);
  const int64_t batch = a.size(0), length = a.size(1);
  const int64_t channels = batch * length == 0 ? 0 : a.numel() / (batch * length);
  if (channels == 0) return h;
  const int64_t blocks = (channels + kBlock - 1) / kBlock;
  const float* ap = a.data_ptr<float>();
  const float* xp = x.data_ptr<float>();
  float* hp = h.data_ptr<float>();
  for_each_task(batch * blocks, a.numel(), [&](int64_t task) {
    const int64_t b = task / blocks, c0 = (task % blocks) * kBlock;
    const int64_t base = b * length * channels + c0;
    forward_block(ap + base, xp + base, hp + base, length, channels,
                  std::min(kBlock, channels - c0));
  });
  return h;
}

std::vector<torch::Tensor> pscan_cpu_bwd(const torch::Tensor& a, const torch::Tensor& h,
                                         const torch::Tensor& dh) {
  check(a, "a");
  check(h, "h");
  check(dh, "dh");
  TORCH_CHECK(a.sizes() == h.sizes() && a.sizes() == dh.sizes(),
              "cpu scan: a, h and dh must have the same shape");
  torch::Tensor da = torch::empty_like(a), dx = torch::empty_like(a);
  const int64_t batch = a.size(0), length = a.size(1);
  const int64_t channels = batch * length == 0 ? 0 : a.numel() / (batch * length);
  if (channels == 0) return {da, dx};
  const int64_t blocks = (channels + kBlock - 1) / kBlock;
  const float* ap = a.data_ptr<float>();
  const float* hp = h.data_ptr<float>();
  const float* gp = dh.data_ptr<float>();
  float* dap = da.data_ptr<float>();
  float* dxp = dx.data_ptr<float>();
  for_each_task(batch * blocks, a.numel(), [&](int64_t task) {
    const int64_t b = task / blocks, c0 = (task % blocks) * kBlock;
    const int64_t base = b * length * channels + c0;
    backward_block(ap + base, hp + base, gp + base, dap + base, dxp + base, length, channels,
                   std::min(kBlock, channels - c0));
  });
  return {da, dx};
}

}  // namespace ob_cpu
