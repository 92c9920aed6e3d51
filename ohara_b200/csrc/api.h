// Declarations of the torch-free kernel launchers. All pointers are device pointers; every launch
// goes to the given stream and returns without synchronising.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.h"

namespace ob {

// gemm_sm100.cu
void gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int batches, bool a_mn,
               bool b_mn, int64_t lda, int64_t ldb, int64_t ldc, int64_t strideA, int64_t strideB,
               int64_t strideC, bool a_batched, bool b_batched, int b_batches, bool out_f32,
               int splits, bool reduce, float alpha, const int* m_tile_batch,
               const int* k_offsets, int64_t a_rows, int64_t b_rows, int num_sms,
               const void* R, int64_t ldr, int64_t strideR, float beta, cudaStream_t stream,
               int m_tile_rows = 128);

// Fused collective of a GEMM (see gemm_sm100.cu). mode 1: gather the rows of A from `world` peers
// (`a_maps`: device array of tensor maps built by make_peer_row_maps, `ready`: this rank's flag
// slots). mode 2: push row block r of C into `c_peer[r]` (row pitch `c_peer_ld` elements).
struct GemmComm {
  int mode = 0;
  int world = 1;
  int rank = 0;
  unsigned int epoch = 0;
  unsigned long long limit_ns = 0;
  const void* a_maps = nullptr;
  const unsigned int* ready = nullptr;
  void* c_peer[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  long long c_peer_ld = 0;
};
void gemm_bf16_comm(const void* A, const void* B, void* C, int M, int N, int K, int batches,
                    bool a_mn, bool b_mn, int64_t lda, int64_t ldb, int64_t ldc, int64_t strideA,
                    int64_t strideB, int64_t strideC, bool a_batched, bool b_batched, int b_batches,
                    bool out_f32, int splits, bool reduce, float alpha, const int* m_tile_batch,
                    const int* k_offsets, int64_t a_rows, int64_t b_rows, int num_sms,
                    const void* R, int64_t ldr, int64_t strideR, float beta, const GemmComm* comm,
                    cudaStream_t stream, int m_tile_rows = 128);
// Encodes one (rows x K, K-major, pitch ld) A-operand tensor map per peer buffer into `out`
// (host memory, 128 bytes each).
void make_peer_row_maps(const int64_t* bases, int world, int64_t rows, int64_t K, int64_t ld,
                        void* out);

// tp_comm.cu
void tp_signal(const int64_t* flag_pads, int slot_base, int rank, int world, unsigned int epoch,
               cudaStream_t stream);
void tp_reduce_slots(const void* slots, const unsigned int* flags, const void* residual, void* out,
                     int64_t rows, int64_t cols, int world, unsigned int epoch,
                     unsigned long long limit_ns, cudaStream_t stream);
void tp_gather_rows(const int64_t* bases, const unsigned int* flags, void* out,
                    int64_t bytes_per_rank, int rank, int world, unsigned int epoch,
                    unsigned long long limit_ns, cudaStream_t stream);

// ep.cu
void ep_publish_counts(const int64_t* tables, const int* counts, int experts, int rank, int world,
                       cudaStream_t stream);
void ep_plan(const int* table, const int* indices, int experts, int world, int rank, int tile,
             int num_tiles, int capacity_rows, int64_t pairs, int* pair_base, int* k_offsets,
             int* tile_expert, int* fill_begin, int* fill_end, int* cursor, int* rows_used,
             int* dest_rank, int* dest_row, cudaStream_t stream);
void ep_zero_fill(const int* fill_begin, const int* fill_end, void* buffer, int local_experts, int d,
                  int capacity_rows, cudaStream_t stream);
void ep_push_rows(const void* src, const int* dest_rank, const int* dest_row, const float* scale,
                  const int64_t* buffers, int world, int64_t pairs, int k, int d, int capacity,
                  cudaStream_t stream);
void ep_pull_combine(const int64_t* buffers, int world, const int* dest_rank, const int* dest_row,
                     const float* scale, const void* other, void* out, float* dot, int64_t tokens,
                     int k, int d, int capacity, cudaStream_t stream);

// stream_ops.cpp
void stream_wait_value32(cudaStream_t stream, uint64_t addr, uint32_t value);
void stream_write_value32(cudaStream_t stream, uint64_t addr, uint32_t value);

// elementwise.cu
void rmsnorm_fwd(const void* x, const void* delta, const float* w, void* y, void* x_out, float* rstd,
                 int rows, int d, float eps, cudaStream_t stream);
void rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, const void* dres,
                 void* dx, float* dw, int rows, int d, cudaStream_t stream);
void rope_qk(const void* q, const void* k, void* qo, void* ko, const float* cos_t,
             const float* sin_t, int B, int T, int H, int Hk, int D, bool inverse,
             int64_t q_row_stride, int64_t k_row_stride, int64_t qo_row_stride,
             int64_t ko_row_stride, cudaStream_t stream);
void swiglu_fwd(const void* g, const void* u, void* a, int64_t rows, int h, int64_t g_pitch,
                int64_t u_pitch, int64_t a_pitch, cudaStream_t stream);
void swiglu_bwd(const void* da, const void* g, const void* u, void* dg, void* du, int64_t rows,
                int h, int64_t da_pitch, int64_t g_pitch, int64_t u_pitch, int64_t dg_pitch,
                int64_t du_pitch, cudaStream_t stream);
// out[i] = bf16(in[i] * scale)
void cast_f32_bf16(const float* in, void* out, int64_t n, cudaStream_t stream, float scale = 1.f);
void embedding_fwd(const int64_t* ids, const float* table, void* out, int64_t tokens, int d,
                   int vocab, cudaStream_t stream);
void embedding_bwd(const int64_t* ids, const void* dout, float* dtable, int64_t tokens, int d,
                   int vocab, cudaStream_t stream);
void adamw_step(float* p, const void* g, bool grad_is_bf16, float* m, float* v, void* shadow,
                int64_t n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                float bc2, float grad_scale, cudaStream_t stream);

// attention_fwd_sm100.cu
void flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T,
                    int S, int H, int Hk, int D, bool causal, float scale, int64_t q_tok_stride,
                    int64_t k_tok_stride, int64_t v_tok_stride, int64_t q_batch_stride,
                    int64_t k_batch_stride, int64_t v_batch_stride, cudaStream_t stream);

// muon.cu: stages of the Muon step around the Newton-Schulz GEMMs. Matrices of a group are reached
// through a pointer table; entry k covers `per_pointer` consecutive matrices (1 for separate
// parameters, B for one pre-stacked expert tensor).
constexpr int kMuonMaxPointers = 128;
struct MuonTable {
  void* ptr[kMuonMaxPointers];
};
void muon_momentum(const MuonTable& grads, float* momentum, void* u, float* norm2, int batch,
                   int64_t numel, float mu, int per_pointer, cudaStream_t stream);
void muon_scale(void* x, const float* norm2, int batch, int64_t numel, cudaStream_t stream);
void muon_variance(const void* x, float* v, int batch, int rows, int cols, bool by_row,
                   cudaStream_t stream);
void muon_apply(const MuonTable& params, const MuonTable* shadows, const void* x, const float* factor,
                int batch, int rows, int cols, float lr, float wd, bool by_row, int per_pointer,
                cudaStream_t stream);

// pscan.cu: h[t] = a[t] * h[t-1] + x[t] along dim 1 of contiguous (batch, length, channels) fp32
// tensors, and its gradients (da, dx) from dh, in one pass over the sequence each.
void pscan_forward(const float* a, const float* x, float* h, int64_t batch, int length,
                   int64_t channels, cudaStream_t stream);
void pscan_backward(const float* a, const float* h, const float* dh, float* da, float* dx,
                    int64_t batch, int length, int64_t channels, cudaStream_t stream);

// sinkhorn.cu: `count` row-major n x n fp32 matrices -> doubly stochastic matrices, and the
// vector-Jacobian product of that map.
bool sinkhorn_supported(int n, int iters);
void sinkhorn_forward(const float* in, float* out, int64_t count, int n, int iters,
                      cudaStream_t stream);
// `tape`: scratch of `count * sinkhorn_tape_floats(n, iters)` floats (may be null when that is 0).
int64_t sinkhorn_tape_floats(int n, int iters);
void sinkhorn_backward(const float* in, const float* grad_out, float* grad_in, float* tape,
                       int64_t count, int n, int iters, cudaStream_t stream);

// multimem.cu: out = scale * (sum over the ranks of a multicast group) of `bytes` bytes of bf16 or
// fp32 values at the multicast address (one switch-side reduction per 16 bytes; no waits inside).
void multimem_sum(const void* multicast, void* out, int64_t bytes, bool bf16, float scale,
                  cudaStream_t stream);

// quantize.cu: quantisers of BitNet b1.58 layers.
// q (bf16, integer values in [-128, 127]) and dequant (one factor per row) from x (bf16, rows x d);
// with `norm_weight` the row is RMS-normalised first and `rstd` (may be null) receives 1 / rms.
void bitnet_act_quant(const void* x, const float* norm_weight, void* q, float* dequant, float* rstd,
                      int rows, int d, float eps, cudaStream_t stream);
// ternary (bf16 in {-1, 0, 1}) and scale[0] = max(mean |w|, 1e-5) from n weights (fp32 or bf16);
// `partials`: scratch of `bitnet_partial_count()` floats.
int bitnet_partial_count();
void bitnet_weight_quant(const void* w, bool w_is_f32, int64_t n, void* ternary, float* scale,
                         float* partials, cudaStream_t stream);
// out (bf16) = acc (fp32, rows x n) * row_factor[row] * weight_scale[0] (+ bias[col], may be null).
void bitnet_scale_rows(const float* acc, const float* row_factor, const float* weight_scale,
                       const float* bias, void* out, int64_t rows, int n, cudaStream_t stream);

// attention_bwd_sm100.cu
void attn_delta(const void* o, const void* d_o, float* delta, int B, int T, int H, int D,
                int64_t do_tok_stride, int64_t do_batch_stride, cudaStream_t stream);
// `dq` (fp32, zero-initialised by the caller) receives the gradient of Q *without* the softmax
// scale: multiply by `scale` when converting it (cast_f32_bf16 takes the factor). dk / dv are final.
void flash_attn_bwd(const void* q, const void* k, const void* v, const void* d_o, float* dq,
                    void* dk, void* dv, const float* lse, const float* delta, int B, int T, int S,
                    int H, int Hk, int D, bool causal, float scale, const int64_t* strides,
                    cudaStream_t stream);

// peer.cu
void* peer_alloc(size_t bytes, char handle_out[64]);
void* peer_open(const char handle_in[64]);
void peer_close(void* ptr);
void peer_free(void* ptr);
void peer_barrier_launch(const int64_t* pads, int rank, int world, uint32_t epoch,
                         uint64_t limit_ns, cudaStream_t stream);
void peer_reduce_scatter_mean(const int64_t* grads, const int64_t* pads, float* out, int64_t region,
                              int rank, int world, uint32_t epoch, uint64_t limit_ns,
                              cudaStream_t stream);
void peer_all_gather(const int64_t* weights, const int64_t* pads, int64_t region_bytes, int rank,
                     int world, uint32_t epoch, uint64_t limit_ns, cudaStream_t stream);

void peer_all_reduce(const int64_t* bufs, const int64_t* pads, void* out, int64_t n, bool bf16,
                     float scale, int rank, int world, uint32_t epoch, uint64_t limit_ns,
                     cudaStream_t stream);
// Single-block, CUDA-graph-replayable all-reduce for small messages: the epoch is kept in the
// device word `counter`; `bufs` hold two slots of `slot_elems` elements per rank.
void peer_all_reduce_small(const int64_t* bufs, const int64_t* pads, uint32_t* counter,
                           const void* in, void* out, int64_t n, int64_t slot_elems, bool bf16,
                           float scale, int rank, int world, uint64_t limit_ns,
                           cudaStream_t stream);

// cross_entropy.cu
void cross_entropy_rows(void* logits, const int64_t* targets, float* row_loss, float* row_lse,
                        int* row_correct, const float* scale_ptr, int64_t rows, int vocab,
                        int64_t pitch, int64_t ignore_index, bool write_grad, cudaStream_t stream);
void scale_by_scalar(void* x, bool is_bf16, const float* scalar, int64_t n, cudaStream_t stream);

// gemv.cu
bool gemv_supported(int M, int N, int K);
void gemv_bf16(const void* x, const void* w, void* y, int M, int N, int K, int64_t ldx, int64_t ldw,
               int64_t ldy, cudaStream_t stream);

// moe.cu
void route_topk(const float* logits, const float* bias, int* indices, float* weights, float* alpha,
                int* counts, int tokens, int experts, int k, bool sigmoid_gate, bool normalize,
                bool want_alpha, cudaStream_t stream);
void moe_plan(const int* indices, const int* counts, int* seg_start, int* k_offsets,
              int* tile_expert, int* cursor, int* dest_row, int* row_pair, int64_t pairs,
              int experts, int tile, int num_tiles, cudaStream_t stream);
void moe_scatter_rows(const void* src, const int* dest_row, const float* scale,
                      const int* row_pair, int64_t padded_rows, void* dst, int64_t pairs, int k,
                      int d, cudaStream_t stream);
void moe_gather_combine(const void* rows, const int* dest_row, const float* scale, const void* other,
                        void* out, float* dot, int64_t tokens, int k, int d, cudaStream_t stream);
void qb_quantile(const float* logits, const float* alpha, float* beta_sum, int tokens, int experts,
                 int rank, cudaStream_t stream);

// decode.cu
void rope_append(const void* q, const void* k, const void* v, void* q_out, void* cache_k,
                 void* cache_v, float* k_scale, float* k_min, float* v_scale, float* v_min,
                 const float* cos_t, const float* sin_t, int B, int T, int H, int Hk, int D, int pos,
                 const int* pos_dev, int cache_len, int table_len, bool int8, cudaStream_t stream);
int decode_attention_splits(int B, int Hk, int len);
void decode_attention(const void* q, const void* cache_k, const void* cache_v, const float* k_scale,
                      const float* k_min, const float* v_scale, const float* v_min, void* out,
                      float* partial, int B, int H, int Hk, int D, int cache_len, int len,
                      const int* pos_dev, int splits, float scale, bool int8, cudaStream_t stream);
void sample_tokens(const void* logits, bool logits_bf16, int64_t row_stride, int rows, int vocab,
                   int valid_vocab, float temperature, int top_k, float top_p,
                   const float* uniforms, int64_t* out_tokens, int64_t out_stride,
                   int64_t* next_input, int* step_dev, int* pos_dev, unsigned int* done,
                   float* workspace, cudaStream_t stream);

}  // namespace ob
