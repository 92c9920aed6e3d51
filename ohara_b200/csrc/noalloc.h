// ob_flash_attn_bwd_noalloc: attention backward for callers that are not allowed to allocate.
//
// This entry point has no counterpart in the reference project. It exists for code that embeds the
// kernels somewhere device allocation is off the table: inside a region that a framework has
// frozen for replay, under an allocator that must account for every byte, in a real-time serving
// loop where a cudaMalloc (which may synchronise the whole device) would break the latency budget,
// or from a plain C host program that links the shared object without PyTorch's allocator.
//
// The regular entry point (flash_attn_bwd in the Python bindings) asks the caller's allocator for
// two pieces of scratch: an fp32 accumulator for dQ (summed across key tiles by the TMA reduce
// engine) and the per-row `delta = rowsum(dO * O)`. This variant keeps that scratch in a
// file-scope `static __device__` array inside the library instead, so it calls no cudaMalloc,
// no cudaFree and no allocating library routine.
//
// Limits (checked, with a message, before anything is launched):
//   B * T * H * D <= OB_NOALLOC_MAX_DQ_ELEMS   (8 Mi elements = 32 MiB of fp32 dQ accumulators)
//   B * H * T     <= OB_NOALLOC_MAX_ROWS       (256 Ki rows = 1 MiB of fp32 delta)
// The array is 33 MiB; every GPU on which a process loads this library holds it until the process
// exits, whether or not this function is ever called.
//
// Set-up: the first call on a device looks up the array's device address (cudaGetSymbolAddress,
// with that device current) and configures the kernel's shared-memory limit. Make that first call
// outside any stream capture; later calls only enqueue work on `stream`.
//
// Sharing: every call on a device uses the same array and the array keeps the previous call's
// contents. The function clears the part that must start at zero on `stream` before use. Two calls
// whose work overlaps on the GPU (different streams, or different host threads without ordering)
// race on the scratch and produce garbage: serialise them.
//
// Layouts: q, out, dout, dq are (B, T, H, D) bf16; k, v, dk, dv are (B, S, Hk, D) bf16; lse is
// (B, H, T) fp32 as written by the forward pass; all contiguous, all 16-byte aligned. D is 64 or
// 128; H is a multiple of Hk; causal attention needs S >= T. `status` may be null or point to 4
// ints of device memory that receive a non-zero code if an in-kernel wait timed out.
//
// Returns 0 on success; -1 bad argument, -2 problem larger than the scratch, -3 CUDA error. On
// failure a one-line description is copied into `err` (if non-null, at most `err_len` bytes).
#pragma once

#include <stddef.h>

#define OB_NOALLOC_MAX_DQ_ELEMS (8ll * 1024 * 1024)
#define OB_NOALLOC_MAX_ROWS (256ll * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int ob_flash_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out,
                              const void* dout, const float* lse, void* dq, void* dk, void* dv,
                              int B, int T, int S, int H, int Hk, int D, int causal, float scale,
                              void* stream, int* status, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
