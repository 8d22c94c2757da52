// Allocation-free entry point for the flash-attention backward pass.
//
// This function has no counterpart in the reference implementation. It exists for callers that
// cannot allocate device memory at the point where they need the backward pass: code running
// inside a region where the allocator must stay untouched (a caller-managed memory pool whose
// budget is fixed up front, a real-time loop, a plugin that was handed its buffers by a host
// application and must not grow them). The regular entry point (nc::attention_bwd, reached from
// Python as _C.attn_bwd) needs one scratch vector, delta[b,h,t] = sum_d dO*O, which its caller
// allocates. Here that vector lives in a fixed array inside the library image, so the call
// performs no cudaMalloc / cudaFree and uses no allocating library routine.
//
// Limits and rules
//   * B * H * Tq must not exceed NC_NOALLOC_MAX_DELTA (1,048,576 floats = 4 MiB per GPU that loads
//     the library; the array is held until the process exits). Larger problems are rejected with
//     NC_NOALLOC_TOO_LARGE and a message retrievable through nc_noalloc_last_error().
//   * The first call on each device resolves the device address of the array (one
//     cudaGetSymbolAddress with that device current) and raises the kernels' shared-memory limit.
//     Make that first call before any stream capture begins.
//   * Every call on a device shares the one array and leaves the last call's values in it. Nothing
//     in it has to start at zero (the pre-pass overwrites the B*H*Tq entries the kernels read).
//     Two calls that overlap in time on the same GPU (different streams) race on it: serialise them.
//   * Inputs and outputs are still the caller's: q, k, v, o, lse, d_o are read; dq, dk, dv written.
//     Pointers must be non-null and 16-byte aligned, strides positive multiples of 8 elements; anything
//     else is refused with NC_NOALLOC_BAD_ARGUMENT before a kernel is launched.
//   * The first call on a device may come from any host thread; concurrent first calls resolve the
//     address once (the set-up is guarded by a mutex).
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NC_NOALLOC_MAX_DELTA (1 << 20)

enum {
  NC_NOALLOC_OK = 0,
  NC_NOALLOC_TOO_LARGE = 1,      // B*H*Tq > NC_NOALLOC_MAX_DELTA
  NC_NOALLOC_BAD_ARGUMENT = 2,   // unsupported head grouping / Tq > Tk / null or misaligned pointer / bad stride
  NC_NOALLOC_CUDA_ERROR = 3,     // a CUDA call failed; see nc_noalloc_last_error()
  NC_NOALLOC_WAIT_TIMEOUT = 4,   // reported by nc_noalloc_status(): a bounded in-kernel wait gave up
};

// Tensors are bf16 with the head dimension (128) contiguous; strides are in elements:
//   q, o, d_o, dq : (B, Tq, H,   128)   strides {*_bat, *_tok, *_head}
//   k, v, dk, dv  : (B, Tk, Hkv, 128)
//   lse           : (B, H, Tq) fp32, as written by the forward pass
// `window` < 0 means unlimited left context. Returns one of the NC_NOALLOC_* codes; the kernels run
// asynchronously on `stream`.
int nc_attention_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const float* lse,
                             const void* d_o, void* dq, void* dk, void* dv,
                             int B, int Tq, int Tk, int H, int Hkv,
                             long long q_bat, long long q_tok, long long q_head,
                             long long kv_bat, long long kv_tok, long long kv_head,
                             long long o_bat, long long o_tok, long long o_head,
                             int window, float scale, cudaStream_t stream);

// Synchronises `stream` and returns NC_NOALLOC_OK, or NC_NOALLOC_WAIT_TIMEOUT if a kernel launched
// through the entry point above abandoned a wait since the last query. The word is then cleared by a
// memset queued on `stream`: it is ordered before later work on that stream only, so a launch on another
// stream right after this call may still see (and re-report) the old value.
int nc_noalloc_status(cudaStream_t stream);

// Text of the last error returned on this thread ("" if none).
const char* nc_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
