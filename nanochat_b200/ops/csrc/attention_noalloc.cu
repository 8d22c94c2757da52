// Allocation-free entry point for the flash-attention backward pass (declared in attention_noalloc.h).
// It forwards to nc::attention_bwd with the delta scratch vector and the status word taken from
// fixed arrays inside the library image instead of caller-allocated memory.
#include "attention.h"
#include "attention_noalloc.h"

#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <mutex>

namespace {

// Scratch for delta = rowsum(dO * O) and the status word, resident in the library image. In host code
// these names are stand-ins, not device addresses: the address is resolved per device below.
static __device__ __align__(256) float g_noalloc_delta[NC_NOALLOC_MAX_DELTA];
static __device__ __align__(256) int g_noalloc_status[4];

constexpr int kMaxDevices = 64;
float* g_delta_ptr[kMaxDevices];
int* g_status_ptr[kMaxDevices];
// Set last, with release order, after both addresses above are written; readers load it with acquire order. The
// mutex makes the first call on a device from several host threads resolve the addresses exactly once.
std::atomic<bool> g_ready[kMaxDevices];
std::mutex g_setup_mutex;
thread_local char g_last_error[256] = "";

int fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess) snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
  else snprintf(g_last_error, sizeof(g_last_error), "%s", what);
  return code;
}

// One-time set-up for the CURRENT device: resolve the device addresses of the two arrays.
int setup_current_device(int* dev_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(NC_NOALLOC_CUDA_ERROR, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(NC_NOALLOC_BAD_ARGUMENT, "device index out of range");
  if (!g_ready[dev].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_ready[dev].load(std::memory_order_relaxed)) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_delta);
      if (e != cudaSuccess) return fail(NC_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress(delta scratch)", e);
      g_delta_ptr[dev] = static_cast<float*>(p);
      e = cudaGetSymbolAddress(&p, g_noalloc_status);
      if (e != cudaSuccess) return fail(NC_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress(status word)", e);
      g_status_ptr[dev] = static_cast<int*>(p);
      g_ready[dev].store(true, std::memory_order_release);
    }
  }
  *dev_out = dev;
  return NC_NOALLOC_OK;
}

}  // namespace

extern "C" int nc_attention_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                        const void* d_o, void* dq, void* dk, void* dv, int B, int Tq, int Tk, int H,
                                        int Hkv, long long q_bat, long long q_tok, long long q_head,
                                        long long kv_bat, long long kv_tok, long long kv_head, long long o_bat,
                                        long long o_tok, long long o_head, int window, float scale,
                                        cudaStream_t stream) {
  g_last_error[0] = 0;
  if (B <= 0 || Tq <= 0 || Tk <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || Tq > Tk)
    return fail(NC_NOALLOC_BAD_ARGUMENT, "need B,Tq,Tk,H,Hkv > 0, H divisible by Hkv and Tq <= Tk");
  // Everything the kernels assume about the caller's memory is checked here, before anything is launched: they read
  // and write 16-byte vectors, so a null or misaligned base, or a stride that is not a whole number of such vectors,
  // is refused instead of becoming a device fault.
  const void* ptrs[] = {q, k, v, o, lse, d_o, dq, dk, dv};
  for (const void* p : ptrs) {
    if (p == nullptr) return fail(NC_NOALLOC_BAD_ARGUMENT, "null tensor pointer");
    if (reinterpret_cast<uintptr_t>(p) % 16 != 0)
      return fail(NC_NOALLOC_BAD_ARGUMENT, "tensor pointers must be 16-byte aligned");
  }
  const long long strides[] = {q_bat, q_tok, q_head, kv_bat, kv_tok, kv_head, o_bat, o_tok, o_head};
  for (long long st : strides) {
    if (st <= 0 || st % 8 != 0)
      return fail(NC_NOALLOC_BAD_ARGUMENT, "strides must be positive multiples of 8 elements (16 bytes)");
  }
  if (q_head < 128 || kv_head < 128 || o_head < 128)
    return fail(NC_NOALLOC_BAD_ARGUMENT, "head stride smaller than the head dimension (128)");
  const long long need = 1ll * B * H * Tq;
  if (need > NC_NOALLOC_MAX_DELTA) {
    snprintf(g_last_error, sizeof(g_last_error),
             "B*H*Tq = %lld exceeds the built-in scratch of %d floats; use the allocating entry point", need,
             NC_NOALLOC_MAX_DELTA);
    return NC_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  if (int rc = setup_current_device(&dev)) return rc;
  nc::AttnBwdDesc d{};
  nc::AttnDesc& f = d.fwd;
  f.q = q; f.k = k; f.v = v; f.o = const_cast<void*>(o); f.lse = const_cast<float*>(lse);
  f.q_bat = q_bat; f.q_tok = q_tok; f.q_head = q_head;
  f.k_bat = kv_bat; f.k_tok = kv_tok; f.k_head = kv_head;
  f.v_bat = kv_bat; f.v_tok = kv_tok; f.v_head = kv_head;
  f.o_bat = o_bat; f.o_tok = o_tok; f.o_head = o_head;
  f.B = B; f.Tq = Tq; f.Tk = Tk; f.H = H; f.Hkv = Hkv; f.D = 128;
  f.window = window; f.scale = scale;
  d.d_o = d_o; d.do_bat = o_bat; d.do_tok = o_tok; d.do_head = o_head;
  d.dq = dq; d.dq_bat = q_bat; d.dq_tok = q_tok; d.dq_head = q_head;
  d.dk = dk; d.dk_bat = kv_bat; d.dk_tok = kv_tok; d.dk_head = kv_head;
  d.dv = dv; d.dv_bat = kv_bat; d.dv_tok = kv_tok; d.dv_head = kv_head;
  d.delta = g_delta_ptr[dev];
  cudaError_t e = nc::attention_bwd(d, g_status_ptr[dev], stream);
  if (e != cudaSuccess) return fail(NC_NOALLOC_CUDA_ERROR, "attention backward launch", e);
  return NC_NOALLOC_OK;
}

extern "C" int nc_noalloc_status(cudaStream_t stream) {
  g_last_error[0] = 0;
  int dev = 0;
  if (int rc = setup_current_device(&dev)) return rc;
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyAsync(host, g_status_ptr[dev], sizeof(host), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(NC_NOALLOC_CUDA_ERROR, "reading the status word", e);
  if (host[0] != 0) {
    cudaMemsetAsync(g_status_ptr[dev], 0, sizeof(host), stream);
    snprintf(g_last_error, sizeof(g_last_error), "a kernel abandoned a bounded wait (code %d, detail %d)",
             host[0] >> 24, host[0] & 0xffffff);
    return NC_NOALLOC_WAIT_TIMEOUT;
  }
  return NC_NOALLOC_OK;
}

extern "C" const char* nc_noalloc_last_error(void) { return g_last_error; }
