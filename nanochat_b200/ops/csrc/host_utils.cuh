// Host-side helpers shared by the launchers: TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda) and device properties.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

namespace nc {

// Per-device "configured" flags. A kernel attribute (the raised dynamic shared-memory limit) belongs to one device,
// so a process that drives several GPUs has to set it on each; `once(f)` runs f for the current device until it has
// succeeded there once. Two threads racing on the first call both run f, which is idempotent.
struct PerDeviceOnce {
  static constexpr int kMax = 64;
  std::atomic<unsigned char> done[kMax] = {};
  template <class F>
  cudaError_t once(F&& f) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMax) return f();
    if (done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    e = f();
    if (e == cudaSuccess) done[dev].store(1, std::memory_order_release);
    return e;
  }
};

inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) return nullptr;
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// rank-`rank` tiled map with 128-byte swizzle. dims/box are innermost-first; strides_bytes has rank-1
// entries (byte pitch of dims 1..rank-1). Returns false when the encoder rejects the layout.
inline bool make_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  // Driver entry points need a current context on the calling thread; autograd's worker threads have
  // none until their first runtime call, so make the primary context current here. Once per thread: the call
  // is not allowed while a stream capture is in progress, and a thread that captures has launched eagerly before.
  static thread_local bool context_ready = false;
  if (!context_ready) {
    cudaFree(nullptr);
    context_ready = true;
  }
  auto enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bdim[i] = box[i]; estr[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = enc(out, dtype, rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[nanochat_b200] cuTensorMapEncodeTiled failed (%d): rank %d dims", (int)r, rank);
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %llu", (unsigned long long)dims[i]);
    fprintf(stderr, " box");
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %u", box[i]);
    fprintf(stderr, " base %p\n", base);
    return false;
  }
  return true;
}

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace nc
