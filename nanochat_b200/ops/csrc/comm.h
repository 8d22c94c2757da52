// Host interface of the peer-to-peer optimizer kernels (comm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "fused.h"

namespace nc {

constexpr int MAX_RANKS = 8;

// Base pointers of one symmetric buffer on every rank (index = rank), as mapped into this process.
struct PeerPtrs {
  void* p[MAX_RANKS];
};

// All offsets are in ELEMENTS of the buffer's type (fp32 for gradients, bf16 for outputs).
cudaError_t p2p_barrier(const PeerPtrs& pads, int rank, int world, int epoch, int* status, cudaStream_t s);
cudaError_t p2p_adamw(const PeerPtrs& grads, size_t grad_off, int world, int rank, void* p, int p_bf16, void* m, void* v,
                      const PeerPtrs& out, size_t out_off, int write_local_out, size_t n, AdamWArgs a, int max_ctas,
                      cudaStream_t s);
cudaError_t p2p_muon_momentum(const PeerPtrs& grads, size_t grad_off, int world, float* buf, void* X, float* rowss,
                              float mu, int k, int r, int c, int max_ctas, cudaStream_t s);
// Parameter update of this rank's chunk with the bf16 result stored into every rank's shadow stack (out_off in bf16
// elements from each rank's base). `scale`: k*r (r >= c) or k*c entries from muon_stats.
cudaError_t p2p_muon_apply(float* p, const void* X, const float* scale, const PeerPtrs& out, size_t out_off, int world,
                           int k, int r, int c, float lr, float wd, cudaStream_t s);
cudaError_t p2p_bcast_bf16(const void* src, const PeerPtrs& dst, size_t dst_off, int world, int rank, size_t n,
                           cudaStream_t s);
// Gradient pushes (the reduce-scatter's transfer when no GEMM epilogue delivers it): see comm.cu.
cudaError_t p2p_push_slices(const float* src, size_t n, size_t slice, const PeerPtrs& stage, size_t dst_off, int rank,
                            int max_ctas, cudaStream_t s);
cudaError_t p2p_copy_f32(const float* src, float* dst, size_t n, cudaStream_t s);
cudaError_t p2p_small_adamw(const PeerPtrs& grads, size_t grad_off, int world, float* p, float* m, float* v, int n,
                            AdamWArgs a, cudaStream_t s);

}  // namespace nc
