// Host interface of the Muon elementwise stages (optim.cu). k matrices of r x c, fp32 masters,
// bf16 work matrix X. Scratch vectors are caller-provided fp32 device buffers:
//   rowss, rowss2: k*r ; total, total2: k ; ss_scratch, scale_scratch: k*max(r,c).
#pragma once

#include <cuda_runtime.h>

namespace nc {

cudaError_t muon_momentum(const float* g, float* buf, void* X, float* rowss, float* total, float mu,
                          float grad_scale, int k, int r, int c, cudaStream_t s);
cudaError_t muon_equilibrate(void* X, const float* rowss, const float* total, float* rowss2, float* total2, int k,
                             int r, int c, cudaStream_t s);
// total[mat] = sum of rowss over the rows of each of the k matrices (fixed order).
cudaError_t muon_total(const float* rowss, float* total, int k, int r, cudaStream_t s);
// The statistics half of muon_finish: sums of squares of X, NorMuon second moment, per-row / per-column scale.
cudaError_t muon_stats(const void* X, float* second_buf, float* ss_scratch, float* scale_scratch, int k, int r, int c,
                       float beta2, cudaStream_t s);
cudaError_t muon_finish(float* p, const void* X, float* second_buf, float* ss_scratch, float* scale_scratch,
                        void* shadow, int k, int r, int c, float lr, float wd, float beta2, cudaStream_t s);

}  // namespace nc
