// Host interface of the sm_100a tcgen05 bf16 GEMM (gemm.cu).
#pragma once

#include <cuda_runtime.h>

namespace nc {

enum GemmEpilogue : int {
  EPI_LINEAR = 0,    // C = alpha*acc + beta*aux           (aux optional, same dtype as C)
  EPI_RELU2 = 1,     // C = relu(alpha*acc)^2              (bf16 C)
  EPI_MUL2SQRT = 2,  // C = alpha*acc * 2*sqrt(aux)        (bf16 C; backward of relu^2 from its output)
};

// C[b] (M x N, row-major, leading dim ldc) = epilogue(alpha * A[b] * B[b]^T, aux[b])
//   a_mn = 0: A stored [M][K] (K contiguous), lda = row pitch in elements
//   a_mn = 1: A stored [K][M] (M contiguous), lda = pitch of a K-row
//   b_mn = 0: B stored [N][K];  b_mn = 1: B stored [K][N]
// bs* are batch strides in elements. bf16 operands; C (and aux) bf16 or fp32 (c_f32).
struct GemmDesc {
  const void* A; int a_mn; long long lda, bsa;
  const void* B; int b_mn; long long ldb, bsb;
  void* C; int c_f32; long long ldc, bsc;
  const void* aux; long long ldaux, bsaux;
  int M, N, K, batch;
  float alpha, beta;
  int epi;
  int bn;   // N tile override (256/208/128/64/32); 0 = pick automatically
};

cudaError_t gemm_bf16(const GemmDesc& d, int* status, cudaStream_t stream);
int gemm_pick_bn(int M, int N, int batch);

}  // namespace nc
