// Host interface of the sm_100a tcgen05 GEMMs (gemm.cu): bf16 operands, or 8-bit float operands with
// per-tensor scales.
#pragma once

#include <cuda_runtime.h>

namespace nc {

enum GemmEpilogue : int {
  EPI_LINEAR = 0,    // C = alpha*acc + beta*aux           (aux optional, same dtype as C)
  EPI_RELU2 = 1,     // C = relu(alpha*acc)^2              (bf16 C)
  EPI_MUL2SQRT = 2,  // C = alpha*acc * 2*sqrt(aux)        (bf16 C; backward of relu^2 from its output)
  EPI_RELU = 3,      // C = relu(alpha*acc)                (bf16 C; the fp8 MLP keeps relu(x) and squares it while quantising)
  EPI_MULAUX = 4,    // C = alpha*acc * aux                (bf16 C; backward of relu^2 from relu(x), with alpha carrying the 2)
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
  // Optional, any operand type: device scalars multiplied into alpha when the kernel runs (the
  // de-quantisation scales of per-tensor-scaled fp8 operands), and a device word that receives
  // max |C| over the stored values (atomic max on the fp32 bit pattern; zero it beforehand).
  const float* scale_a = nullptr;
  const float* scale_b = nullptr;
  float* amax_out = nullptr;
  // gemm_fp8 only: operand element formats (0 = e4m3, 1 = e5m2)
  int a_e5m2 = 0, b_e5m2 = 0;
  // CTA-pair kernel (256 x BN tiles on two SMs): 1 = use it, 0 = never, -1 = let the library decide
  int pair = -1;
  // 1 = the product is symmetric by construction (X X^T, A A with A symmetric; M == N): only the square tiles on and
  // above the diagonal are computed (57 % of them at 1664 / 256) and the part of C below those tiles is left untouched;
  // `symmetrize_bf16` then copies the upper triangle over the lower one.
  int symmetric = 0;
};

// C[b][j][i] = C[b][i][j] for j > i: bf16 (batch, n, n) with row pitch ld and batch stride bs (elements).
cudaError_t symmetrize_bf16(void* C, int n, long long ld, long long bs, int batch, cudaStream_t stream);

cudaError_t gemm_bf16(const GemmDesc& d, int* status, cudaStream_t stream);

// Block-scaled 8-bit GEMM (MXFP8: tcgen05.mma.kind::mxf8f6f4.block_scale): A (M x K) and B (N x K) are K-major e4m3 /
// e5m2 bytes, every 32 consecutive K elements of a row share one E8M0 scale. K % 128 == 0. Scale factors come in the
// tensor core's blocked layout: for each block of 128 rows and 128 K elements one 512-byte chunk, chunks ordered
// [row block][k block], byte (r % 32) * 16 + ((r % 128) / 32) * 4 + (k / 32) % 4 for row r and element k. The scale
// arrays cover whole 128-row blocks (pad rows: any finite scale, e.g. 127 = 2^0). Same epilogues as the other GEMMs.
struct MxScales {
  const unsigned char* sfa;    // ceil(M/128) * (K/128) chunks
  const unsigned char* sfb;    // ceil(N/128) * (K/128) chunks
};
cudaError_t gemm_mxfp8(const GemmDesc& d, const MxScales& sf, int* status, cudaStream_t stream);
// Rows of a bf16 matrix (R x K, row pitch ld, K % 128 == 0) to MXFP8: q dense (R x K) bytes, sf in the blocked layout
// above (ceil(R/128) * (K/128) chunks; the caller pre-fills pad rows). Scale of a block = 2^(floor(log2 amax) - emax),
// emax = 8 (e4m3) or 15 (e5m2); an all-zero block gets 2^-127.
cudaError_t mx_quantize_bf16(const void* x, long long ld, int rows, int cols, void* q, unsigned char* sf, int e5m2,
                             cudaStream_t stream);
// Same contract with 1-byte A and B (lda/ldb/bs* in elements = bytes, multiples of 16).
cudaError_t gemm_fp8(const GemmDesc& d, int* status, cudaStream_t stream);
int gemm_pick_bn(int M, int N, int batch);

}  // namespace nc
