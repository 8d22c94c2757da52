// Per-tensor ("tensorwise") dynamic scaling to 8-bit floats for the fp8 GEMMs.
//
//   amax  = max |x|                                   (amax_bf16: grid reduction, atomic max on the fp32 bits)
//   scale = FMAX / max(amax, 1e-12)                   (FMAX = 448 for e4m3, 57344 for e5m2)
//   q     = saturate_to_fp8(x * scale),  inv = 1/scale   (quantize_bf16; the GEMM multiplies inv back in)
//
// This is the arithmetic of torch's scaled-matmul recipe (reference: nanochat/fp8.py:82-107). The amax
// word is an input of the second kernel, so a producer that already knows it (a GEMM epilogue) can skip
// the first pass. Rows may be strided (row pitch in elements); the fp8 output is dense.
#include "fused.h"
#include "gemm.h"
#include "host_utils.cuh"
#include "ptx.cuh"

#include <cuda_fp8.h>

namespace nc {

__global__ void __launch_bounds__(256)
amax_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int rows, int cols, float* __restrict__ amax) {
  const int vec_per_row = cols >> 3;
  const long long total = (long long)rows * vec_per_row;
  float m = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row), c = (int)(i - (long long)r * vec_per_row);
    const uint4 v = *reinterpret_cast<const uint4*>(x + (long long)r * ld + c * 8);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int w = 16; w > 0; w >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, w));
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 8) {
    m = part[threadIdx.x];
#pragma unroll
    for (int w = 4; w > 0; w >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffu, m, w));
    // non-negative floats order like their bit patterns
    if (threadIdx.x == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));
  }
}

// SQUARE: the tensor quantised is x^2 (x = relu output of the MLP's up projection, kept in bf16 for the backward pass;
// its square is the down projection's input and exists only in fp8); `amax` then holds max|x| and max|x^2| is its square.
template <bool E5M2, bool SQUARE>
__global__ void __launch_bounds__(256)
quantize_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int rows, int cols,
                     const float* __restrict__ amax, uint8_t* __restrict__ q, float* __restrict__ inv_scale) {
  constexpr float FMAX = E5M2 ? 57344.f : 448.f;
  const float a_in = __ldg(amax);
  const float a = fmaxf(SQUARE ? a_in * a_in : a_in, 1e-12f);
  const float scale = FMAX / a;
  if (blockIdx.x == 0 && threadIdx.x == 0) *inv_scale = a / FMAX;
  const int vec_per_row = cols >> 4;      // 16 elements per thread step: 32 B in, 16 B out
  const long long total = (long long)rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row), c = (int)(i - (long long)r * vec_per_row);
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ld + c * 16);
    const uint4 v0 = src[0], v1 = src[1];
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 lo = unpack_bf16(w[2 * j]), hi = unpack_bf16(w[2 * j + 1]);
      if (SQUARE) { lo.x *= lo.x; lo.y *= lo.y; hi.x *= hi.x; hi.y *= hi.y; }
      lo.x *= scale; lo.y *= scale; hi.x *= scale; hi.y *= scale;
      const __nv_fp8x2_storage_t p0 = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
      const __nv_fp8x2_storage_t p1 = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
      out[j] = static_cast<uint32_t>(p0) | (static_cast<uint32_t>(p1) << 16);
    }
    *reinterpret_cast<uint4*>(q + (long long)r * cols + c * 16) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

static int quant_grid(long long work_items) {
  const long long blocks = (work_items + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

cudaError_t amax_bf16(const void* x, long long ld, int rows, int cols, float* amax, cudaStream_t s) {
  if ((cols & 7) || (ld & 7)) return cudaErrorInvalidValue;
  amax_bf16_kernel<<<quant_grid((long long)rows * (cols >> 3)), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ld, rows, cols, amax);
  return cudaGetLastError();
}

cudaError_t quantize_bf16(const void* x, long long ld, int rows, int cols, const float* amax, void* q,
                          float* inv_scale, int e5m2, int square, cudaStream_t s) {
  if ((cols & 15) || (ld & 7)) return cudaErrorInvalidValue;
  const int grid = quant_grid((long long)rows * (cols >> 4));
  auto* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* qp = reinterpret_cast<uint8_t*>(q);
  if (e5m2 && square) return cudaErrorInvalidValue;          // squared tensors are forward activations: e4m3
  if (e5m2)        quantize_bf16_kernel<true, false><<<grid, 256, 0, s>>>(xp, ld, rows, cols, amax, qp, inv_scale);
  else if (square) quantize_bf16_kernel<false, true><<<grid, 256, 0, s>>>(xp, ld, rows, cols, amax, qp, inv_scale);
  else             quantize_bf16_kernel<false, false><<<grid, 256, 0, s>>>(xp, ld, rows, cols, amax, qp, inv_scale);
  return cudaGetLastError();
}


// ------------------------------------------------------------------------------ MXFP8
// One thread per block of 32 consecutive elements of a row: amax of the block, scale 2^(floor(log2 amax) - emax) stored
// as an E8M0 byte in the tensor core's blocked scale layout (gemm.h: MxScales), elements divided by the scale and
// converted with saturation. The block's 64 bytes come in as four 16-byte loads and leave as two.
template <bool E5M2>
__global__ void __launch_bounds__(256)
mx_quantize_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int rows, int cols, uint8_t* __restrict__ q,
                        uint8_t* __restrict__ sf) {
  constexpr int EMAX = E5M2 ? 15 : 8;                 // exponent of the largest power of two the format holds
  const int blocks_per_row = cols >> 5;
  const int k_chunks = cols >> 7;                     // 128-element K blocks per row = scale chunks per row block
  const long long total = (long long)rows * blocks_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / blocks_per_row), kb = (int)(i - (long long)r * blocks_per_row);
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ld + kb * 32);
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 v = src[j];
      w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 f = unpack_bf16(w[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    int se = static_cast<int>((__float_as_uint(amax) >> 23) & 0xff) - 127 - EMAX;     // floor(log2 amax) - emax
    se = se < -127 ? -127 : se;
    const float inv = __uint_as_float(static_cast<uint32_t>(127 - se) << 23);         // 2^-se, exact
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2 lo = unpack_bf16(w[2 * j]), hi = unpack_bf16(w[2 * j + 1]);
      lo.x *= inv; lo.y *= inv; hi.x *= inv; hi.y *= inv;
      const __nv_fp8x2_storage_t p0 = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
      const __nv_fp8x2_storage_t p1 = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
      out[j] = static_cast<uint32_t>(p0) | (static_cast<uint32_t>(p1) << 16);
    }
    uint4* dst = reinterpret_cast<uint4*>(q + (long long)r * cols + kb * 32);
    dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
    dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    const size_t chunk = static_cast<size_t>(r >> 7) * k_chunks + (kb >> 2);
    sf[chunk * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3)] = static_cast<uint8_t>(se + 127);
  }
}

cudaError_t mx_quantize_bf16(const void* x, long long ld, int rows, int cols, void* q, unsigned char* sf, int e5m2,
                             cudaStream_t s) {
  if ((cols & 127) || (ld & 7)) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const int grid = quant_grid((long long)rows * (cols >> 5));
  auto* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* qp = reinterpret_cast<uint8_t*>(q);
  if (e5m2) mx_quantize_bf16_kernel<true><<<grid, 256, 0, s>>>(xp, ld, rows, cols, qp, sf);
  else      mx_quantize_bf16_kernel<false><<<grid, 256, 0, s>>>(xp, ld, rows, cols, qp, sf);
  return cudaGetLastError();
}

}  // namespace nc
