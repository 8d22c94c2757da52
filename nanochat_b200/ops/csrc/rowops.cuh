// Warp-per-row building blocks for the fused elementwise / normalisation kernels.
// A row of C bf16 values (C % 8 == 0, C <= 32*8*NV) is held in registers by one warp:
// lane l owns the 16-byte vectors l, l+32, l+64, ... so global accesses are coalesced
// and every reduction is a pure shuffle tree (no shared memory, no block barrier).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nc {

constexpr float RMS_EPS = 1.1920928955078125e-07f;  // fp32 machine epsilon (F.rms_norm default)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct bf16x8 { uint4 u; };

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
    float2 t = __bfloat1622float2(p);
    f[2 * j] = t.x; f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Round through bf16 (what storing and re-loading a bf16 activation would do).
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int NV>
struct RowF {
  float v[NV][8];
};

template <int NV>
__device__ __forceinline__ void load_row(RowF<NV>& r, const __nv_bfloat16* p, int nvec, int lane) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
    if (vi < nvec) {
      uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + vi);
      unpack8(u, r.v[i]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) r.v[i][j] = 0.f;
    }
  }
}
template <int NV>
__device__ __forceinline__ void store_row(const RowF<NV>& r, __nv_bfloat16* p, int nvec, int lane) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
    if (vi < nvec) reinterpret_cast<uint4*>(p)[vi] = pack8(r.v[i]);
  }
}
template <int NV>
__device__ __forceinline__ float row_dot(const RowF<NV>& a, const RowF<NV>& b) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) s += a.v[i][j] * b.v[i][j];
  return warp_sum(s);
}
template <int NV>
__device__ __forceinline__ float row_sumsq(const RowF<NV>& a) { return row_dot(a, a); }

// max |a| over this lane's part of the row, as the values will read back from bf16 storage
template <int NV>
__device__ __forceinline__ float lane_absmax_bf16(const RowF<NV>& a, float m) {
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(bf16_round(a.v[i][j])));
  return m;
}
// One atomic per warp: non-negative floats order like their bit patterns.
__device__ __forceinline__ void publish_absmax(float m, float* amax, int lane) {
  m = warp_max(m);
  if (lane == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));
}

}  // namespace nc
