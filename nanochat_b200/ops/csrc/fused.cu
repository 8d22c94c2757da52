// Fused elementwise / normalisation kernels of the transformer layer (forward and
// backward). All are HBM-bound: each reads its inputs once, keeps the row in
// registers (one warp per row, see rowops.cuh) and writes its outputs once.
//
//   mixnorm_fwd       xm = lr*x + l0*x0 ; xn = rmsnorm(xm)
//   norm_fwd          y  = rmsnorm(x)
//   normadd_bwd       dx = dres + d(rmsnorm)(dy; x)
//   mixnorm_bwd       dxm = dres + d(rmsnorm)(dxn [+ gate grad on 12 cols]; xm);
//                     dx = lr*dxm ; dx0 = l0*dxm ; dlr += <dxm,x> ; dl0 += <dxm,x0>
//   qkv_post_fwd/bwd  rotary (half split, -theta) -> rmsnorm -> x1.2 on q,k heads and the
//                     gated value-embedding add on v heads, in place on a [M, (H+2Hkv)*D] buffer
//   backout_norm      y = rmsnorm(x - lam*xb) and its backward
//   embed             token embedding -> rmsnorm -> previous-token smear, and its backward
#include "fused.h"
#include "rowops.cuh"

namespace nc {

constexpr int ROW_WARPS = 4;  // warps (rows in flight) per CTA

template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32, 6)
mixnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x0,
                   const float* __restrict__ lam_r, const float* __restrict__ lam_0, int layer,
                   __nv_bfloat16* __restrict__ xm, __nv_bfloat16* __restrict__ xn, float* __restrict__ amax_xn,
                   int M, int C) {
  const int lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  const float lr = lam_r[layer], l0 = lam_0[layer];
  float mx = 0.f;
  for (int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); row < M; row += gridDim.x * ROW_WARPS) {
    RowF<NV> a, b;
    load_row(a, x + (size_t)row * C, nvec, lane);
    load_row(b, x0 + (size_t)row * C, nvec, lane);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) a.v[i][j] = bf16_round(lr * a.v[i][j] + l0 * b.v[i][j]);
    store_row(a, xm + (size_t)row * C, nvec, lane);
    const float rstd = rsqrtf(row_sumsq(a) / C + RMS_EPS);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) a.v[i][j] *= rstd;
    store_row(a, xn + (size_t)row * C, nvec, lane);
    if (amax_xn) mx = lane_absmax_bf16(a, mx);
  }
  if (amax_xn) publish_absmax(mx, amax_xn, lane);
}

template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, float* __restrict__ amax_y, int M,
                int C) {
  const int lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  float mx = 0.f;
  for (int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); row < M; row += gridDim.x * ROW_WARPS) {
    RowF<NV> a;
    load_row(a, x + (size_t)row * C, nvec, lane);
    const float rstd = rsqrtf(row_sumsq(a) / C + RMS_EPS);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) a.v[i][j] *= rstd;
    store_row(a, y + (size_t)row * C, nvec, lane);
    if (amax_y) mx = lane_absmax_bf16(a, mx);
  }
  if (amax_y) publish_absmax(mx, amax_y, lane);
}

// g <- grad wrt the norm input, given g = grad wrt the norm output and the norm input xin.
template <int NV>
__device__ __forceinline__ void rmsnorm_bwd_inplace(RowF<NV>& g, const RowF<NV>& xin, int C) {
  const float rstd = rsqrtf(row_sumsq(xin) / C + RMS_EPS);
  const float proj = row_dot(g, xin) * rstd * rstd / C;   // mean(g * xhat) * rstd, with xhat = xin*rstd
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) g.v[i][j] = rstd * (g.v[i][j] - xin.v[i][j] * proj);
}

template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32, 4)
normadd_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, float* __restrict__ amax_dx,
                   int M, int C) {
  const int lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  float mx = 0.f;
  for (int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); row < M; row += gridDim.x * ROW_WARPS) {
    RowF<NV> g, xin;
    load_row(g, dy + (size_t)row * C, nvec, lane);
    load_row(xin, x + (size_t)row * C, nvec, lane);
    rmsnorm_bwd_inplace(g, xin, C);
    if (dres) {
      RowF<NV> r;
      load_row(r, dres + (size_t)row * C, nvec, lane);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) g.v[i][j] += r.v[i][j];
    }
    store_row(g, dx + (size_t)row * C, nvec, lane);
    if (amax_dx) mx = lane_absmax_bf16(g, mx);
  }
  if (amax_dx) publish_absmax(mx, amax_dx, lane);
}

template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32, 3)      // 168 registers instead of 214: three CTAs per SM, not two
mixnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dxn, const __nv_bfloat16* __restrict__ dres,
                   const float* __restrict__ dgate /* [M,12] or null */,
                   const __nv_bfloat16* __restrict__ xm, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ x0, const float* __restrict__ lam_r,
                   const float* __restrict__ lam_0, int layer, __nv_bfloat16* __restrict__ dx,
                   __nv_bfloat16* __restrict__ dx0, int accumulate_dx0, float* __restrict__ dlam_r,
                   float* __restrict__ dlam_0, float* __restrict__ amax_dx, int M, int C) {
  __shared__ float red[2][ROW_WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = C >> 3;
  const float lr = lam_r[layer], l0 = lam_0[layer];
  float acc_r = 0.f, acc_0 = 0.f, mx = 0.f;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < M; row += gridDim.x * ROW_WARPS) {
    RowF<NV> g, t;
    load_row(g, dxn + (size_t)row * C, nvec, lane);
    if (dgate && lane < 2) {   // columns 0..11 live in vector 0 (lane 0) and half of vector 1 (lane 1)
      const float* dg = dgate + (size_t)row * 12;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = lane * 8 + j;
        if (c < 12) g.v[0][j] += dg[c];
      }
    }
    load_row(t, xm + (size_t)row * C, nvec, lane);
    rmsnorm_bwd_inplace(g, t, C);
    load_row(t, dres + (size_t)row * C, nvec, lane);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) g.v[i][j] += t.v[i][j];      // g = dxm
    load_row(t, x + (size_t)row * C, nvec, lane);
    acc_r += row_dot(g, t);
    load_row(t, x0 + (size_t)row * C, nvec, lane);
    acc_0 += row_dot(g, t);
    if (accumulate_dx0) {
      load_row(t, dx0 + (size_t)row * C, nvec, lane);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) t.v[i][j] += l0 * g.v[i][j];
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) t.v[i][j] = l0 * g.v[i][j];
    }
    store_row(t, dx0 + (size_t)row * C, nvec, lane);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) g.v[i][j] *= lr;
    store_row(g, dx + (size_t)row * C, nvec, lane);
    if (amax_dx) mx = lane_absmax_bf16(g, mx);
  }
  if (amax_dx) publish_absmax(mx, amax_dx, lane);
  if (lane == 0) { red[0][warp] = acc_r; red[1][warp] = acc_0; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float sr = 0.f, s0 = 0.f;
    for (int w = 0; w < ROW_WARPS; ++w) { sr += red[0][w]; s0 += red[1][w]; }
    atomicAdd(dlam_r + layer, sr);
    atomicAdd(dlam_0 + layer, s0);
  }
}

// ------------------------------------------------------------------ backout + norm
template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32)
backout_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ xb,
                        const float* __restrict__ lam, __nv_bfloat16* __restrict__ y, int M, int C) {
  const int lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  const float l = bf16_round(lam[0]);
  for (int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); row < M; row += gridDim.x * ROW_WARPS) {
    RowF<NV> a, b;
    load_row(a, x + (size_t)row * C, nvec, lane);
    if (xb) {
      load_row(b, xb + (size_t)row * C, nvec, lane);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) a.v[i][j] = bf16_round(a.v[i][j] - l * b.v[i][j]);
    }
    const float rstd = rsqrtf(row_sumsq(a) / C + RMS_EPS);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) a.v[i][j] *= rstd;
    store_row(a, y + (size_t)row * C, nvec, lane);
  }
}

template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32)
backout_norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ xb, const float* __restrict__ lam,
                        __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dxb,
                        float* __restrict__ dlam, int M, int C) {
  __shared__ float red[ROW_WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = C >> 3;
  const float l = bf16_round(lam[0]);
  float acc = 0.f;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < M; row += gridDim.x * ROW_WARPS) {
    RowF<NV> g, z, b;
    load_row(g, dy + (size_t)row * C, nvec, lane);
    load_row(z, x + (size_t)row * C, nvec, lane);
    if (xb) {
      load_row(b, xb + (size_t)row * C, nvec, lane);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) z.v[i][j] = bf16_round(z.v[i][j] - l * b.v[i][j]);
    }
    rmsnorm_bwd_inplace(g, z, C);
    store_row(g, dx + (size_t)row * C, nvec, lane);
    if (xb) {
      acc -= row_dot(g, b);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) g.v[i][j] *= -l;
      store_row(g, dxb + (size_t)row * C, nvec, lane);
    }
  }
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0 && xb) {
    float s = 0.f;
    for (int w = 0; w < ROW_WARPS; ++w) s += red[w];
    atomicAdd(dlam, s);
  }
}

// ---------------------------------------------------------------- q/k/v post-processing
// Buffer layout per token: [ q: H heads | k: Hkv heads | v: Hkv heads ] x 128 dims, row pitch `ld`.
// Eight lanes own one head: lane s holds dims [8s, 8s+8) and [64+8s, 64+8s+8), so the
// rotation pairs (d, d+64) are lane-local and the norm reduces over 8 lanes.
// Sum over the 8 lanes of one head group. The four groups of a warp may sit in different branches
// (rotary head / value head / idle), so the shuffle names only the group's own lanes.
__device__ __forceinline__ float group8_sum(float v, int grp) {
  const unsigned mask = 0xffu << (grp * 8);
  v += __shfl_xor_sync(mask, v, 1);
  v += __shfl_xor_sync(mask, v, 2);
  v += __shfl_xor_sync(mask, v, 4);
  return v;
}

__device__ __forceinline__ float ve_gate_value(const __nv_bfloat16* xn_row, const float* wg_h) {
  float z = 0.f;
#pragma unroll
  for (int c = 0; c < 12; ++c) z += __bfloat162float(xn_row[c]) * bf16_round(wg_h[c]);
  return bf16_round(z);
}

__global__ void __launch_bounds__(128)
qkv_post_fwd_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, int H, int Hkv,
                    const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t, int T,
                    float* __restrict__ rstd_out /* [M, H+Hkv] */,
                    const __nv_bfloat16* __restrict__ xn, long long ld_xn, const float* __restrict__ wg,
                    const __nv_bfloat16* __restrict__ ve, const long long* __restrict__ idx, int M) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, grp = lane >> 3;
  const int n_rot = H + Hkv;
  const int n_items = n_rot + (ve ? Hkv : 0);
  for (int tok = blockIdx.x * 4 + warp; tok < M; tok += gridDim.x * 4) {
    const int t = tok % T;
    __nv_bfloat16* row = qkv + (size_t)tok * ld;
    float c[8], s[8];
    {
      float tmp[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(cos_t + (size_t)t * 64) + sub), tmp);
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = tmp[j];
      unpack8(__ldg(reinterpret_cast<const uint4*>(sin_t + (size_t)t * 64) + sub), tmp);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] = tmp[j];
    }
    // The update is in place, so the compiler may not move an item's loads above the previous item's stores; the next
    // item's two 16-byte pieces are requested by hand before the current item is worked on (every item lives at
    // row + item * 128, rotary heads and value heads alike).
    uint4 na = make_uint4(0, 0, 0, 0), nb = na;
    if (grp < n_items) {
      na = *(reinterpret_cast<const uint4*>(row + (size_t)grp * 128) + sub);
      nb = *(reinterpret_cast<const uint4*>(row + (size_t)grp * 128) + 8 + sub);
    }
    for (int base = 0; base < n_items; base += 4) {
      const int item = base + grp;
      const uint4 ca = na, cb = nb;
      if (item + 4 < n_items) {
        na = *(reinterpret_cast<const uint4*>(row + (size_t)(item + 4) * 128) + sub);
        nb = *(reinterpret_cast<const uint4*>(row + (size_t)(item + 4) * 128) + 8 + sub);
      }
      if (item < n_rot) {
        __nv_bfloat16* h = row + (size_t)item * 128;
        float a[8], b[8];
        unpack8(ca, a);
        unpack8(cb, b);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float y1 = bf16_round(a[j] * c[j] + b[j] * s[j]);
          const float y2 = bf16_round(b[j] * c[j] - a[j] * s[j]);
          a[j] = y1; b[j] = y2;
          ss += y1 * y1 + y2 * y2;
        }
        ss = group8_sum(ss, grp);
        const float rstd = rsqrtf(ss * (1.f / 128.f) + RMS_EPS);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a[j] = bf16_round(a[j] * rstd) * 1.2f;
          b[j] = bf16_round(b[j] * rstd) * 1.2f;
        }
        *(reinterpret_cast<uint4*>(h) + sub) = pack8(a);
        *(reinterpret_cast<uint4*>(h) + 8 + sub) = pack8(b);
        if (sub == 0) rstd_out[(size_t)tok * n_rot + item] = rstd;
      } else if (item < n_items) {
        const int hv = item - n_rot;
        __nv_bfloat16* h = row + (size_t)(n_rot + hv) * 128;
        const float z = ve_gate_value(xn + (size_t)tok * ld_xn, wg + hv * 12);
        const float gate = bf16_round(3.f * bf16_round(1.f / (1.f + __expf(-z))));
        const __nv_bfloat16* e = ve + (size_t)idx[tok] * (Hkv * 128) + hv * 128;
        float a[8], b[8], ea[8], eb[8];
        unpack8(ca, a);
        unpack8(cb, b);
        unpack8(__ldg(reinterpret_cast<const uint4*>(e) + sub), ea);
        unpack8(__ldg(reinterpret_cast<const uint4*>(e) + 8 + sub), eb);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a[j] += bf16_round(gate * ea[j]);
          b[j] += bf16_round(gate * eb[j]);
        }
        *(reinterpret_cast<uint4*>(h) + sub) = pack8(a);
        *(reinterpret_cast<uint4*>(h) + 8 + sub) = pack8(b);
      }
    }
  }
}

// Backward, in place on dqkv (same layout as qkv). `qkv` holds the forward OUTPUT (post rope/norm).
__global__ void __launch_bounds__(128)
qkv_post_bwd_kernel(__nv_bfloat16* __restrict__ dqkv, const __nv_bfloat16* __restrict__ qkv, long long ld,
                    int H, int Hkv, const __nv_bfloat16* __restrict__ cos_t,
                    const __nv_bfloat16* __restrict__ sin_t, int T, const float* __restrict__ rstd_in,
                    const __nv_bfloat16* __restrict__ xn, long long ld_xn, const float* __restrict__ wg,
                    const __nv_bfloat16* __restrict__ ve, const long long* __restrict__ idx,
                    float* __restrict__ dve /* [V, Hkv*128] fp32 */, float* __restrict__ dwg /* [Hkv,12] */,
                    float* __restrict__ dgate_x /* [M,12] */, float* __restrict__ amax_qk /* max |dq|, |dk| or null */,
                    int M) {
  __shared__ float s_dwg[32 * 12];     // Hkv <= 32
  __shared__ float s_dz[4][32];        // per warp, per kv head
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, grp = lane >> 3;
  const int n_rot = H + Hkv;
  const int n_items = n_rot + (ve ? Hkv : 0);
  for (int i = threadIdx.x; i < Hkv * 12; i += blockDim.x) s_dwg[i] = 0.f;
  __syncthreads();
  float mxqk = 0.f;
  for (int tok = blockIdx.x * 4 + warp; tok < M; tok += gridDim.x * 4) {
    const int t = tok % T;
    __nv_bfloat16* drow = dqkv + (size_t)tok * ld;
    const __nv_bfloat16* row = qkv + (size_t)tok * ld;
    float c[8], s[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(cos_t + (size_t)t * 64) + sub), c);
    unpack8(__ldg(reinterpret_cast<const uint4*>(sin_t + (size_t)t * 64) + sub), s);
    // in place on dqkv: the next item's gradient pieces (and, for rotary heads, its forward outputs) are requested
    // before the current item's results are stored (see the forward kernel)
    uint4 nga = make_uint4(0, 0, 0, 0), ngb = nga, nya = nga, nyb = nga;
    if (grp < n_items) {
      nga = *(reinterpret_cast<const uint4*>(drow + (size_t)grp * 128) + sub);
      ngb = *(reinterpret_cast<const uint4*>(drow + (size_t)grp * 128) + 8 + sub);
      if (grp < n_rot) {
        nya = *(reinterpret_cast<const uint4*>(row + (size_t)grp * 128) + sub);
        nyb = *(reinterpret_cast<const uint4*>(row + (size_t)grp * 128) + 8 + sub);
      }
    }
    for (int base = 0; base < n_items; base += 4) {
      const int item = base + grp;
      const uint4 cga = nga, cgb = ngb, cya = nya, cyb = nyb;
      if (item + 4 < n_items) {
        nga = *(reinterpret_cast<const uint4*>(drow + (size_t)(item + 4) * 128) + sub);
        ngb = *(reinterpret_cast<const uint4*>(drow + (size_t)(item + 4) * 128) + 8 + sub);
        if (item + 4 < n_rot) {
          nya = *(reinterpret_cast<const uint4*>(row + (size_t)(item + 4) * 128) + sub);
          nyb = *(reinterpret_cast<const uint4*>(row + (size_t)(item + 4) * 128) + 8 + sub);
        }
      }
      if (item < n_rot) {
        __nv_bfloat16* dh = drow + (size_t)item * 128;
        float ya[8], yb[8], ga[8], gb[8];
        unpack8(cya, ya);
        unpack8(cyb, yb);
        unpack8(cga, ga);
        unpack8(cgb, gb);
        const float rstd = rstd_in[(size_t)tok * n_rot + item];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ya[j] *= (1.f / 1.2f); yb[j] *= (1.f / 1.2f);     // xhat
          ga[j] *= 1.2f; gb[j] *= 1.2f;                     // grad wrt xhat
          dot += ga[j] * ya[j] + gb[j] * yb[j];
        }
        dot = group8_sum(dot, grp) * (1.f / 128.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d1 = rstd * (ga[j] - ya[j] * dot);    // grad wrt rotated values
          const float d2 = rstd * (gb[j] - yb[j] * dot);
          ga[j] = d1 * c[j] - d2 * s[j];                    // inverse rotation
          gb[j] = d1 * s[j] + d2 * c[j];
          mxqk = fmaxf(mxqk, fmaxf(fabsf(ga[j]), fabsf(gb[j])));
        }
        *(reinterpret_cast<uint4*>(dh) + sub) = pack8(ga);
        *(reinterpret_cast<uint4*>(dh) + 8 + sub) = pack8(gb);
      } else if (item < n_items) {
        const int hv = item - n_rot;
        const float z = ve_gate_value(xn + (size_t)tok * ld_xn, wg + hv * 12);
        const float sg = 1.f / (1.f + __expf(-z));
        const float gate = 3.f * sg;
        const size_t erow = (size_t)idx[tok] * (Hkv * 128) + hv * 128;
        float ga[8], gb[8], ea[8], eb[8];
        unpack8(cga, ga);
        unpack8(cgb, gb);
        unpack8(__ldg(reinterpret_cast<const uint4*>(ve + erow) + sub), ea);
        unpack8(__ldg(reinterpret_cast<const uint4*>(ve + erow) + 8 + sub), eb);
        float dg = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) dg += ga[j] * ea[j] + gb[j] * eb[j];
        dg = group8_sum(dg, grp);
        float* dst = dve + erow;
#pragma unroll
        for (int j = 0; j < 8; j += 4) {
          atomicAdd(reinterpret_cast<float4*>(dst + sub * 8 + j),
                    make_float4(gate * ga[j], gate * ga[j + 1], gate * ga[j + 2], gate * ga[j + 3]));
          atomicAdd(reinterpret_cast<float4*>(dst + 64 + sub * 8 + j),
                    make_float4(gate * gb[j], gate * gb[j + 1], gate * gb[j + 2], gate * gb[j + 3]));
        }
        if (sub == 0) s_dz[warp][hv] = dg * 3.f * sg * (1.f - sg);
      }
    }
    if (ve) {
      __syncwarp();
      // d(gate logits) -> dWg (block partial) and the 12-column gradient into xn
      const __nv_bfloat16* xr = xn + (size_t)tok * ld_xn;
      if (lane < 12) {
        float acc = 0.f;
        const float xv = __bfloat162float(xr[lane]);
        for (int hv = 0; hv < Hkv; ++hv) {
          const float dz = s_dz[warp][hv];
          acc += dz * wg[hv * 12 + lane];
          atomicAdd(&s_dwg[hv * 12 + lane], dz * xv);
        }
        dgate_x[(size_t)tok * 12 + lane] = acc;
      }
      __syncwarp();
    }
  }
  __syncthreads();
  if (ve)
    for (int i = threadIdx.x; i < Hkv * 12; i += blockDim.x) atomicAdd(dwg + i, s_dwg[i]);
  if (amax_qk) publish_absmax(mxqk * 1.00390625f, amax_qk, lane);   // margin for the bf16 rounding of the stores
}

// -------------------------------------------------------------------------- embedding
// x[t] = e[t] + lam*sigmoid(<e[t][:24], w>) * e[t-1]   (t >= 1 within a sequence), e = rmsnorm(wte[idx])
template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32)
embed_fwd_kernel(const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ wte,
                 const float* __restrict__ gate_w /* [24] */, const float* __restrict__ lam,
                 __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ e_last /* [B,C] or null */,
                 int M, int T, int C) {
  const int lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  const float l = bf16_round(lam[0]);
  for (int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); row < M; row += gridDim.x * ROW_WARPS) {
    const int t = row % T;
    RowF<NV> e, p;
    load_row(e, wte + (size_t)idx[row] * C, nvec, lane);
    float rstd = rsqrtf(row_sumsq(e) / C + RMS_EPS);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) e.v[i][j] = bf16_round(e.v[i][j] * rstd);
    if (e_last && t == T - 1) store_row(e, e_last + (size_t)(row / T) * C, nvec, lane);
    if (t > 0) {
      load_row(p, wte + (size_t)idx[row - 1] * C, nvec, lane);
      rstd = rsqrtf(row_sumsq(p) / C + RMS_EPS);
      float z = 0.f;
      if (lane < 3) {
#pragma unroll
        for (int j = 0; j < 8; ++j) z += e.v[0][j] * bf16_round(gate_w[lane * 8 + j]);
      }
      z = bf16_round(warp_sum(z));
      const float g = bf16_round(l * bf16_round(1.f / (1.f + __expf(-z))));
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) e.v[i][j] += bf16_round(g * bf16_round(p.v[i][j] * rstd));
    }
    store_row(e, x + (size_t)row * C, nvec, lane);
  }
}

// Backward of the above into a dense fp32 gradient table (atomic adds) and the gate scalars.
template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32)
embed_bwd_kernel(const __nv_bfloat16* __restrict__ dx, const long long* __restrict__ idx,
                 const __nv_bfloat16* __restrict__ wte, const float* __restrict__ gate_w,
                 const float* __restrict__ lam, float* __restrict__ dwte, float* __restrict__ dgate_w,
                 float* __restrict__ dlam, int M, int T, int C) {
  __shared__ float s_dw[24];
  __shared__ float s_dl;
  const int lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  const float l = lam[0];
  if (threadIdx.x < 24) s_dw[threadIdx.x] = 0.f;
  if (threadIdx.x == 0) s_dl = 0.f;
  __syncthreads();
  for (int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); row < M; row += gridDim.x * ROW_WARPS) {
    const int t = row % T;
    // de[t] = dx[t] + g[t+1]*dx[t+1] + (gate-logit grad of position t on the first 24 channels)
    RowF<NV> raw, e, de, tmp;
    load_row(raw, wte + (size_t)idx[row] * C, nvec, lane);
    const float rstd = rsqrtf(row_sumsq(raw) / C + RMS_EPS);
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) e.v[i][j] = raw.v[i][j] * rstd;
    load_row(de, dx + (size_t)row * C, nvec, lane);
    if (t > 0) {
      // this position's own gate: z = <e[:24], w>, g = l*sigmoid(z); dg = <dx[t], e[t-1]>
      load_row(tmp, wte + (size_t)idx[row - 1] * C, nvec, lane);
      const float rp = rsqrtf(row_sumsq(tmp) / C + RMS_EPS);
      const float dgv = row_dot(de, tmp) * rp;
      float z = 0.f;
      if (lane < 3) {
#pragma unroll
        for (int j = 0; j < 8; ++j) z += e.v[0][j] * gate_w[lane * 8 + j];
      }
      z = warp_sum(z);
      const float sg = 1.f / (1.f + __expf(-z));
      const float dz = dgv * l * sg * (1.f - sg);
      if (lane < 3) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          atomicAdd(&s_dw[lane * 8 + j], dz * e.v[0][j]);
          de.v[0][j] += dz * gate_w[lane * 8 + j];
        }
      }
      if (lane == 0) atomicAdd(&s_dl, dgv * sg);
    }
    if (t + 1 < T) {
      // contribution through the next position's smear: g[t+1] * dx[t+1]
      RowF<NV> en;
      load_row(en, wte + (size_t)idx[row + 1] * C, nvec, lane);
      const float rn = rsqrtf(row_sumsq(en) / C + RMS_EPS);
      float z = 0.f;
      if (lane < 3) {
#pragma unroll
        for (int j = 0; j < 8; ++j) z += en.v[0][j] * rn * gate_w[lane * 8 + j];
      }
      z = warp_sum(z);
      const float g = l / (1.f + __expf(-z));
      load_row(tmp, dx + (size_t)(row + 1) * C, nvec, lane);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) de.v[i][j] += g * tmp.v[i][j];
    }
    // through the rmsnorm to the raw embedding row, then scatter-add
    rmsnorm_bwd_inplace(de, raw, C);
    float* dst = dwte + (size_t)idx[row] * C;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + 32 * i;
      if (vi < nvec) {
        atomicAdd(reinterpret_cast<float4*>(dst + vi * 8),
                  make_float4(de.v[i][0], de.v[i][1], de.v[i][2], de.v[i][3]));
        atomicAdd(reinterpret_cast<float4*>(dst + vi * 8 + 4),
                  make_float4(de.v[i][4], de.v[i][5], de.v[i][6], de.v[i][7]));
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < 24) atomicAdd(dgate_w + threadIdx.x, s_dw[threadIdx.x]);
  if (threadIdx.x == 0) atomicAdd(dlam, s_dl);
}

// ---------------------------------------------------------------------------- casts
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(src)[2 * i];
    const float4 b = reinterpret_cast<const float4*>(src)[2 * i + 1];
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    reinterpret_cast<uint4*>(dst)[i] = pack8(f);
  }
}

// ============================================================================ launchers
static inline int row_grid(int M) {
  const int need = (M + ROW_WARPS - 1) / ROW_WARPS;
  const int cap = 148 * 16;
  return need < cap ? need : cap;
}

#define NC_DISPATCH_NV(C, ...)                                        \
  do {                                                                \
    if ((C) <= 1024) { constexpr int NV = 4; __VA_ARGS__; }           \
    else if ((C) <= 2048) { constexpr int NV = 8; __VA_ARGS__; }      \
    else if ((C) <= 4096) { constexpr int NV = 16; __VA_ARGS__; }     \
    else return cudaErrorInvalidValue;                                \
  } while (0)

cudaError_t mixnorm_fwd(const void* x, const void* x0, const float* lam_r, const float* lam_0, int layer,
                        void* xm, void* xn, float* amax_xn, int M, int C, cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (mixnorm_fwd_kernel<NV><<<row_grid(M), ROW_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)x0, lam_r, lam_0, layer,
      (__nv_bfloat16*)xm, (__nv_bfloat16*)xn, amax_xn, M, C)));
  return cudaGetLastError();
}

cudaError_t norm_fwd(const void* x, void* y, float* amax_y, int M, int C, cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (norm_fwd_kernel<NV><<<row_grid(M), ROW_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, amax_y, M, C)));
  return cudaGetLastError();
}

cudaError_t normadd_bwd(const void* dy, const void* x, const void* dres, void* dx, float* amax_dx, int M, int C,
                        cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (normadd_bwd_kernel<NV><<<row_grid(M), ROW_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, amax_dx, M,
      C)));
  return cudaGetLastError();
}

cudaError_t mixnorm_bwd(const void* dxn, const void* dres, const float* dgate, const void* xm, const void* x,
                        const void* x0, const float* lam_r, const float* lam_0, int layer, void* dx, void* dx0,
                        int accumulate_dx0, float* dlam_r, float* dlam_0, float* amax_dx, int M, int C,
                        cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (mixnorm_bwd_kernel<NV><<<row_grid(M), ROW_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)dxn, (const __nv_bfloat16*)dres, dgate, (const __nv_bfloat16*)xm,
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)x0, lam_r, lam_0, layer, (__nv_bfloat16*)dx,
      (__nv_bfloat16*)dx0, accumulate_dx0, dlam_r, dlam_0, amax_dx, M, C)));
  return cudaGetLastError();
}

cudaError_t backout_norm_fwd(const void* x, const void* xb, const float* lam, void* y, int M, int C, cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (backout_norm_fwd_kernel<NV><<<row_grid(M), ROW_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)xb, lam, (__nv_bfloat16*)y, M, C)));
  return cudaGetLastError();
}

cudaError_t backout_norm_bwd(const void* dy, const void* x, const void* xb, const float* lam, void* dx, void* dxb,
                             float* dlam, int M, int C, cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (backout_norm_bwd_kernel<NV><<<row_grid(M), ROW_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)xb, lam, (__nv_bfloat16*)dx,
      (__nv_bfloat16*)dxb, dlam, M, C)));
  return cudaGetLastError();
}

cudaError_t qkv_post_fwd(void* qkv, long long ld, int H, int Hkv, const void* cos_t, const void* sin_t, int T,
                         float* rstd, const void* xn, long long ld_xn, const float* wg, const void* ve,
                         const long long* idx, int M, cudaStream_t s) {
  if (Hkv > 32 || (ld & 7)) return cudaErrorInvalidValue;
  const int grid = (M + 3) / 4 < 148 * 16 ? (M + 3) / 4 : 148 * 16;
  qkv_post_fwd_kernel<<<grid, 128, 0, s>>>((__nv_bfloat16*)qkv, ld, H, Hkv, (const __nv_bfloat16*)cos_t,
                                           (const __nv_bfloat16*)sin_t, T, rstd, (const __nv_bfloat16*)xn, ld_xn,
                                           wg, (const __nv_bfloat16*)ve, idx, M);
  return cudaGetLastError();
}

cudaError_t qkv_post_bwd(void* dqkv, const void* qkv, long long ld, int H, int Hkv, const void* cos_t,
                         const void* sin_t, int T, const float* rstd, const void* xn, long long ld_xn,
                         const float* wg, const void* ve, const long long* idx, float* dve, float* dwg,
                         float* dgate_x, float* amax_qk, int M, cudaStream_t s) {
  if (Hkv > 32 || (ld & 7)) return cudaErrorInvalidValue;
  const int grid = (M + 3) / 4 < 148 * 8 ? (M + 3) / 4 : 148 * 8;
  qkv_post_bwd_kernel<<<grid, 128, 0, s>>>((__nv_bfloat16*)dqkv, (const __nv_bfloat16*)qkv, ld, H, Hkv,
                                           (const __nv_bfloat16*)cos_t, (const __nv_bfloat16*)sin_t, T, rstd,
                                           (const __nv_bfloat16*)xn, ld_xn, wg, (const __nv_bfloat16*)ve, idx, dve,
                                           dwg, dgate_x, amax_qk, M);
  return cudaGetLastError();
}

cudaError_t embed_fwd(const long long* idx, const void* wte, const float* gate_w, const float* lam, void* x,
                      void* e_last, int M, int T, int C, cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (embed_fwd_kernel<NV><<<row_grid(M), ROW_WARPS * 32, 0, s>>>(
      idx, (const __nv_bfloat16*)wte, gate_w, lam, (__nv_bfloat16*)x, (__nv_bfloat16*)e_last, M, T, C)));
  return cudaGetLastError();
}

cudaError_t embed_bwd(const void* dx, const long long* idx, const void* wte, const float* gate_w, const float* lam,
                      float* dwte, float* dgate_w, float* dlam, int M, int T, int C, cudaStream_t s) {
  if (C & 7) return cudaErrorInvalidValue;
  NC_DISPATCH_NV(C, (embed_bwd_kernel<NV><<<row_grid(M) / 2 + 1, ROW_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)dx, idx, (const __nv_bfloat16*)wte, gate_w, lam, dwte, dgate_w, dlam, M, T, C)));
  return cudaGetLastError();
}

cudaError_t cast_f32_bf16(const float* src, void* dst, size_t n, cudaStream_t s) {
  if (n & 7) return cudaErrorInvalidValue;
  const size_t n8 = n >> 3;
  const int grid = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  if (n8) cast_f32_bf16_kernel<<<grid, 256, 0, s>>>(src, (__nv_bfloat16*)dst, n8);
  return cudaGetLastError();
}

}  // namespace nc
