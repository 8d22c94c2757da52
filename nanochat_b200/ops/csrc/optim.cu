// Optimizer kernels: fused AdamW and the elementwise stages of the Muon step
// (the matrix products of the polar iteration run on the tcgen05 GEMM in gemm.cu).
//
// Muon on a stack of k matrices (r x c), in order:
//   muon_momentum   buf <- lerp(buf, g, 1-mu); u = lerp(g, buf, mu) (Nesterov); X = bf16(u);
//                   rowss[i] = sum_j X_ij^2
//   muon_equilibrate X <- bf16(X * (||X||_F/sqrt(r)) / max(||row_i||, 1e-6)); accumulates ||X'||_F^2
//   muon_scale      X <- X / (||X'||_F * 1.01 + 1e-6)
//   (5 polar-express steps: A = X X^T, B = bA + cAA, X = aX + BX   -- GEMMs)
//   muon_sumsq      per-row or per-column sums of squares of X
//   muon_stats      Frobenius renorm to sqrt(min(r,c)), factored second moment (NorMuon) and the
//                   resulting per-row/col scale; one CTA per matrix
//   muon_apply      p <- p - lr*scale_i*X - lr*wd*p*[X*p >= 0]; refreshes the bf16 shadow of p
#include "fused.h"
#include "optim.h"
#include "rowops.cuh"

namespace nc {

// ------------------------------------------------------------------------------ AdamW
template <typename PT, typename GT>
__global__ void adamw_kernel(PT* __restrict__ p, const GT* __restrict__ g, PT* __restrict__ m, PT* __restrict__ v,
                             __nv_bfloat16* __restrict__ shadow, size_t n, AdamWArgs a) {
  const float step_size = a.lr / a.bias1;
  const float inv_bias2 = 1.f / a.bias2;
  const float decay = 1.f - a.lr * a.wd;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float pv = static_cast<float>(p[i]);
    const float gv = static_cast<float>(g[i]) * a.grad_scale;
    float mv = static_cast<float>(m[i]);
    float vv = static_cast<float>(v[i]);
    pv *= decay;
    mv += (1.f - a.beta1) * (gv - mv);
    vv += (1.f - a.beta2) * (gv * gv - vv);
    const float denom = sqrtf(vv * inv_bias2) + a.eps;
    pv -= step_size * (mv / denom);
    p[i] = static_cast<PT>(pv);
    m[i] = static_cast<PT>(mv);
    v[i] = static_cast<PT>(vv);
    if (shadow) shadow[i] = __float2bfloat16_rn(pv);
  }
}

static inline int ew_grid(size_t n, int threads) {
  size_t need = (n + threads - 1) / threads;
  size_t cap = 148 * 16;
  return (int)(need < cap ? (need ? need : 1) : cap);
}

cudaError_t adamw_step(void* p, int p_bf16, const void* g, int g_bf16, void* m, void* v, void* shadow, size_t n,
                       AdamWArgs a, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const int grid = ew_grid(n, 256);
  if (p_bf16 && g_bf16)
    adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)p, (const __nv_bfloat16*)g,
                                                                    (__nv_bfloat16*)m, (__nv_bfloat16*)v, nullptr, n, a);
  else if (p_bf16)
    adamw_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>((__nv_bfloat16*)p, (const float*)g, (__nv_bfloat16*)m,
                                                            (__nv_bfloat16*)v, nullptr, n, a);
  else if (g_bf16)
    adamw_kernel<float, __nv_bfloat16><<<grid, 256, 0, s>>>((float*)p, (const __nv_bfloat16*)g, (float*)m, (float*)v,
                                                            (__nv_bfloat16*)shadow, n, a);
  else
    adamw_kernel<float, float><<<grid, 256, 0, s>>>((float*)p, (const float*)g, (float*)m, (float*)v,
                                                    (__nv_bfloat16*)shadow, n, a);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------- Muon
// One warp per matrix row; c may be small (12) or large (6656), so rows are walked with a lane stride.
__global__ void __launch_bounds__(128)
muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ buf, __nv_bfloat16* __restrict__ X,
                     float* __restrict__ rowss, float mu, float grad_scale, long long rows, int c) {
  const int lane = threadIdx.x & 31;
  const bool vec = (c & 3) == 0;            // rows of whole float4s (every matrix the fused path sees)
  for (long long row = blockIdx.x * 4ll + (threadIdx.x >> 5); row < rows; row += gridDim.x * 4ll) {
    const float* gr = g + row * c;
    float* br = buf + row * c;
    __nv_bfloat16* xr = X + row * c;
    float ss = 0.f;
    if (vec) {
      for (int j = lane * 4; j < c; j += 128) {
        const float4 g4 = *reinterpret_cast<const float4*>(gr + j);
        const float4 b4 = *reinterpret_cast<const float4*>(br + j);
        float gv[4] = {g4.x * grad_scale, g4.y * grad_scale, g4.z * grad_scale, g4.w * grad_scale};
        float bv[4] = {b4.x, b4.y, b4.z, b4.w};
        __nv_bfloat16 xb[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          bv[e] += (1.f - mu) * (gv[e] - bv[e]);
          const float u = gv[e] + mu * (bv[e] - gv[e]);
          xb[e] = __float2bfloat16_rn(u);
          const float xf = __bfloat162float(xb[e]);
          ss += xf * xf;
        }
        *reinterpret_cast<float4*>(br + j) = make_float4(bv[0], bv[1], bv[2], bv[3]);
        __nv_bfloat162 lo(xb[0], xb[1]), hi(xb[2], xb[3]);
        *reinterpret_cast<uint2*>(xr + j) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      }
    } else {
      for (int j = lane; j < c; j += 32) {
        const float gv = gr[j] * grad_scale;
        float bv = br[j];
        bv += (1.f - mu) * (gv - bv);
        br[j] = bv;
        const float u = gv + mu * (bv - gv);
        const __nv_bfloat16 xb = __float2bfloat16_rn(u);
        xr[j] = xb;
        const float xf = __bfloat162float(xb);
        ss += xf * xf;
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) rowss[row] = ss;
  }
}

// total[mat] = sum of rowss over the matrix' rows (deterministic: one CTA per matrix, fixed order)
__global__ void __launch_bounds__(256)
muon_total_kernel(const float* __restrict__ rowss, float* __restrict__ total, int r) {
  __shared__ float red[8];
  const int mat = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < r; i += 256) s += rowss[(size_t)mat * r + i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    total[mat] = t;
  }
}

__global__ void __launch_bounds__(128)
muon_equilibrate_kernel(__nv_bfloat16* __restrict__ X, const float* __restrict__ rowss,
                        const float* __restrict__ total, float* __restrict__ rowss2, long long rows, int r, int c) {
  const int lane = threadIdx.x & 31;
  const bool vec = (c & 7) == 0;            // rows of whole 16-byte vectors
  for (long long row = blockIdx.x * 4ll + (threadIdx.x >> 5); row < rows; row += gridDim.x * 4ll) {
    const int mat = (int)(row / r);
    const float target = sqrtf(total[mat]) * rsqrtf((float)r);
    const float rn = fmaxf(sqrtf(rowss[row]), 1e-6f);
    const float scale = bf16_round(target / rn);
    __nv_bfloat16* xr = X + row * c;
    float ss = 0.f;
    if (vec) {
      for (int j = lane * 8; j < c; j += 256) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + j), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[e] = bf16_round(f[e] * scale);
          ss += f[e] * f[e];
        }
        *reinterpret_cast<uint4*>(xr + j) = pack8(f);
      }
    } else {
      for (int j = lane; j < c; j += 32) {
        const __nv_bfloat16 xb = __float2bfloat16_rn(__bfloat162float(xr[j]) * scale);
        xr[j] = xb;
        const float xf = __bfloat162float(xb);
        ss += xf * xf;
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) rowss2[row] = ss;
  }
}

__global__ void muon_scale_kernel(__nv_bfloat16* __restrict__ X, const float* __restrict__ total2, size_t per_mat,
                                  size_t n) {
  if ((per_mat & 7) == 0) {                 // 16-byte vectors never straddle two matrices
    const size_t n8 = n >> 3, per_mat8 = per_mat >> 3;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
      const int mat = (int)(i / per_mat8);
      const float nrm = bf16_round(sqrtf(total2[mat]));
      const float den = bf16_round(bf16_round(nrm * 1.01f) + 1e-6f);
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(X)[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = f[e] / den;
      reinterpret_cast<uint4*>(X)[i] = pack8(f);
    }
    return;
  }
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int mat = (int)(i / per_mat);
    const float nrm = bf16_round(sqrtf(total2[mat]));
    const float den = bf16_round(bf16_round(nrm * 1.01f) + 1e-6f);
    X[i] = __float2bfloat16_rn(__bfloat162float(X[i]) / den);
  }
}

// ss[mat, i] over rows (per_row=1: i indexes rows, reduce over columns) or columns (per_row=0).
__global__ void __launch_bounds__(128)
muon_sumsq_rows_kernel(const __nv_bfloat16* __restrict__ X, float* __restrict__ ss, long long rows, int c) {
  const int lane = threadIdx.x & 31;
  const bool vec = (c & 7) == 0;
  for (long long row = blockIdx.x * 4ll + (threadIdx.x >> 5); row < rows; row += gridDim.x * 4ll) {
    const __nv_bfloat16* xr = X + row * c;
    float s = 0.f;
    if (vec) {
      for (int j = lane * 8; j < c; j += 256) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + j), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += f[e] * f[e];
      }
    } else {
      for (int j = lane; j < c; j += 32) { const float f = __bfloat162float(xr[j]); s += f * f; }
    }
    s = warp_sum(s);
    if (lane == 0) ss[row] = s;
  }
}
__global__ void __launch_bounds__(256)
muon_sumsq_cols_kernel(const __nv_bfloat16* __restrict__ X, float* __restrict__ ss, int r, int c) {
  // grid: (ceil(c/256), k); each thread owns one column of one matrix and walks the rows
  const int mat = blockIdx.y;
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col >= c) return;
  const __nv_bfloat16* xm = X + (size_t)mat * r * c + col;
  float s = 0.f;
  for (int i = 0; i < r; ++i) { const float f = __bfloat162float(xm[(size_t)i * c]); s += f * f; }
  ss[(size_t)mat * c + col] = s;
}

// One CTA per matrix: n = number of kept entries (r if red over columns, else c), n_red = the other dim.
__global__ void __launch_bounds__(256)
muon_stats_kernel(const float* __restrict__ ss, float* __restrict__ second_buf, float* __restrict__ scale_out,
                  int n, int n_red, float target_norm, float beta2) {
  __shared__ float red[8];
  __shared__ float bcast;
  const int mat = blockIdx.x;
  const float* s = ss + (size_t)mat * n;
  float* sb = second_buf + (size_t)mat * n;
  float* so = scale_out + (size_t)mat * n;
  auto block_total = [&](float v) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) { float t = 0.f; for (int w = 0; w < 8; ++w) t += red[w]; bcast = t; }
    __syncthreads();
    const float out = bcast;
    __syncthreads();
    return out;
  };
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) acc += s[i];
  const float fro2 = block_total(acc);
  const float rho = target_norm / fmaxf(sqrtf(fro2), 1e-6f);         // Frobenius renorm factor
  // v_mean_i = rho^2 * ss_i / n_red ; v_norm^2 = sum_i v_mean_i * n_red = rho^2 * fro2
  const float v_norm = rho * sqrtf(fro2);
  float acc2 = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) {
    const float v_mean = rho * rho * s[i] / (float)n_red;
    float b = sb[i];
    b += (1.f - beta2) * (v_mean - b);
    sb[i] = b;
    const float step = rsqrtf(fmaxf(b, 1e-10f));
    so[i] = step;
    acc2 += v_mean * (float)n_red * step * step;
  }
  const float v_norm_new = sqrtf(block_total(acc2));
  const float fin = v_norm / fmaxf(v_norm_new, 1e-10f);
  for (int i = threadIdx.x; i < n; i += 256) so[i] = so[i] * fin * rho;
}

__global__ void muon_apply_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ X,
                                  const float* __restrict__ scale, __nv_bfloat16* __restrict__ shadow, int r, int c,
                                  int per_row, float lr, float wd, size_t n) {
  const size_t per_mat = (size_t)r * c;
  if ((c & 7) == 0) {                       // 8 elements per thread: they share a row
    const size_t n8 = n >> 3, per_mat8 = per_mat >> 3;
    const int c8 = c >> 3;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
      const size_t mat = i / per_mat8;
      const size_t rem = i - mat * per_mat8;
      const int row = (int)(rem / c8), col = (int)(rem - (size_t)row * c8) * 8;
      float xv[8], pv[8], sc[8];
      unpack8(reinterpret_cast<const uint4*>(X)[i], xv);
      const float4 p0 = reinterpret_cast<const float4*>(p)[2 * i], p1 = reinterpret_cast<const float4*>(p)[2 * i + 1];
      pv[0] = p0.x; pv[1] = p0.y; pv[2] = p0.z; pv[3] = p0.w; pv[4] = p1.x; pv[5] = p1.y; pv[6] = p1.z; pv[7] = p1.w;
      if (per_row) {
        const float sv = scale[mat * r + row];
#pragma unroll
        for (int e = 0; e < 8; ++e) sc[e] = sv;
      } else {
        const float4 s0 = *reinterpret_cast<const float4*>(scale + mat * c + col);
        const float4 s1 = *reinterpret_cast<const float4*>(scale + mat * c + col + 4);
        sc[0] = s0.x; sc[1] = s0.y; sc[2] = s0.z; sc[3] = s0.w; sc[4] = s1.x; sc[5] = s1.y; sc[6] = s1.z; sc[7] = s1.w;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float gv = xv[e] * sc[e];
        const float mask = (gv * pv[e] >= 0.f) ? 1.f : 0.f;
        pv[e] -= lr * gv + lr * wd * pv[e] * mask;
      }
      reinterpret_cast<float4*>(p)[2 * i] = make_float4(pv[0], pv[1], pv[2], pv[3]);
      reinterpret_cast<float4*>(p)[2 * i + 1] = make_float4(pv[4], pv[5], pv[6], pv[7]);
      if (shadow) reinterpret_cast<uint4*>(shadow)[i] = pack8(pv);
    }
    return;
  }
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t mat = i / per_mat;
    const size_t rem = i - mat * per_mat;
    const int row = (int)(rem / c), col = (int)(rem - (size_t)row * c);
    const float sc = per_row ? scale[mat * r + row] : scale[mat * c + col];
    const float gv = __bfloat162float(X[i]) * sc;
    float pv = p[i];
    const float mask = (gv * pv >= 0.f) ? 1.f : 0.f;
    pv -= lr * gv + lr * wd * pv * mask;
    p[i] = pv;
    if (shadow) shadow[i] = __float2bfloat16_rn(pv);
  }
}

cudaError_t muon_momentum(const float* g, float* buf, void* X, float* rowss, float* total, float mu,
                          float grad_scale, int k, int r, int c, cudaStream_t s) {
  const long long rows = (long long)k * r;
  const int grid = (int)((rows + 3) / 4 < 148 * 16 ? (rows + 3) / 4 : 148 * 16);
  muon_momentum_kernel<<<grid, 128, 0, s>>>(g, buf, (__nv_bfloat16*)X, rowss, mu, grad_scale, rows, c);
  muon_total_kernel<<<k, 256, 0, s>>>(rowss, total, r);
  return cudaGetLastError();
}

cudaError_t muon_equilibrate(void* X, const float* rowss, const float* total, float* rowss2, float* total2, int k,
                             int r, int c, cudaStream_t s) {
  const long long rows = (long long)k * r;
  const int grid = (int)((rows + 3) / 4 < 148 * 16 ? (rows + 3) / 4 : 148 * 16);
  muon_equilibrate_kernel<<<grid, 128, 0, s>>>((__nv_bfloat16*)X, rowss, total, rowss2, rows, r, c);
  muon_total_kernel<<<k, 256, 0, s>>>(rowss2, total2, r);
  const size_t n = (size_t)k * r * c;
  muon_scale_kernel<<<ew_grid(n, 256), 256, 0, s>>>((__nv_bfloat16*)X, total2, (size_t)r * c, n);
  return cudaGetLastError();
}

cudaError_t muon_total(const float* rowss, float* total, int k, int r, cudaStream_t s) {
  if (k == 0) return cudaSuccess;
  muon_total_kernel<<<k, 256, 0, s>>>(rowss, total, r);
  return cudaGetLastError();
}

cudaError_t muon_stats(const void* X, float* second_buf, float* ss_scratch, float* scale_scratch, int k, int r, int c,
                       float beta2, cudaStream_t s) {
  const int per_row = r >= c;                 // factored second moment keeps rows when r >= c
  const int n = per_row ? r : c, n_red = per_row ? c : r;
  if (per_row) {
    const long long rows = (long long)k * r;
    const int grid = (int)((rows + 3) / 4 < 148 * 16 ? (rows + 3) / 4 : 148 * 16);
    muon_sumsq_rows_kernel<<<grid, 128, 0, s>>>((const __nv_bfloat16*)X, ss_scratch, rows, c);
  } else {
    dim3 grid((c + 255) / 256, k);
    muon_sumsq_cols_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)X, ss_scratch, r, c);
  }
  const float target = sqrtf((float)(r < c ? r : c));
  muon_stats_kernel<<<k, 256, 0, s>>>(ss_scratch, second_buf, scale_scratch, n, n_red, target, beta2);
  return cudaGetLastError();
}

cudaError_t muon_finish(float* p, const void* X, float* second_buf, float* ss_scratch, float* scale_scratch,
                        void* shadow, int k, int r, int c, float lr, float wd, float beta2, cudaStream_t s) {
  cudaError_t e = muon_stats(X, second_buf, ss_scratch, scale_scratch, k, r, c, beta2, s);
  if (e != cudaSuccess) return e;
  const size_t total = (size_t)k * r * c;
  muon_apply_kernel<<<ew_grid(total, 256), 256, 0, s>>>(p, (const __nv_bfloat16*)X, scale_scratch,
                                                        (__nv_bfloat16*)shadow, r, c, r >= c, lr, wd, total);
  return cudaGetLastError();
}

}  // namespace nc
