// Optimizer kernels fused with their collectives over NVLink peer memory.
//
// Every rank maps the same symmetric allocations of all ranks (gradient buffers, bf16 parameter
// shadows, a small signal pad). A kernel receives the N base pointers of a buffer and addresses
// peer r's copy directly:
//
//   p2p_barrier        one CTA: release-store this rank's epoch into every peer's pad, then
//                      acquire-spin (bounded) until every peer's epoch has arrived here
//   p2p_adamw          reduce-scatter + AdamW + all-gather in one pass over the rank's row slice:
//                      pull the slice of every rank's gradient (16-byte ld.global.cg over NVLink),
//                      sum in rank order in fp32, x 1/N, update the local fp32/bf16 state, and store
//                      the new bf16 values into every rank's parameter/shadow buffer
//   p2p_muon_momentum  the Muon momentum stage (optim.cu) with the gradient averaged from all ranks
//   p2p_muon_apply     the Muon parameter update (optim.cu: muon_apply) whose bf16 result is stored into every
//                      rank's shadow from the same registers: the all-gather is the update's write-back
//   p2p_bcast_shadow   bf16 values of this rank written to every peer (kept for callers that update elsewhere)
//   p2p_small_adamw    replicated parameters (< 1024 elements): every rank averages all ranks'
//                      gradients itself and applies AdamW to its own copy (no write-back needed)
//
// Sums are taken in rank order 0..N-1, so the result does not depend on timing. Plain peer loads
// and stores only: no multimem, no TMA on peer memory.
//
// A remote load takes a few microseconds, so what sets the pull rate is how many of them a thread has in flight.
// The pulling kernels are templates on the world size: a thread first issues the 16-byte loads of ALL ranks for its
// elements (2 x N independent loads), and only then adds them up in rank order.
#include "comm.h"
#include "rowops.cuh"

namespace nc {

constexpr unsigned long long P2P_WAIT_NS = 2000000000ull;

__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// pads.p[r] points at rank r's pad: int[MAX_RANKS] slots, slot s = last epoch announced by rank s.
__global__ void p2p_barrier_kernel(PeerPtrs pads, int rank, int world, int epoch, int* status) {
  const int t = threadIdx.x;
  __threadfence_system();     // order this rank's earlier global writes before the announcement
  if (t < world) st_release_sys(reinterpret_cast<int*>(pads.p[t]) + rank, epoch);
  if (t < world) {
    const int* slot = reinterpret_cast<const int*>(pads.p[rank]) + t;
    const unsigned long long t0 = gtimer();
    while (ld_acquire_sys(slot) < epoch) {
      if (gtimer() - t0 > P2P_WAIT_NS) {
        atomicCAS(status, 0, (5 << 24) | (t << 8) | (epoch & 0xff));   // ST_WAIT_PEER, which peer, which epoch
        break;
      }
      __nanosleep(200);
    }
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(__nv_bfloat16 a, __nv_bfloat16 b) {
  __nv_bfloat162 v(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// Gradients fp32. p: this rank's slice (fp32 master or bf16 table rows); out.p[r] + out_off: where the new
// bf16 values go on rank r (shadow of an fp32 master, or the bf16 table itself). n % 8 == 0.
// 128 threads and at most 64 registers per thread: one such CTA fits on an SM beside a resident tensor-core GEMM CTA
// (320 threads x 168 registers), so the pull can share the GPU with the polar iteration running on another stream.
template <bool P_BF16, int WORLD>
__global__ void __launch_bounds__(128, 8)
p2p_adamw_kernel(PeerPtrs grads, size_t grad_off, int world_rt, void* __restrict__ p,
                 void* __restrict__ m, void* __restrict__ v, PeerPtrs out, size_t out_off,
                 int write_local_out, int rank, size_t n, AdamWArgs a) {
  const int world = WORLD > 0 ? WORLD : world_rt;
  const float step_size = a.lr / a.bias1, inv_bias2 = 1.f / a.bias2, decay = 1.f - a.lr * a.wd;
  const float inv_world = 1.f / world;
  for (size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) * 8; i < n; i += (size_t)gridDim.x * blockDim.x * 8) {
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (WORLD > 0) {
      float4 x[WORLD > 0 ? WORLD : 1], y[WORLD > 0 ? WORLD : 1];
#pragma unroll
      for (int r = 0; r < WORLD; ++r) {          // every rank's loads are in flight before the first add
        const float* src = reinterpret_cast<const float*>(grads.p[r]) + grad_off + i;
        x[r] = ldcg4(src);
        y[r] = ldcg4(src + 4);
      }
#pragma unroll
      for (int r = 0; r < WORLD; ++r) {
        g[0] += x[r].x; g[1] += x[r].y; g[2] += x[r].z; g[3] += x[r].w;
        g[4] += y[r].x; g[5] += y[r].y; g[6] += y[r].z; g[7] += y[r].w;
      }
    } else {
      for (int r = 0; r < world; ++r) {
        const float* src = reinterpret_cast<const float*>(grads.p[r]) + grad_off + i;
        const float4 x = ldcg4(src), y = ldcg4(src + 4);
        g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w; g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
      }
    }
    float pv[8], mv[8], vv[8];
    if (P_BF16) {
      unpack8(reinterpret_cast<const uint4*>(p)[i / 8], pv);
      unpack8(reinterpret_cast<const uint4*>(m)[i / 8], mv);
      unpack8(reinterpret_cast<const uint4*>(v)[i / 8], vv);
    } else {
      const float4 *pp = reinterpret_cast<const float4*>(p) + i / 4, *mp = reinterpret_cast<const float4*>(m) + i / 4,
                   *vp = reinterpret_cast<const float4*>(v) + i / 4;
      const float4 p0 = pp[0], p1 = pp[1], m0 = mp[0], m1 = mp[1], v0 = vp[0], v1 = vp[1];
      pv[0] = p0.x; pv[1] = p0.y; pv[2] = p0.z; pv[3] = p0.w; pv[4] = p1.x; pv[5] = p1.y; pv[6] = p1.z; pv[7] = p1.w;
      mv[0] = m0.x; mv[1] = m0.y; mv[2] = m0.z; mv[3] = m0.w; mv[4] = m1.x; mv[5] = m1.y; mv[6] = m1.z; mv[7] = m1.w;
      vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gv = g[j] * inv_world * a.grad_scale;
      pv[j] *= decay;
      mv[j] += (1.f - a.beta1) * (gv - mv[j]);
      vv[j] += (1.f - a.beta2) * (gv * gv - vv[j]);
      pv[j] -= step_size * (mv[j] / (sqrtf(vv[j] * inv_bias2) + a.eps));
    }
    const uint4 packed = pack8(pv);
    if (P_BF16) {
      reinterpret_cast<uint4*>(p)[i / 8] = packed;
      reinterpret_cast<uint4*>(m)[i / 8] = pack8(mv);
      reinterpret_cast<uint4*>(v)[i / 8] = pack8(vv);
    } else {
      float4* pp = reinterpret_cast<float4*>(p) + i / 4;
      float4* mp = reinterpret_cast<float4*>(m) + i / 4;
      float4* vp = reinterpret_cast<float4*>(v) + i / 4;
      pp[0] = make_float4(pv[0], pv[1], pv[2], pv[3]); pp[1] = make_float4(pv[4], pv[5], pv[6], pv[7]);
      mp[0] = make_float4(mv[0], mv[1], mv[2], mv[3]); mp[1] = make_float4(mv[4], mv[5], mv[6], mv[7]);
      vp[0] = make_float4(vv[0], vv[1], vv[2], vv[3]); vp[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    }
    for (int r = 0; r < world; ++r) {
      if (r == rank && !write_local_out) continue;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out.p[r]) + out_off)[i / 8] = packed;
    }
  }
}

// Muon momentum with the gradient averaged over ranks. grads.p[r] + grad_off addresses the (k, r, c) chunk
// this rank owns inside rank r's gradient stack.
template <int WORLD>
__global__ void __launch_bounds__(128)
p2p_muon_momentum_kernel(PeerPtrs grads, size_t grad_off, int world_rt, float* __restrict__ buf,
                         __nv_bfloat16* __restrict__ X, float* __restrict__ rowss, float mu, long long rows, int c) {
  const int world = WORLD > 0 ? WORLD : world_rt;
  const int lane = threadIdx.x & 31;
  const float inv_world = 1.f / world;
  for (long long row = blockIdx.x * 4ll + (threadIdx.x >> 5); row < rows; row += gridDim.x * 4ll) {
    float* br = buf + row * c;
    __nv_bfloat16* xr = X + row * c;
    float ss = 0.f;
    for (int j = lane * 4; j < c; j += 128) {
      float4 g = make_float4(0, 0, 0, 0);
      if (WORLD > 0) {
        float4 x[WORLD > 0 ? WORLD : 1];
#pragma unroll
        for (int r = 0; r < WORLD; ++r)
          x[r] = ldcg4(reinterpret_cast<const float*>(grads.p[r]) + grad_off + row * c + j);
#pragma unroll
        for (int r = 0; r < WORLD; ++r) { g.x += x[r].x; g.y += x[r].y; g.z += x[r].z; g.w += x[r].w; }
      } else {
        for (int r = 0; r < world; ++r) {
          const float4 x = ldcg4(reinterpret_cast<const float*>(grads.p[r]) + grad_off + row * c + j);
          g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
        }
      }
      float gv[4] = {g.x * inv_world, g.y * inv_world, g.z * inv_world, g.w * inv_world};
      float4 b = *reinterpret_cast<float4*>(br + j);
      float bv[4] = {b.x, b.y, b.z, b.w};
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
      *reinterpret_cast<uint2*>(xr + j) = make_uint2(pack_bf16x2(xb[0], xb[1]), pack_bf16x2(xb[2], xb[3]));
    }
    ss = warp_sum(ss);
    if (lane == 0) rowss[row] = ss;
  }
}

// Muon's parameter update on this rank's chunk of a stack (k matrices of r x c fp32 masters; X the orthogonalised
// update in bf16; scale per row (per_row) or per column): p <- p - lr*scale*X - lr*wd*p*[X*p >= 0]. The new value is
// rounded to bf16 once and stored from registers into every rank's shadow stack at out_off (this rank's included):
// the parameter all-gather is this kernel's write-back. 8 elements per thread (c % 8 == 0: they share a row).
__global__ void __launch_bounds__(256)
p2p_muon_apply_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ X, const float* __restrict__ scale,
                      PeerPtrs out, size_t out_off, int world, int r, int c, int per_row, float lr, float wd,
                      size_t n8) {
  const size_t per_mat8 = (size_t)r * c / 8;
  const int c8 = c / 8;
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
    const uint4 packed = pack8(pv);
    for (int q = 0; q < world; ++q)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out.p[q]) + out_off)[i] = packed;
  }
}

// Copy n bf16 values from this rank's shadow chunk to the same offset of every peer's shadow buffer.
__global__ void p2p_bcast_kernel(const __nv_bfloat16* __restrict__ src, PeerPtrs dst, size_t dst_off, int world,
                                 int rank, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 val = reinterpret_cast<const uint4*>(src)[i];
    for (int r = 0; r < world; ++r) {
      if (r == rank) continue;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[r]) + dst_off)[i] = val;
    }
  }
}

// Push half of the reduce-scatter for gradients that no GEMM epilogue can deliver to their owner (embedding tables,
// whose gradient is a scatter-add, and any tensor whose backward ran outside the last micro-batch's fused path).
// `src` is this rank's fp32 gradient of a tensor sharded into equal contiguous slices of `slice` elements, slice o owned
// by rank o. Every element outside this rank's own slice is stored into its owner's staging region: stage.p[o] +
// dst_off addresses the slot reserved for THIS rank there. n % 4 == 0, slice % 4 == 0.
__global__ void __launch_bounds__(256)
p2p_push_slices_kernel(const float* __restrict__ src, size_t n4, size_t slice4, PeerPtrs stage, size_t dst_off, int rank) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const int owner = (int)(i / slice4);
    if (owner == rank) continue;
    const float4 val = reinterpret_cast<const float4*>(src)[i];
    reinterpret_cast<float4*>(reinterpret_cast<float*>(stage.p[owner]) + dst_off)[i - (size_t)owner * slice4] = val;
  }
}

// Plain vector copy of n fp32 values to an address that may be peer memory (one matrix to its owner's slot).
__global__ void __launch_bounds__(256)
p2p_copy_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, size_t n4) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
    reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
}

// Replicated small parameter: average all ranks' gradients, AdamW on the local copy.
__global__ void p2p_small_adamw_kernel(PeerPtrs grads, size_t grad_off, int world, float* __restrict__ p,
                                       float* __restrict__ m, float* __restrict__ v, int n, AdamWArgs a) {
  const float step_size = a.lr / a.bias1, inv_bias2 = 1.f / a.bias2, decay = 1.f - a.lr * a.wd;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    float g = 0.f;
    for (int r = 0; r < world; ++r) g += __ldcg(reinterpret_cast<const float*>(grads.p[r]) + grad_off + i);
    g = g / world * a.grad_scale;
    float pv = p[i] * decay, mv = m[i], vv = v[i];
    mv += (1.f - a.beta1) * (g - mv);
    vv += (1.f - a.beta2) * (g * g - vv);
    pv -= step_size * (mv / (sqrtf(vv * inv_bias2) + a.eps));
    p[i] = pv; m[i] = mv; v[i] = vv;
  }
}

static inline int grid_for(size_t work, int threads) {
  size_t need = (work + threads - 1) / threads;
  return (int)(need < 148 * 8 ? (need ? need : 1) : 148 * 8);
}

// `max_ctas` > 0 caps the grid: a link-bound kernel that shares the GPU with tensor-core work on another stream needs
// bytes in flight, not SMs.
static inline int cap_grid(int grid, int max_ctas) { return (max_ctas > 0 && grid > max_ctas) ? max_ctas : grid; }

cudaError_t p2p_barrier(const PeerPtrs& pads, int rank, int world, int epoch, int* status, cudaStream_t s) {
  if (world > MAX_RANKS) return cudaErrorInvalidValue;
  p2p_barrier_kernel<<<1, 32, 0, s>>>(pads, rank, world, epoch, status);
  return cudaGetLastError();
}

template <bool P_BF16>
static void launch_p2p_adamw(int grid, cudaStream_t s, const PeerPtrs& grads, size_t grad_off, int world, void* p, void* m,
                             void* v, const PeerPtrs& out, size_t out_off, int write_local_out, int rank, size_t n,
                             AdamWArgs a) {
#define NC_ADAMW_CASE(W) \
  p2p_adamw_kernel<P_BF16, W><<<grid, 128, 0, s>>>(grads, grad_off, world, p, m, v, out, out_off, write_local_out, rank, n, a)
  switch (world) {
    case 2: NC_ADAMW_CASE(2); break;
    case 4: NC_ADAMW_CASE(4); break;
    case 8: NC_ADAMW_CASE(8); break;
    default: NC_ADAMW_CASE(0); break;
  }
#undef NC_ADAMW_CASE
}

cudaError_t p2p_adamw(const PeerPtrs& grads, size_t grad_off, int world, int rank, void* p, int p_bf16, void* m, void* v,
                      const PeerPtrs& out, size_t out_off, int write_local_out, size_t n, AdamWArgs a, int max_ctas,
                      cudaStream_t s) {
  if ((n & 7) || (grad_off & 3) || (out_off & 7)) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  const size_t need = (n / 8 + 127) / 128;
  const int grid = cap_grid((int)(need < 148 * 16 ? need : 148 * 16), max_ctas);
  if (p_bf16) launch_p2p_adamw<true>(grid, s, grads, grad_off, world, p, m, v, out, out_off, write_local_out, rank, n, a);
  else launch_p2p_adamw<false>(grid, s, grads, grad_off, world, p, m, v, out, out_off, write_local_out, rank, n, a);
  return cudaGetLastError();
}

cudaError_t p2p_muon_momentum(const PeerPtrs& grads, size_t grad_off, int world, float* buf, void* X, float* rowss,
                              float mu, int k, int r, int c, int max_ctas, cudaStream_t s) {
  if ((c & 3) || (grad_off & 3)) return cudaErrorInvalidValue;
  const long long rows = (long long)k * r;
  if (rows == 0) return cudaSuccess;
  const int grid = cap_grid((int)((rows + 3) / 4 < 148 * 16 ? (rows + 3) / 4 : 148 * 16), max_ctas);
#define NC_MOM_CASE(W) \
  p2p_muon_momentum_kernel<W><<<grid, 128, 0, s>>>(grads, grad_off, world, buf, (__nv_bfloat16*)X, rowss, mu, rows, c)
  switch (world) {
    case 2: NC_MOM_CASE(2); break;
    case 4: NC_MOM_CASE(4); break;
    case 8: NC_MOM_CASE(8); break;
    default: NC_MOM_CASE(0); break;
  }
#undef NC_MOM_CASE
  return cudaGetLastError();
}

cudaError_t p2p_muon_apply(float* p, const void* X, const float* scale, const PeerPtrs& out, size_t out_off, int world,
                           int k, int r, int c, float lr, float wd, cudaStream_t s) {
  if ((c & 7) || (out_off & 7) || world > MAX_RANKS) return cudaErrorInvalidValue;
  const size_t n8 = (size_t)k * r * c / 8;
  if (n8 == 0) return cudaSuccess;
  p2p_muon_apply_kernel<<<grid_for(n8, 256), 256, 0, s>>>(p, (const __nv_bfloat16*)X, scale, out, out_off, world, r, c,
                                                          r >= c, lr, wd, n8);
  return cudaGetLastError();
}

cudaError_t p2p_bcast_bf16(const void* src, const PeerPtrs& dst, size_t dst_off, int world, int rank, size_t n,
                           cudaStream_t s) {
  if ((n & 7) || (dst_off & 7)) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  p2p_bcast_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const __nv_bfloat16*)src, dst, dst_off, world, rank, n / 8);
  return cudaGetLastError();
}

cudaError_t p2p_push_slices(const float* src, size_t n, size_t slice, const PeerPtrs& stage, size_t dst_off, int rank,
                            int max_ctas, cudaStream_t s) {
  if ((n & 3) || (slice & 3) || (dst_off & 3) || slice == 0) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  p2p_push_slices_kernel<<<cap_grid(grid_for(n / 4, 256), max_ctas), 256, 0, s>>>(src, n / 4, slice / 4, stage, dst_off, rank);
  return cudaGetLastError();
}

cudaError_t p2p_copy_f32(const float* src, float* dst, size_t n, cudaStream_t s) {
  if ((n & 3) || (reinterpret_cast<size_t>(dst) & 15) || (reinterpret_cast<size_t>(src) & 15)) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  p2p_copy_f32_kernel<<<grid_for(n / 4, 256), 256, 0, s>>>(src, dst, n / 4);
  return cudaGetLastError();
}

cudaError_t p2p_small_adamw(const PeerPtrs& grads, size_t grad_off, int world, float* p, float* m, float* v, int n,
                            AdamWArgs a, cudaStream_t s) {
  p2p_small_adamw_kernel<<<1, 256, 0, s>>>(grads, grad_off, world, p, m, v, n, a);
  return cudaGetLastError();
}

}  // namespace nc
