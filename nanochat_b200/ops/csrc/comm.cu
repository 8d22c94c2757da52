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
//   p2p_bcast_shadow   the updated bf16 matrices of this rank's Muon chunk written to every peer
//   p2p_small_adamw    replicated parameters (< 1024 elements): every rank averages all ranks'
//                      gradients itself and applies AdamW to its own copy (no write-back needed)
//
// Sums are taken in rank order 0..N-1, so the result does not depend on timing. Plain peer loads
// and stores only: no multimem, no TMA on peer memory.
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
template <bool P_BF16>
__global__ void p2p_adamw_kernel(PeerPtrs grads, size_t grad_off, int world, void* __restrict__ p,
                                 void* __restrict__ m, void* __restrict__ v, PeerPtrs out, size_t out_off,
                                 int write_local_out, int rank, size_t n, AdamWArgs a) {
  const float step_size = a.lr / a.bias1, inv_bias2 = 1.f / a.bias2, decay = 1.f - a.lr * a.wd;
  const float inv_world = 1.f / world;
  for (size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) * 8; i < n; i += (size_t)gridDim.x * blockDim.x * 8) {
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      const float* src = reinterpret_cast<const float*>(grads.p[r]) + grad_off + i;
      const float4 x = ldcg4(src), y = ldcg4(src + 4);
      g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w; g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
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
__global__ void __launch_bounds__(128)
p2p_muon_momentum_kernel(PeerPtrs grads, size_t grad_off, int world, float* __restrict__ buf,
                         __nv_bfloat16* __restrict__ X, float* __restrict__ rowss, float mu, long long rows, int c) {
  const int lane = threadIdx.x & 31;
  const float inv_world = 1.f / world;
  for (long long row = blockIdx.x * 4ll + (threadIdx.x >> 5); row < rows; row += gridDim.x * 4ll) {
    float* br = buf + row * c;
    __nv_bfloat16* xr = X + row * c;
    float ss = 0.f;
    for (int j = lane * 4; j < c; j += 128) {
      float4 g = make_float4(0, 0, 0, 0);
      for (int r = 0; r < world; ++r) {
        const float4 x = ldcg4(reinterpret_cast<const float*>(grads.p[r]) + grad_off + row * c + j);
        g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
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

cudaError_t p2p_barrier(const PeerPtrs& pads, int rank, int world, int epoch, int* status, cudaStream_t s) {
  if (world > MAX_RANKS) return cudaErrorInvalidValue;
  p2p_barrier_kernel<<<1, 32, 0, s>>>(pads, rank, world, epoch, status);
  return cudaGetLastError();
}

cudaError_t p2p_adamw(const PeerPtrs& grads, size_t grad_off, int world, int rank, void* p, int p_bf16, void* m, void* v,
                      const PeerPtrs& out, size_t out_off, int write_local_out, size_t n, AdamWArgs a, cudaStream_t s) {
  if ((n & 7) || (grad_off & 3) || (out_off & 7)) return cudaErrorInvalidValue;
  const int grid = grid_for(n / 8, 256);
  if (p_bf16) p2p_adamw_kernel<true><<<grid, 256, 0, s>>>(grads, grad_off, world, p, m, v, out, out_off, write_local_out, rank, n, a);
  else p2p_adamw_kernel<false><<<grid, 256, 0, s>>>(grads, grad_off, world, p, m, v, out, out_off, write_local_out, rank, n, a);
  return cudaGetLastError();
}

cudaError_t p2p_muon_momentum(const PeerPtrs& grads, size_t grad_off, int world, float* buf, void* X, float* rowss,
                              float mu, int k, int r, int c, cudaStream_t s) {
  if ((c & 3) || (grad_off & 3)) return cudaErrorInvalidValue;
  const long long rows = (long long)k * r;
  const int grid = (int)((rows + 3) / 4 < 148 * 16 ? (rows + 3) / 4 : 148 * 16);
  p2p_muon_momentum_kernel<<<grid, 128, 0, s>>>(grads, grad_off, world, buf, (__nv_bfloat16*)X, rowss, mu, rows, c);
  return cudaGetLastError();
}

cudaError_t p2p_bcast_bf16(const void* src, const PeerPtrs& dst, size_t dst_off, int world, int rank, size_t n,
                           cudaStream_t s) {
  if ((n & 7) || (dst_off & 7)) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  p2p_bcast_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const __nv_bfloat16*)src, dst, dst_off, world, rank, n / 8);
  return cudaGetLastError();
}

cudaError_t p2p_small_adamw(const PeerPtrs& grads, size_t grad_off, int world, float* p, float* m, float* v, int n,
                            AdamWArgs a, cudaStream_t s) {
  p2p_small_adamw_kernel<<<1, 256, 0, s>>>(grads, grad_off, world, p, m, v, n, a);
  return cudaGetLastError();
}

}  // namespace nc
