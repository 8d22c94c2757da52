// Single-token decode kernels (a few rows per step, positions read from device memory so that a
// captured CUDA graph can be replayed without host-side arguments changing).
//
//   gemv_rows        out[b, n] = epi( sum_k x[b, k] W[n, k] , aux[b, n] ),  b < 8. One warp per output
//                    column streams its weight row once with 16-byte loads; the handful of activation
//                    rows stay in L1. Decode is bound by reading every weight once per token, so the
//                    kernel is a bandwidth kernel: no tensor cores, many loads in flight.
//   decode_qkv_post  rotary at position seqlens[b], RMS norm and scale of q and k, value-embedding gate
//                    on v, and the append of k and v to the (B, T, Hkv, D) cache: one warp per head.
//   decode_attn      flash-decoding: grid (splits, heads, rows), each CTA reduces a slice of the visible
//                    keys with an online softmax; the CTA that finishes last merges the slices.
// The reference does these steps with generic library ops (reference: nanochat/gpt.py:84-107,
// nanochat/flash_attention.py:113-170 for the cached-attention call).
#include "decode.h"
#include "host_utils.cuh"
#include "ptx.cuh"

namespace nc {

namespace {

constexpr float kRmsEps = 1.1920929e-07f;   // fp32 machine epsilon, as F.rms_norm(eps=None)

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its predecessor in the
// stream is still running; pdl_wait() blocks until the predecessor has completed and its writes are visible,
// pdl_trigger() lets the successor be scheduled once every CTA of this grid has issued it. Launch latency of a
// chain of short kernels then overlaps with their execution. Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int w = 16; w > 0; w >>= 1) v += __shfl_xor_sync(0xffffffffu, v, w);
  return v;
}

template <int B>
__global__ void __launch_bounds__(256)
gemv_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ W, long long ldw,
                 __nv_bfloat16* __restrict__ out, long long ldo, const __nv_bfloat16* __restrict__ aux, long long ldaux,
                 int N, int K, int epi, int norm_input) {
  const int lane = threadIdx.x & 31;
  const int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (n >= N) return;                       // whole warps leave together
  const __nv_bfloat16* wrow = W + (long long)n * ldw;
  float acc[B], ss[B];
#pragma unroll
  for (int b = 0; b < B; ++b) { acc[b] = 0.f; ss[b] = 0.f; }
  // the weights do not depend on the previous kernel: the first loads are in flight while it finishes
  constexpr int PRE = 4;
  uint4 pre[PRE];
#pragma unroll
  for (int i = 0; i < PRE; ++i) {
    const int k = lane * 8 + i * 256;
    pre[i] = k < K ? ld_stream(wrow + k) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  pdl_trigger();
  auto fma_chunk = [&](const uint4& wv, int k) {
    const float2 w0 = unpack_bf16(wv.x), w1 = unpack_bf16(wv.y), w2 = unpack_bf16(wv.z), w3 = unpack_bf16(wv.w);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const uint4 xv = *reinterpret_cast<const uint4*>(x + b * ldx + k);
      const float2 x0 = unpack_bf16(xv.x), x1 = unpack_bf16(xv.y), x2 = unpack_bf16(xv.z), x3 = unpack_bf16(xv.w);
      acc[b] += w0.x * x0.x + w0.y * x0.y + w1.x * x1.x + w1.y * x1.y + w2.x * x2.x + w2.y * x2.y + w3.x * x3.x +
                w3.y * x3.y;
      // rmsnorm(x) . w = rstd * (x . w): the row's sum of squares rides along (every warp sees the whole row)
      if (norm_input)
        ss[b] += x0.x * x0.x + x0.y * x0.y + x1.x * x1.x + x1.y * x1.y + x2.x * x2.x + x2.y * x2.y + x3.x * x3.x +
                 x3.y * x3.y;
    }
  };
#pragma unroll
  for (int i = 0; i < PRE; ++i) {
    const int k = lane * 8 + i * 256;
    if (k < K) fma_chunk(pre[i], k);
  }
#pragma unroll 4
  for (int k = lane * 8 + PRE * 256; k < K; k += 256) fma_chunk(ld_stream(wrow + k), k);
#pragma unroll
  for (int b = 0; b < B; ++b) {
    acc[b] = warp_sum(acc[b]);
    if (norm_input) acc[b] *= rsqrtf(warp_sum(ss[b]) / K + kRmsEps);
  }
  if (lane < B) {
    float v = 0.f;
#pragma unroll
    for (int b = 0; b < B; ++b) v = lane == b ? acc[b] : v;
    if (epi == DEC_EPI_RELU2) { v = fmaxf(v, 0.f); v *= v; }
    if (aux) v += __bfloat162float(aux[lane * ldaux + n]);
    out[lane * ldo + n] = __float2bfloat16(v);
  }
}

// One warp per (row, head slot): slots [0,H) = q heads, [H,H+Hkv) = k heads, [H+Hkv,H+2Hkv) = v heads. D = 128.
__global__ void __launch_bounds__(128)
decode_qkv_post_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, int H, int Hkv, const __nv_bfloat16* __restrict__ cos_t,
                       const __nv_bfloat16* __restrict__ sin_t, const int* __restrict__ seqlens,
                       const __nv_bfloat16* __restrict__ xn, long long ld_xn, const float* __restrict__ wg,
                       const __nv_bfloat16* __restrict__ ve, long long ld_ve, const long long* __restrict__ idx,
                       __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, long long c_bat,
                       long long c_tok, int t_max, int B, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int slot_all = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int slots = H + 2 * Hkv;
  if (slot_all >= B * slots) return;
  pdl_wait();
  pdl_trigger();
  const int b = slot_all / slots, slot = slot_all - b * slots;
  const int pos = seqlens[b];
  if (pos < 0 || pos >= t_max) {            // a full cache: record it and leave the row untouched
    if (lane == 0 && status) atomicCAS(status, 0, (ST_BAD_ARG << 24) | 0xdec0de);
    return;
  }
  __nv_bfloat16* row = qkv + b * ld + slot * 128;
  // lane owns dims 2l, 2l+1 of the first half and the rotary partners 64+2l, 64+2l+1
  const uint32_t a_raw = *reinterpret_cast<const uint32_t*>(row + 2 * lane);
  const uint32_t b_raw = *reinterpret_cast<const uint32_t*>(row + 64 + 2 * lane);
  float2 x1 = unpack_bf16(a_raw), x2 = unpack_bf16(b_raw);
  if (slot < H + Hkv) {
    const float2 c = unpack_bf16(*reinterpret_cast<const uint32_t*>(cos_t + (long long)pos * 64 + 2 * lane));
    const float2 s = unpack_bf16(*reinterpret_cast<const uint32_t*>(sin_t + (long long)pos * 64 + 2 * lane));
    float2 y1, y2;
    y1.x = x1.x * c.x + x2.x * s.x; y1.y = x1.y * c.y + x2.y * s.y;
    y2.x = x2.x * c.x - x1.x * s.x; y2.y = x2.y * c.y - x1.y * s.y;
    const float ss = warp_sum(y1.x * y1.x + y1.y * y1.y + y2.x * y2.x + y2.y * y2.y);
    const float r = rsqrtf(ss * (1.f / 128.f) + kRmsEps) * 1.2f;
    x1.x = y1.x * r; x1.y = y1.y * r; x2.x = y2.x * r; x2.y = y2.y * r;
  } else if (ve) {
    const int hkv = slot - H - Hkv;
    float g = lane < 12 ? __bfloat162float(xn[b * ld_xn + lane]) * wg[hkv * 12 + lane] : 0.f;
    g = 3.f / (1.f + __expf(-warp_sum(g)));
    const __nv_bfloat16* vrow = ve + idx[b] * ld_ve + hkv * 128;
    const float2 e1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(vrow + 2 * lane));
    const float2 e2 = unpack_bf16(*reinterpret_cast<const uint32_t*>(vrow + 64 + 2 * lane));
    x1.x += g * e1.x; x1.y += g * e1.y; x2.x += g * e2.x; x2.y += g * e2.y;
  }
  const uint32_t o1 = pack_bf16(x1.x, x1.y), o2 = pack_bf16(x2.x, x2.y);
  __nv_bfloat16* dst = row;
  if (slot >= H) {
    const bool is_v = slot >= H + Hkv;
    const int hkv = slot - H - (is_v ? Hkv : 0);
    dst = (is_v ? v_cache : k_cache) + b * c_bat + (long long)pos * c_tok + hkv * 128;
  }
  *reinterpret_cast<uint32_t*>(dst + 2 * lane) = o1;
  *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = o2;
}

constexpr int kSplits = 8;

// grid (kSplits, H, B), 128 threads. partial: (B, H, kSplits, 130) fp32 = [m, l, o[128]].
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, long long c_bat, long long c_tok,
                   const int* __restrict__ seqlens, int H, int Hkv, int window, float scale_log2,
                   float* __restrict__ partial, unsigned int* __restrict__ arrivals, __nv_bfloat16* __restrict__ y,
                   long long ldy) {
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hkv = h / (H / Hkv);
  pdl_wait();
  pdl_trigger();
  const int pos = seqlens[b];                         // the new token sits at `pos`; it sees keys lo..pos
  const int lo = window < 0 ? 0 : max(0, pos - window);
  const int n_keys = pos - lo + 1;
  const int chunk = (n_keys + kSplits - 1) / kSplits;
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);
  const uint2 qraw = *reinterpret_cast<const uint2*>(q + b * ldq + h * 128 + lane * 4);
  const float2 q01 = unpack_bf16(qraw.x), q23 = unpack_bf16(qraw.y);
  const __nv_bfloat16* kb = k_cache + b * c_bat + hkv * 128 + lane * 4;
  const __nv_bfloat16* vb = v_cache + b * c_bat + hkv * 128 + lane * 4;
  float m = -1.0e30f, l = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
  for (int j = k_begin + warp; j < k_end; j += 4) {
    const uint2 kr = *reinterpret_cast<const uint2*>(kb + (long long)j * c_tok);
    const uint2 vr = *reinterpret_cast<const uint2*>(vb + (long long)j * c_tok);
    const float2 k01 = unpack_bf16(kr.x), k23 = unpack_bf16(kr.y);
    const float s = warp_sum(q01.x * k01.x + q01.y * k01.y + q23.x * k23.x + q23.y * k23.y) * scale_log2;
    const float m_new = fmaxf(m, s);
    const float alpha = exp2f(m - m_new), p = exp2f(s - m_new);
    const float2 v01 = unpack_bf16(vr.x), v23 = unpack_bf16(vr.y);
    l = l * alpha + p;
    o0 = o0 * alpha + p * v01.x; o1 = o1 * alpha + p * v01.y; o2 = o2 * alpha + p * v23.x; o3 = o3 * alpha + p * v23.y;
    m = m_new;
  }
  __shared__ float sm[4][130];
  if (lane == 0) { sm[warp][0] = m; sm[warp][1] = l; }
  sm[warp][2 + lane * 4] = o0; sm[warp][3 + lane * 4] = o1; sm[warp][4 + lane * 4] = o2; sm[warp][5 + lane * 4] = o3;
  __syncthreads();
  const int d = threadIdx.x;                          // 128 threads = 128 output dims
  const float M = fmaxf(fmaxf(sm[0][0], sm[1][0]), fmaxf(sm[2][0], sm[3][0]));
  float L = 0.f, O = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const float f = exp2f(sm[w][0] - M);
    L += f * sm[w][1];
    O += f * sm[w][2 + d];
  }
  float* dst = partial + (((long long)b * H + h) * kSplits + split) * 130;
  if (d == 0) { dst[0] = M; dst[1] = L; }
  dst[2 + d] = O;
  // the split that arrives last merges all of them (the counter wraps back to zero by itself)
  __shared__ unsigned int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicInc(arrivals + b * H + h, kSplits - 1) == kSplits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const volatile float* src = partial + ((long long)b * H + h) * kSplits * 130;
  float Mx = -1.0e30f;
#pragma unroll
  for (int s = 0; s < kSplits; ++s) Mx = fmaxf(Mx, src[s * 130]);
  float Ls = 0.f, Os = 0.f;
#pragma unroll
  for (int s = 0; s < kSplits; ++s) {
    const float f = exp2f(src[s * 130] - Mx);
    Ls += f * src[s * 130 + 1];
    Os += f * src[s * 130 + 2 + d];
  }
  y[b * ldy + h * 128 + d] = __float2bfloat16(Ls > 0.f ? Os / Ls : 0.f);
}

}  // namespace

cudaError_t gemv_rows(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                      const void* aux, long long ldaux, int B, int N, int K, int epi, int norm_input, cudaStream_t s) {
  if (B < 1 || B > 8 || (K & 7) || (ldx & 7) || (ldw & 7)) return cudaErrorInvalidValue;
  const int grid = (N + 7) / 8;
  auto xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto wp = reinterpret_cast<const __nv_bfloat16*>(W);
  auto op = reinterpret_cast<__nv_bfloat16*>(out);
  auto ap = reinterpret_cast<const __nv_bfloat16*>(aux);
  cudaError_t e = cudaSuccess;
#define NC_GEMV(BB) case BB: e = launch_pdl(gemv_rows_kernel<BB>, dim3(grid), dim3(256), s, xp, ldx, wp, ldw, op, ldo, ap, ldaux, N, K, epi, norm_input); break;
  switch (B) {
    NC_GEMV(1) NC_GEMV(2) NC_GEMV(3) NC_GEMV(4) NC_GEMV(5) NC_GEMV(6) NC_GEMV(7) NC_GEMV(8)
  }
#undef NC_GEMV
  return e;
}

cudaError_t decode_qkv_post(void* qkv, long long ld, int H, int Hkv, const void* cos_t, const void* sin_t,
                            const int* seqlens, const void* xn, long long ld_xn, const float* wg, const void* ve,
                            long long ld_ve, const long long* idx, void* k_cache, void* v_cache, long long c_bat,
                            long long c_tok, int t_max, int B, int* status, cudaStream_t s) {
  const int warps = B * (H + 2 * Hkv);
  return launch_pdl(decode_qkv_post_kernel, dim3((warps + 3) / 4), dim3(128), s,
      reinterpret_cast<__nv_bfloat16*>(qkv), ld, H, Hkv, reinterpret_cast<const __nv_bfloat16*>(cos_t),
      reinterpret_cast<const __nv_bfloat16*>(sin_t), seqlens, reinterpret_cast<const __nv_bfloat16*>(xn), ld_xn, wg,
      reinterpret_cast<const __nv_bfloat16*>(ve), ld_ve, idx, reinterpret_cast<__nv_bfloat16*>(k_cache),
      reinterpret_cast<__nv_bfloat16*>(v_cache), c_bat, c_tok, t_max, B, status);
}

// partial results plus one arrival counter per (row, head); the counters must start at zero (they return to zero)
size_t decode_attn_scratch_floats(int B, int H) { return (size_t)B * H * kSplits * 130 + (size_t)B * H; }

cudaError_t decode_attn(const void* q, long long ldq, const void* k_cache, const void* v_cache, long long c_bat,
                        long long c_tok, const int* seqlens, int B, int H, int Hkv, int window, float scale,
                        float* scratch, void* y, long long ldy, cudaStream_t s) {
  if (H % Hkv != 0) return cudaErrorInvalidValue;
  unsigned int* arrivals = reinterpret_cast<unsigned int*>(scratch + (size_t)B * H * kSplits * 130);
  return launch_pdl(decode_attn_kernel, dim3(kSplits, H, B), dim3(128), s,
      reinterpret_cast<const __nv_bfloat16*>(q), ldq, reinterpret_cast<const __nv_bfloat16*>(k_cache),
      reinterpret_cast<const __nv_bfloat16*>(v_cache), c_bat, c_tok, seqlens, H, Hkv, window,
      scale * 1.4426950408889634f, scratch, arrivals, reinterpret_cast<__nv_bfloat16*>(y), ldy);
}

}  // namespace nc
