// Single-token decode kernels (a few rows per step, positions read from device memory so that a
// captured CUDA graph can be replayed without host-side arguments changing).
//
//   gemv_rows        out[b, n] = epi( sum_k x[b, k] W[n, k] , aux[b, n] ),  b < 8. A CTA owns four output
//                    columns and its 256 threads split K, streaming the weight rows once with 16-byte
//                    loads; the handful of activation rows stay in L1. Decode is bound by reading every
//                    weight once per token, so the kernel is a bandwidth kernel: no tensor cores, many
//                    loads in flight on every SM whatever the shape.
//   decode_embed     token embedding, RMS norm and the smear with the previous token's embedding: one CTA per row.
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

constexpr int GEMV_ROWS = 4;       // output columns per CTA: all 256 threads split K for each of them

__host__ __device__ constexpr int pow2_ceil(int n) { int p = 1; while (p < n) p <<= 1; return p; }
__host__ __device__ constexpr int ilog2(int n) { int l = 0; while ((1 << l) < n) ++l; return l; }

// Warp-wide sums of NV values per lane (NV a power of two <= 32). Step s pairs lanes 16 >> s apart: the lower lane keeps
// the first half of its list and the upper lane the second half, each adding the partner's copy of the half it keeps,
// so after log2(NV) steps lane l holds one value, index l >> (5 - log2 NV), summed over the lanes that share l's low
// bits; plain butterfly steps over those low bits finish it. NV - 1 + (5 - log2 NV) shuffles instead of 5 NV.
template <int NV>
__device__ __forceinline__ float warp_sum_many(float (&v)[NV], int lane) {
  constexpr int LOG = ilog2(NV);
  static_assert((1 << LOG) == NV && NV <= 32, "NV must be a power of two <= 32");
#pragma unroll
  for (int s = 0; s < LOG; ++s) {
    const int off = 16 >> s, half = NV >> (s + 1);
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  float r = v[0];
#pragma unroll
  for (int off = 16 >> LOG; off >= 1; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
  return r;
}

// MIX: the input row is the layer's mixed residual stream, built on the fly: xm = bf16(lam_r[layer] * x + lam_0[layer] * x0),
// fed to the dot products as rmsnorm(xm) (norm_input semantics). The first CTA also writes xm (the residual the
// attention projection adds back) and the first `head_cols` channels of rmsnorm(xm) (the value-embedding gate's input),
// so no separate mix+norm kernel runs in the decode step.
// The weight matrix the NEXT kernel of the decode step will stream: every CTA of this kernel asks the L2 for its
// slice of it (cp.async.bulk.prefetch.L2) before doing its own work, so HBM stays busy across kernel boundaries and
// the next kernel's loads hit L2. A one-shot GEMV of a 22 MB weight is otherwise latency-bound (12 us against 3.4 us
// at the copy rate). ptr = nullptr switches it off.
struct GemvNext {
  const char* ptr;
  long long bytes;
};

__device__ __forceinline__ void prefetch_next_weights(const GemvNext& next) {
  if (next.ptr == nullptr || threadIdx.x != 0) return;
  long long chunk = (next.bytes + gridDim.x - 1) / gridDim.x;
  chunk = (chunk + 15) & ~15ll;
  const long long begin = (long long)blockIdx.x * chunk;
  if (begin >= next.bytes) return;
  long long n = next.bytes - begin < chunk ? next.bytes - begin : chunk;
  n &= ~15ll;
  if (n <= 0) return;
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(next.ptr + begin), "r"((uint32_t)n) : "memory");
}

struct GemvMix {
  const __nv_bfloat16* x0; long long ldx0;
  const float* lam_r; const float* lam_0; int layer;
  __nv_bfloat16* xm; long long ldxm;
  __nv_bfloat16* xn_head; long long ldxn; int head_cols;
};

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }

template <int B, bool MIX>
__global__ void __launch_bounds__(256)
gemv_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ W, long long ldw,
                 __nv_bfloat16* __restrict__ out, long long ldo, const __nv_bfloat16* __restrict__ aux, long long ldaux,
                 int N, int K, int epi, int norm_input, GemvMix mix, GemvNext next) {
  __shared__ float s_acc[8][GEMV_ROWS][B];
  __shared__ float s_ss[8][B];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * GEMV_ROWS;
  float acc[GEMV_ROWS][B], ss[B];
#pragma unroll
  for (int b = 0; b < B; ++b) {
    ss[b] = 0.f;
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) acc[r][b] = 0.f;
  }
  prefetch_next_weights(next);
  // the weights do not depend on the previous kernel: the first loads are in flight while it finishes
  uint4 pre[GEMV_ROWS];
  const int k_first = tid * 8;
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r) {
    const int n = min(n0 + r, N - 1);
    pre[r] = k_first < K ? ld_stream(W + (long long)n * ldw + k_first) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  pdl_trigger();
  float lam_r = 1.f, lam_0 = 0.f;
  if (MIX) { lam_r = mix.lam_r[mix.layer]; lam_0 = mix.lam_0[mix.layer]; }
  auto fma_chunk = [&](const uint4 (&wv)[GEMV_ROWS], int k) {
    float wf[GEMV_ROWS][8];
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
      const float2 w0 = unpack_bf16(wv[r].x), w1 = unpack_bf16(wv[r].y), w2 = unpack_bf16(wv[r].z), w3 = unpack_bf16(wv[r].w);
      wf[r][0] = w0.x; wf[r][1] = w0.y; wf[r][2] = w1.x; wf[r][3] = w1.y;
      wf[r][4] = w2.x; wf[r][5] = w2.y; wf[r][6] = w3.x; wf[r][7] = w3.y;
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const uint4 xv = *reinterpret_cast<const uint4*>(x + b * ldx + k);
      const float2 xa = unpack_bf16(xv.x), xb = unpack_bf16(xv.y), xc = unpack_bf16(xv.z), xd = unpack_bf16(xv.w);
      float xf[8] = {xa.x, xa.y, xb.x, xb.y, xc.x, xc.y, xd.x, xd.y};
      if (MIX) {
        const uint4 zv = *reinterpret_cast<const uint4*>(mix.x0 + b * mix.ldx0 + k);
        const float2 za = unpack_bf16(zv.x), zb = unpack_bf16(zv.y), zc = unpack_bf16(zv.z), zd = unpack_bf16(zv.w);
        const float zf[8] = {za.x, za.y, zb.x, zb.y, zc.x, zc.y, zd.x, zd.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) xf[j] = round_bf16(lam_r * xf[j] + lam_0 * zf[j]);
        if (blockIdx.x == 0) {
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(xf[2 * j], xf[2 * j + 1]);
            pk[j] = *reinterpret_cast<const uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(mix.xm + b * mix.ldxm + k) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
      // rmsnorm(x) . w = rstd * (x . w): the row's sum of squares rides along
      if (MIX || norm_input) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ss[b] += xf[j] * xf[j];
      }
#pragma unroll
      for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[r][b] += wf[r][j] * xf[j];
    }
  };
  if (k_first < K) fma_chunk(pre, k_first);
#pragma unroll 2
  for (int k = k_first + 2048; k < K; k += 2048) {
    uint4 wv[GEMV_ROWS];
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) wv[r] = ld_stream(W + (long long)min(n0 + r, N - 1) * ldw + k);
    fma_chunk(wv, k);
  }
  // 4 x B partial dot products per lane: a transposing reduction (the value list halves as the lane distance halves)
  // sums them with ~4B shuffles instead of 5 per value
  {
    constexpr int NV = pow2_ceil(GEMV_ROWS * B), LOW = 5 - ilog2(NV);
    float flat[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) flat[i] = i < GEMV_ROWS * B ? acc[i / B][i % B] : 0.f;
    const float total = warp_sum_many<NV>(flat, lane);
    const int idx = lane >> LOW;                                 // the value this lane ends up owning
    if ((lane & ((1 << LOW) - 1)) == 0 && idx < GEMV_ROWS * B) s_acc[warp][idx / B][idx % B] = total;
  }
  if (MIX || norm_input) {
    constexpr int NB = pow2_ceil(B), LOW = 5 - ilog2(NB);
    float flat[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) flat[i] = i < B ? ss[i] : 0.f;
    const float total = warp_sum_many<NB>(flat, lane);
    const int idx = lane >> LOW;
    if ((lane & ((1 << LOW) - 1)) == 0 && idx < B) s_ss[warp][idx] = total;
  }
  __syncthreads();
  if (MIX && blockIdx.x == 0 && tid < mix.head_cols * B) {
    const int b = tid / mix.head_cols, c = tid - b * mix.head_cols;
    float q = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) q += s_ss[w][b];
    const float xm = round_bf16(lam_r * __bfloat162float(x[b * ldx + c]) + lam_0 * __bfloat162float(mix.x0[b * mix.ldx0 + c]));
    mix.xn_head[b * mix.ldxn + c] = __float2bfloat16(xm * rsqrtf(q / K + kRmsEps));
  }
  if (tid < GEMV_ROWS * B) {
    const int r = tid / B, b = tid - r * B;
    const int n = n0 + r;
    if (n < N) {
      float v = 0.f, q = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) { v += s_acc[w][r][b]; if (MIX || norm_input) q += s_ss[w][b]; }
      if (MIX || norm_input) v *= rsqrtf(q / K + kRmsEps);
      if (epi == DEC_EPI_RELU2) { v = fmaxf(v, 0.f); v *= v; }
      if (aux) v += __bfloat162float(aux[b * ldaux + n]);
      out[b * ldo + n] = __float2bfloat16(v);
    }
  }
}

// One CTA per row: token embedding -> RMS norm -> smear with the previous token's normed embedding
//   e = norm(wte[id]);  out = e + lam * sigmoid(e[:n_gate] . gate_w) * prev;  prev <- e
// (reference: nanochat/gpt.py:471-492, the single-token branch). `prev` holds zeros at the start of a generation
// whose prefill left no state, which makes the smear term vanish.
__global__ void __launch_bounds__(256)
decode_embed_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ wte, long long ldw, int vocab,
                    const float* __restrict__ gate_w, int n_gate, const float* __restrict__ lam,
                    __nv_bfloat16* __restrict__ prev, long long ldp, __nv_bfloat16* __restrict__ out, long long ldo,
                    int C) {
  __shared__ float s_red[8];
  __shared__ float s_head[32];
  __shared__ float s_bcast[2];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long id = ids[b];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);          // an out-of-range id must not become a wild read
  const __nv_bfloat16* row = wte + id * ldw;
  float ss = 0.f;
  for (int c = tid * 8; c < C; c += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + c);
    const float2 a0 = unpack_bf16(v.x), a1 = unpack_bf16(v.y), a2 = unpack_bf16(v.z), a3 = unpack_bf16(v.w);
    ss += a0.x * a0.x + a0.y * a0.y + a1.x * a1.x + a1.y * a1.y + a2.x * a2.x + a2.y * a2.y + a3.x * a3.x + a3.y * a3.y;
  }
  ss = warp_sum(ss);
  if (lane == 0) s_red[warp] = ss;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += s_red[w];
    s_bcast[0] = rsqrtf(t / C + kRmsEps);
  }
  __syncthreads();
  const float rstd = s_bcast[0];
  if (tid < n_gate) s_head[tid] = __bfloat162float(__float2bfloat16(__bfloat162float(row[tid]) * rstd)) * gate_w[tid];
  __syncthreads();
  if (tid == 0) {
    float dot = 0.f;
    for (int i = 0; i < n_gate; ++i) dot += s_head[i];
    s_bcast[1] = lam[0] / (1.f + __expf(-dot));
  }
  __syncthreads();
  const float gate = s_bcast[1];
  for (int c = tid * 8; c < C; c += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + c);
    const uint4 pv = *reinterpret_cast<const uint4*>(prev + b * ldp + c);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w}, pin[4] = {pv.x, pv.y, pv.z, pv.w};
    uint32_t e_out[4], x_out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16(in[j]), p = unpack_bf16(pin[j]);
      const __nv_bfloat162 e = __floats2bfloat162_rn(a.x * rstd, a.y * rstd);          // the normed embedding, as stored
      const float2 ef = __bfloat1622float2(e);
      const __nv_bfloat162 x = __floats2bfloat162_rn(ef.x + gate * p.x, ef.y + gate * p.y);
      e_out[j] = *reinterpret_cast<const uint32_t*>(&e);
      x_out[j] = *reinterpret_cast<const uint32_t*>(&x);
    }
    *reinterpret_cast<uint4*>(prev + b * ldp + c) = make_uint4(e_out[0], e_out[1], e_out[2], e_out[3]);
    *reinterpret_cast<uint4*>(out + b * ldo + c) = make_uint4(x_out[0], x_out[1], x_out[2], x_out[3]);
  }
}

// Where token t of row b lives in one layer's K (or V) store. Contiguous cache: b * c_bat + t * c_tok. Paged cache
// (pages.table != nullptr): the store is a pool of pages of 2^page_shift tokens, c_bat is the pitch of a page and
// table[b * max_pages + (t >> page_shift)] names the page; rows may share pages (a common prompt prefix is held once).
__device__ __forceinline__ long long kv_token_offset(const KvPages& pages, int b, int t, long long c_bat, long long c_tok) {
  if (pages.table == nullptr) return b * c_bat + (long long)t * c_tok;
  const int page = pages.table[(long long)b * pages.max_pages + (t >> pages.page_shift)];
  return page * c_bat + (long long)(t & ((1 << pages.page_shift) - 1)) * c_tok;
}

// One warp per (row, head slot): slots [0,H) = q heads, [H,H+Hkv) = k heads, [H+Hkv,H+2Hkv) = v heads. D = 128.
__global__ void __launch_bounds__(128)
decode_qkv_post_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, int H, int Hkv, const __nv_bfloat16* __restrict__ cos_t,
                       const __nv_bfloat16* __restrict__ sin_t, const int* __restrict__ seqlens,
                       const __nv_bfloat16* __restrict__ xn, long long ld_xn, const float* __restrict__ wg,
                       const __nv_bfloat16* __restrict__ ve, long long ld_ve, const long long* __restrict__ idx,
                       __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, long long c_bat,
                       long long c_tok, int t_max, int B, int* __restrict__ status, KvPages pages) {
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
    dst = (is_v ? v_cache : k_cache) + kv_token_offset(pages, b, pos, c_bat, c_tok) + hkv * 128;
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
                   long long ldy, KvPages pages) {
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hkv = h / (H / Hkv);
  // The row's page table does not change while a sequence is decoded (and the kernel before this one in the stream
  // does not write it), so it is copied to shared memory before the wait on that kernel: the lookups of the key loop
  // then cost a shared-memory read instead of a dependent global load in front of every key.
  __shared__ int s_table[128];
  if (pages.table != nullptr && pages.max_pages <= 128) {
    if ((int)threadIdx.x < pages.max_pages) s_table[threadIdx.x] = pages.table[(long long)b * pages.max_pages + threadIdx.x];
    pages.table = nullptr;
    pages.max_pages = -1;                             // marks "table in shared memory" for the address helper below
  }
  auto token_offset = [&](int t) -> long long {
    if (pages.max_pages == -1) {
      return s_table[t >> pages.page_shift] * c_bat + (long long)(t & ((1 << pages.page_shift) - 1)) * c_tok;
    }
    return kv_token_offset(pages, b, t, c_bat, c_tok);
  };
  pdl_wait();
  pdl_trigger();
  const int pos = seqlens[b];                         // the new token sits at `pos`; it sees keys lo..pos
  const int lo = window < 0 ? 0 : max(0, pos - window);
  const int n_keys = pos - lo + 1;
  const int chunk = (n_keys + kSplits - 1) / kSplits;
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);
  // Two phases per tile of up to 128 keys: scores with one thread per key (no shuffles in the dot product),
  // then the weighted sum of V with one thread per output dim (coalesced rows of V).
  __shared__ float s_q[128];
  __shared__ float s_p[128];
  __shared__ float s_red[8];
  __shared__ float s_o[4][128];
  const int d = threadIdx.x;
  s_q[d] = __bfloat162float(q[b * ldq + h * 128 + d]);
  __syncthreads();
  const __nv_bfloat16* kb = k_cache + hkv * 128;
  const __nv_bfloat16* vb = v_cache + hkv * 128 + lane * 4;   // phase 2: a lane owns 4 dims
  float M = -1.0e30f, L = 0.f, O = 0.f;
  for (int tile = k_begin; tile < k_end; tile += 128) {
    const int j = tile + d;
    float sc = -1.0e30f;
    if (j < k_end) {
      const uint4* kr = reinterpret_cast<const uint4*>(kb + token_offset(j));
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint4 kv = kr[i];
        const float2 k0 = unpack_bf16(kv.x), k1 = unpack_bf16(kv.y), k2 = unpack_bf16(kv.z), k3 = unpack_bf16(kv.w);
        const float* qq = s_q + i * 8;
        acc += k0.x * qq[0] + k0.y * qq[1] + k1.x * qq[2] + k1.y * qq[3] + k2.x * qq[4] + k2.y * qq[5] + k3.x * qq[6] +
               k3.y * qq[7];
      }
      sc = acc * scale_log2;
    }
    float mx = sc;
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    const float m_new = fmaxf(M, fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3])));
    const float pj = j < k_end ? exp2f(sc - m_new) : 0.f;
    s_p[d] = pj;
    const float ps = warp_sum(pj);
    if (lane == 0) s_red[4 + warp] = ps;
    __syncthreads();
    const float alpha = exp2f(M - m_new);
    L = L * alpha + (s_red[4] + s_red[5]) + (s_red[6] + s_red[7]);
    // weighted sum of V: warp w takes keys w, w+4, ... (independent 8-byte loads, many in flight), then the four
    // partial vectors are added per dim
    const int cnt = min(128, k_end - tile);
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll 8
    for (int jj = warp; jj < cnt; jj += 4) {
      const uint2 vr = *reinterpret_cast<const uint2*>(vb + token_offset(tile + jj));
      const float2 v01 = unpack_bf16(vr.x), v23 = unpack_bf16(vr.y);
      const float pw = s_p[jj];
      o0 += pw * v01.x; o1 += pw * v01.y; o2 += pw * v23.x; o3 += pw * v23.y;
    }
    *reinterpret_cast<float4*>(&s_o[warp][lane * 4]) = make_float4(o0, o1, o2, o3);
    __syncthreads();
    O = O * alpha + (s_o[0][d] + s_o[1][d]) + (s_o[2][d] + s_o[3][d]);
    M = m_new;
    __syncthreads();                                   // s_p, s_o and s_red are rewritten by the next tile
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
                      const void* aux, long long ldaux, int B, int N, int K, int epi, int norm_input,
                      const void* next_w, long long next_bytes, cudaStream_t s) {
  if (B < 1 || B > 8 || (K & 7) || (ldx & 7) || (ldw & 7)) return cudaErrorInvalidValue;
  const int grid = (N + GEMV_ROWS - 1) / GEMV_ROWS;
  auto xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto wp = reinterpret_cast<const __nv_bfloat16*>(W);
  auto op = reinterpret_cast<__nv_bfloat16*>(out);
  auto ap = reinterpret_cast<const __nv_bfloat16*>(aux);
  cudaError_t e = cudaSuccess;
  const GemvMix none = {};
  const GemvNext next = {reinterpret_cast<const char*>(next_w), (reinterpret_cast<uintptr_t>(next_w) & 15) ? 0 : next_bytes};
#define NC_GEMV(BB) case BB: e = launch_pdl(gemv_rows_kernel<BB, false>, dim3(grid), dim3(256), s, xp, ldx, wp, ldw, op, ldo, ap, ldaux, N, K, epi, norm_input, none, next); break;
  switch (B) {
    NC_GEMV(1) NC_GEMV(2) NC_GEMV(3) NC_GEMV(4) NC_GEMV(5) NC_GEMV(6) NC_GEMV(7) NC_GEMV(8)
  }
#undef NC_GEMV
  return e;
}

cudaError_t gemv_rows_mix(const void* x, long long ldx, const void* x0, long long ldx0, const float* lam_r,
                          const float* lam_0, int layer, const void* W, long long ldw, void* out, long long ldo,
                          void* xm, long long ldxm, void* xn_head, long long ldxn, int head_cols, int B, int N, int K,
                          const void* next_w, long long next_bytes, cudaStream_t s) {
  if (B < 1 || B > 8 || (K & 7) || (ldx & 7) || (ldx0 & 7) || (ldw & 7) || (ldxm & 7) || head_cols < 0 ||
      head_cols * B > 256 || head_cols > K)
    return cudaErrorInvalidValue;
  const int grid = (N + GEMV_ROWS - 1) / GEMV_ROWS;
  auto xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto wp = reinterpret_cast<const __nv_bfloat16*>(W);
  auto op = reinterpret_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* no_aux = nullptr;
  GemvMix mix = {reinterpret_cast<const __nv_bfloat16*>(x0), ldx0, lam_r, lam_0, layer,
                 reinterpret_cast<__nv_bfloat16*>(xm), ldxm, reinterpret_cast<__nv_bfloat16*>(xn_head), ldxn, head_cols};
  cudaError_t e = cudaSuccess;
  const GemvNext next = {reinterpret_cast<const char*>(next_w), (reinterpret_cast<uintptr_t>(next_w) & 15) ? 0 : next_bytes};
#define NC_GEMV(BB) case BB: e = launch_pdl(gemv_rows_kernel<BB, true>, dim3(grid), dim3(256), s, xp, ldx, wp, ldw, op, ldo, no_aux, 0LL, N, K, (int)DEC_EPI_NONE, 1, mix, next); break;
  switch (B) {
    NC_GEMV(1) NC_GEMV(2) NC_GEMV(3) NC_GEMV(4) NC_GEMV(5) NC_GEMV(6) NC_GEMV(7) NC_GEMV(8)
  }
#undef NC_GEMV
  return e;
}

cudaError_t decode_embed(const long long* ids, const void* wte, long long ldw, int vocab, const float* gate_w, int n_gate,
                         const float* lam, void* prev, long long ldp, void* out, long long ldo, int B, int C,
                         cudaStream_t s) {
  if (B <= 0 || C % 8 != 0 || ldw % 8 != 0 || ldp % 8 != 0 || ldo % 8 != 0 || n_gate < 0 || n_gate > 32 || n_gate > C)
    return cudaErrorInvalidValue;
  decode_embed_kernel<<<B, 256, 0, s>>>(ids, reinterpret_cast<const __nv_bfloat16*>(wte), ldw, vocab, gate_w, n_gate, lam,
                                        reinterpret_cast<__nv_bfloat16*>(prev), ldp,
                                        reinterpret_cast<__nv_bfloat16*>(out), ldo, C);
  return cudaGetLastError();
}

cudaError_t decode_qkv_post(void* qkv, long long ld, int H, int Hkv, const void* cos_t, const void* sin_t,
                            const int* seqlens, const void* xn, long long ld_xn, const float* wg, const void* ve,
                            long long ld_ve, const long long* idx, void* k_cache, void* v_cache, long long c_bat,
                            long long c_tok, int t_max, int B, int* status, const KvPages& pages, cudaStream_t s) {
  if (pages.table != nullptr && (pages.page_shift < 0 || pages.page_shift > 16 || pages.max_pages <= 0 ||
                                 t_max > (pages.max_pages << pages.page_shift)))
    return cudaErrorInvalidValue;
  const int warps = B * (H + 2 * Hkv);
  return launch_pdl(decode_qkv_post_kernel, dim3((warps + 3) / 4), dim3(128), s,
      reinterpret_cast<__nv_bfloat16*>(qkv), ld, H, Hkv, reinterpret_cast<const __nv_bfloat16*>(cos_t),
      reinterpret_cast<const __nv_bfloat16*>(sin_t), seqlens, reinterpret_cast<const __nv_bfloat16*>(xn), ld_xn, wg,
      reinterpret_cast<const __nv_bfloat16*>(ve), ld_ve, idx, reinterpret_cast<__nv_bfloat16*>(k_cache),
      reinterpret_cast<__nv_bfloat16*>(v_cache), c_bat, c_tok, t_max, B, status, pages);
}

// partial results plus one arrival counter per (row, head); the counters must start at zero (they return to zero)
size_t decode_attn_scratch_floats(int B, int H) { return (size_t)B * H * kSplits * 130 + (size_t)B * H; }

cudaError_t decode_attn(const void* q, long long ldq, const void* k_cache, const void* v_cache, long long c_bat,
                        long long c_tok, const int* seqlens, int B, int H, int Hkv, int window, float scale,
                        float* scratch, void* y, long long ldy, const KvPages& pages, cudaStream_t s) {
  if (H % Hkv != 0) return cudaErrorInvalidValue;
  unsigned int* arrivals = reinterpret_cast<unsigned int*>(scratch + (size_t)B * H * kSplits * 130);
  return launch_pdl(decode_attn_kernel, dim3(kSplits, H, B), dim3(128), s,
      reinterpret_cast<const __nv_bfloat16*>(q), ldq, reinterpret_cast<const __nv_bfloat16*>(k_cache),
      reinterpret_cast<const __nv_bfloat16*>(v_cache), c_bat, c_tok, seqlens, H, Hkv, window,
      scale * 1.4426950408889634f, scratch, arrivals, reinterpret_cast<__nv_bfloat16*>(y), ldy, pages);
}

}  // namespace nc
