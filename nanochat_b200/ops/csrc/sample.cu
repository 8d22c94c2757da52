// Next-token sampling in one kernel: argmax, or top-k -> temperature softmax -> inverse-CDF draw.
//
// The reference does this with library calls (topk, softmax, multinomial, gather:
// reference nanochat/engine.py:141-156). Here one CTA per row makes a few passes over the row's logits
// (128 KB for a 32768-token vocabulary, L2 resident):
//   1. block maximum (and, for temperature 0, its first index);
//   2. top-k threshold by a 4 x 8-bit radix select on an order-preserving integer image of the floats;
//   3. per-thread partial sums of exp((v - max) / T) over the selected entries of a contiguous chunk,
//      a block-wide exclusive scan, and the walk that finds where u * total falls.
// The uniform number u comes from the caller (drawn from its seeded generator), which keeps "same seed,
// same tokens" without a second random stream. Entries tied with the k-th largest value are all kept.
#include "fused.h"
#include "ptx.cuh"

namespace nc {

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int PER_MAX = 32;                 // logits per thread held in registers

__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);      // ascending float order == ascending unsigned order
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ u, float temperature,
              int top_k, long long* __restrict__ out) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ unsigned int s_hist[256];
  __shared__ float s_scan[32];
  __shared__ unsigned int s_prefix;
  __shared__ int s_remaining;
  __shared__ float s_total;
  __shared__ int s_choice;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = logits + (long long)row * ld;
  // contiguous chunk per thread (index order), kept in registers for every pass: V <= 32 * 1024
  const int per = ((V + SAMPLE_THREADS - 1) / SAMPLE_THREADS + 3) & ~3;
  const int lo = min(V, tid * per), hi = min(V, lo + per);
  float xv[PER_MAX];
  if ((ld & 3) == 0 && (V & 3) == 0) {
#pragma unroll
    for (int i = 0; i < PER_MAX; i += 4) {
      float4 t = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      if (lo + i < hi) t = *reinterpret_cast<const float4*>(x + lo + i);     // chunks are multiples of 4: all or nothing
      xv[i] = t.x; xv[i + 1] = t.y; xv[i + 2] = t.z; xv[i + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < PER_MAX; ++i) xv[i] = lo + i < hi ? x[lo + i] : -INFINITY;
  }

  // ---- 1. maximum and its first index
  float best = -INFINITY; int best_i = V;
#pragma unroll
  for (int i = 0; i < PER_MAX; ++i) {
    if (xv[i] > best) { best = xv[i]; best_i = lo + i; }
  }
#pragma unroll
  for (int w = 16; w > 0; w >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, w);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, w);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane]; best_i = s_idx[lane];
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, w);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, w);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[0] = best; s_idx[0] = best_i; }
  }
  __syncthreads();
  const float vmax = s_val[0];
  if (temperature <= 0.f) {
    if (tid == 0) out[row] = s_idx[0];
    return;
  }

  // ---- 2. key of the k-th largest entry (0 = keep everything)
  uint32_t threshold = 0;
  if (top_k > 0 && top_k < V) {
    if (tid == 0) { s_prefix = 0; s_remaining = top_k; }
    uint32_t mask = 0;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) s_hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
#pragma unroll
      for (int i = 0; i < PER_MAX; ++i) {
        // logits share most of their high bits, so almost every entry lands in the same few bins: lanes with
        // equal bins elect one of them to add the whole group
        const uint32_t k = ordered_key(xv[i]);
        const bool hit = lo + i < hi && (k & mask) == prefix;
        const unsigned hits = __ballot_sync(0xffffffffu, hit);
        if (hit) {
          const unsigned bin = (k >> shift) & 0xffu;
          const unsigned peers = __match_any_sync(hits, bin);
          if (lane == __ffs(peers) - 1) atomicAdd(&s_hist[bin], static_cast<unsigned>(__popc(peers)));
        }
      }
      __syncthreads();
      if (tid == 0) {
        int remaining = s_remaining, cum = 0, b = 255;
        for (; b > 0; --b) {
          if (cum + (int)s_hist[b] >= remaining) break;
          cum += (int)s_hist[b];
        }
        s_remaining = remaining - cum;
        s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      }
      mask |= 0xffu << shift;
      __syncthreads();
    }
    threshold = s_prefix;
  }

  // ---- 3. weights, scan, draw
  const float inv_t = 1.4426950408889634f / temperature;
  float part = 0.f;
#pragma unroll
  for (int i = 0; i < PER_MAX; ++i) {
    if (lo + i < hi && ordered_key(xv[i]) >= threshold) part += exp2f((xv[i] - vmax) * inv_t);
  }
  float incl = part;                              // inclusive scan inside the warp
#pragma unroll
  for (int w = 1; w < 32; w <<= 1) {
    const float o = __shfl_up_sync(0xffffffffu, incl, w);
    if (lane >= w) incl += o;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    float t = s_scan[lane];
    float acc = t;
#pragma unroll
    for (int w = 1; w < 32; w <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, acc, w);
      if (lane >= w) acc += o;
    }
    s_scan[lane] = acc - t;                       // exclusive offset of each warp
    if (lane == 31) { s_total = acc; s_choice = -1; }
  }
  __syncthreads();
  const float before = s_scan[warp] + incl - part;
  const float total = s_total;
  float target = u[row] * total;
  if (target >= total) target = total * 0.99999994f;
  if (part > 0.f && target >= before && target < before + part) {
    float run = before; int pick = -1, last = -1;
#pragma unroll
    for (int i = 0; i < PER_MAX; ++i) {
      if (pick < 0 && lo + i < hi && ordered_key(xv[i]) >= threshold) {
        last = lo + i;
        run += exp2f((xv[i] - vmax) * inv_t);
        if (target < run) pick = lo + i;
      }
    }
    atomicMax(&s_choice, pick >= 0 ? pick : last);   // rounding may leave the interval open: take its last entry
  }
  __syncthreads();
  // rounding across threads may leave no interval containing the target: fall back to the maximum
  if (tid == 0) out[row] = s_choice >= 0 ? s_choice : s_idx[0];
}

}  // namespace

cudaError_t sample_next_token(const float* logits, long long ld, int B, int V, const float* u, float temperature,
                              int top_k, long long* out, cudaStream_t s) {
  if (B <= 0 || V <= 0 || V > SAMPLE_THREADS * PER_MAX) return cudaErrorInvalidValue;
  sample_kernel<<<B, SAMPLE_THREADS, 0, s>>>(logits, ld, V, u, temperature, top_k, out);
  return cudaGetLastError();
}

}  // namespace nc
