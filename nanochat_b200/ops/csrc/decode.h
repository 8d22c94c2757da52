// Host interface of the single-token decode kernels (decode.cu). All tensors bf16 unless noted; D = 128.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace nc {

enum DecodeEpilogue : int { DEC_EPI_NONE = 0, DEC_EPI_RELU2 = 1 };

// Paged KV store of one layer: a pool (n_pages, 2^page_shift tokens, Hkv, 128) plus a per-row page table
// (B, max_pages) int32. Rows may name the same page (a prompt prefix shared by every sample of a prompt is stored
// once). table == nullptr selects the contiguous (B, Tmax, Hkv, 128) layout; `c_bat` is then the row pitch, with a
// table it is the page pitch.
struct KvPages {
  const int* table = nullptr;
  int max_pages = 0;
  int page_shift = 0;
};

// out[b, n] = epi(sum_k xe[b, k] * W[n, k]) + aux[b, n]   for b < B <= 8 (aux optional). K, ldx, ldw multiples of 8.
// norm_input != 0: xe = rmsnorm(x) (the normalisation is folded into the dot products), else xe = x.
// next_w / next_bytes (optional, 16-byte aligned): memory the kernel AFTER this one will stream (its weight matrix);
// this kernel's CTAs prefetch it into L2 before their own work.
cudaError_t gemv_rows(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                      const void* aux, long long ldaux, int B, int N, int K, int epi, int norm_input,
                      const void* next_w, long long next_bytes, cudaStream_t s);

// The layer's first GEMV with the residual mix and the norm folded in: xm = bf16(lam_r[layer] * x + lam_0[layer] * x0),
// out[b, n] = sum_k rmsnorm(xm)[b, k] * W[n, k]. Also writes xm (B x K) and the first head_cols channels of
// rmsnorm(xm) to xn_head (the value-embedding gate reads them). head_cols * B <= 256.
cudaError_t gemv_rows_mix(const void* x, long long ldx, const void* x0, long long ldx0, const float* lam_r,
                          const float* lam_0, int layer, const void* W, long long ldw, void* out, long long ldo,
                          void* xm, long long ldxm, void* xn_head, long long ldxn, int head_cols, int B, int N, int K,
                          const void* next_w, long long next_bytes, cudaStream_t s);

// out[b] = e + lam * sigmoid(e[:n_gate] . gate_w) * prev[b], e = rmsnorm(wte[ids[b]]); prev[b] <- e. C, ldw, ldp, ldo
// multiples of 8; n_gate <= 32; ids outside [0, vocab) are clamped.
cudaError_t decode_embed(const long long* ids, const void* wte, long long ldw, int vocab, const float* gate_w, int n_gate,
                         const float* lam, void* prev, long long ldp, void* out, long long ldo, int B, int C,
                         cudaStream_t s);

// In place on qkv (B rows of [q heads | k heads | v heads]): rotary at position seqlens[b] + RMS norm + 1.2 on
// q and k; v += 3*sigmoid(xn[:12] . wg[hkv]) * ve[idx[b]] when ve != nullptr; k and v are appended to the
// caches at (b, seqlens[b]) (cache strides c_bat / c_tok in elements, heads contiguous). A row whose position
// is outside [0, t_max) is left alone and `status` records it. With a page table (see KvPages) the token goes to
// page table[b][pos >> page_shift]; t_max must not exceed max_pages << page_shift.
cudaError_t decode_qkv_post(void* qkv, long long ld, int H, int Hkv, const void* cos_t, const void* sin_t,
                            const int* seqlens, const void* xn, long long ld_xn, const float* wg, const void* ve,
                            long long ld_ve, const long long* idx, void* k_cache, void* v_cache, long long c_bat,
                            long long c_tok, int t_max, int B, int* status, const KvPages& pages, cudaStream_t s);

// y[b, h, :] = softmax(q[b, h] . K[b, lo..pos, hkv] * scale) V, pos = seqlens[b], lo = max(0, pos - window)
// (window < 0: 0). scratch: decode_attn_scratch_floats(B, H) floats, zeroed once before the first call.
size_t decode_attn_scratch_floats(int B, int H);
cudaError_t decode_attn(const void* q, long long ldq, const void* k_cache, const void* v_cache, long long c_bat,
                        long long c_tok, const int* seqlens, int B, int H, int Hkv, int window, float scale,
                        float* scratch, void* y, long long ldy, const KvPages& pages, cudaStream_t s);

}  // namespace nc
