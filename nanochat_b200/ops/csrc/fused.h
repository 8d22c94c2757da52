// Host interface of the fused elementwise / normalisation / loss / optimizer kernels.
// All pointers are device pointers; activations are bf16, scalars and gradients of
// scalars / embedding tables are fp32. Every function returns the launch status.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace nc {

// ---- transformer layer (fused.cu)
// The optional amax_* words receive max |output| (atomic max on the fp32 bits; zero them first): the per-tensor
// scale of an fp8 GEMM operand then needs no extra pass over the tensor.
cudaError_t mixnorm_fwd(const void* x, const void* x0, const float* lam_r, const float* lam_0, int layer,
                        void* xm, void* xn, float* amax_xn, int M, int C, cudaStream_t s);
cudaError_t norm_fwd(const void* x, void* y, float* amax_y, int M, int C, cudaStream_t s);
cudaError_t normadd_bwd(const void* dy, const void* x, const void* dres, void* dx, float* amax_dx, int M, int C,
                        cudaStream_t s);
cudaError_t mixnorm_bwd(const void* dxn, const void* dres, const float* dgate, const void* xm, const void* x,
                        const void* x0, const float* lam_r, const float* lam_0, int layer, void* dx, void* dx0,
                        int accumulate_dx0, float* dlam_r, float* dlam_0, float* amax_dx, int M, int C,
                        cudaStream_t s);
cudaError_t backout_norm_fwd(const void* x, const void* xb, const float* lam, void* y, int M, int C, cudaStream_t s);
cudaError_t backout_norm_bwd(const void* dy, const void* x, const void* xb, const float* lam, void* dx, void* dxb,
                             float* dlam, int M, int C, cudaStream_t s);
cudaError_t qkv_post_fwd(void* qkv, long long ld, int H, int Hkv, const void* cos_t, const void* sin_t, int T,
                         float* rstd, const void* xn, long long ld_xn, const float* wg, const void* ve,
                         const long long* idx, int M, cudaStream_t s);
cudaError_t qkv_post_bwd(void* dqkv, const void* qkv, long long ld, int H, int Hkv, const void* cos_t,
                         const void* sin_t, int T, const float* rstd, const void* xn, long long ld_xn,
                         const float* wg, const void* ve, const long long* idx, float* dve, float* dwg,
                         float* dgate_x, float* amax_qk /* optional: max |dq|, |dk| written */, int M, cudaStream_t s);
cudaError_t embed_fwd(const long long* idx, const void* wte, const float* gate_w, const float* lam, void* x,
                      void* e_last, int M, int T, int C, cudaStream_t s);
cudaError_t embed_bwd(const void* dx, const long long* idx, const void* wte, const float* gate_w, const float* lam,
                      float* dwte, float* dgate_w, float* dlam, int M, int T, int C, cudaStream_t s);
cudaError_t cast_f32_bf16(const float* src, void* dst, size_t n, cudaStream_t s);

// ---- per-tensor scaling to 8-bit floats (quant.cu); x is bf16 [rows][cols] with row pitch ld (elements)
// amax: atomic max of |x| into *amax (zero it first). quantize: q = sat(x * FMAX/amax) dense [rows][cols],
// *inv_scale = amax/FMAX; e5m2 selects the 5-bit-exponent format (FMAX 57344) instead of e4m3 (448).
cudaError_t amax_bf16(const void* x, long long ld, int rows, int cols, float* amax, cudaStream_t s);
cudaError_t quantize_bf16(const void* x, long long ld, int rows, int cols, const float* amax, void* q,
                          float* inv_scale, int e5m2, int square, cudaStream_t s);

// ---- soft-capped cross entropy over bf16 logits (loss.cu)
// loss[row] = logsumexp(cap*tanh(l/cap)) - cap*tanh(l[target]/cap); 0 for target < 0. lse is saved.
cudaError_t softcap_ce_fwd(const void* logits, long long ld, const long long* targets, float* loss, float* lse,
                           int M, int V, float cap, cudaStream_t s);
// In place: logits <- d loss / d logits * gscale[row] (gscale_stride 0 = one scalar for all rows).
cudaError_t softcap_ce_bwd(void* logits, long long ld, const long long* targets, const float* lse,
                           const float* gscale, int gscale_stride, int M, int V, int V_padded, float cap,
                           cudaStream_t s);
// dlogits as e5m2 with one scale (amax: device scalar bounding |dlogits|); out dense (M, V_padded) bytes.
cudaError_t softcap_ce_bwd_fp8(const void* logits, long long ld, const long long* targets, const float* lse,
                               const float* gscale, int gscale_stride, const float* amax, void* out, float* inv_scale,
                               int M, int V, int V_padded, float cap, cudaStream_t s);
// Inference: out[row, :V] = cap*tanh(l/cap) in fp32.
cudaError_t softcap_logits(const void* logits, long long ld, float* out, int M, int V, float cap, cudaStream_t s);

// ---- sampling (sample.cu): out[b] = argmax (temperature <= 0) or a draw from softmax(top_k(logits[b]) / temperature)
// at the uniform number u[b] in [0, 1); top_k <= 0 keeps the whole vocabulary. logits fp32 (B, V), row pitch ld.
cudaError_t sample_next_token(const float* logits, long long ld, int B, int V, const float* u, float temperature,
                              int top_k, long long* out, cudaStream_t s);

// ---- optimizer (optim.cu)
struct AdamWArgs {
  float lr, beta1, beta2, eps, wd, bias1, bias2;   // bias_i = 1 - beta_i^step
  float grad_scale;                                 // multiplies the gradient (1/world when summing ranks)
};
// p (fp32 or bf16), g (fp32 or bf16), m/v in p's dtype. Optional bf16 shadow written alongside (fp32 p only).
cudaError_t adamw_step(void* p, int p_bf16, const void* g, int g_bf16, void* m, void* v, void* shadow, size_t n,
                       AdamWArgs a, cudaStream_t s);

}  // namespace nc
