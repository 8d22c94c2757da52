// Host interface of the sm_100a flash-attention kernels (attention.cu).
#pragma once

#include <cuda_runtime.h>

namespace nc {

// q: (B, Tq, H, D), k/v: (B, Tk, Hkv, D), o like q; strides in elements (innermost dim contiguous, D = 128).
// Causal with queries aligned to the END of the keys; `window` = number of keys to the left a query may
// see in addition to itself (< 0 = unlimited). lse: (B, H, Tq) fp32, natural-log sum-exp of scaled scores.
struct AttnDesc {
  const void *q, *k, *v;
  void* o;
  float* lse;
  long long q_bat, q_tok, q_head, k_bat, k_tok, k_head, v_bat, v_tok, v_head, o_bat, o_tok, o_head;
  int B, Tq, Tk, H, Hkv, D;
  int window;
  float scale;
  float* amax_o = nullptr;   // optional: receives max |o| (atomic max on the fp32 bits; zero it first)
};

cudaError_t attention_fwd(const AttnDesc& d, int* status, cudaStream_t stream);

// Backward: fwd holds q,k,v,o,lse and the problem geometry of the forward call. d_o like o; dq like q;
// dk, dv like k, v (strides in elements). delta: (B, H, Tq) fp32 scratch written by the pre-pass.
struct AttnBwdDesc {
  AttnDesc fwd;
  const void* d_o;
  long long do_bat, do_tok, do_head;
  void *dq, *dk, *dv;
  long long dq_bat, dq_tok, dq_head, dk_bat, dk_tok, dk_head, dv_bat, dv_tok, dv_head;
  float* delta;
  float* amax_dv = nullptr;  // optional: receives max |dv| (atomic max on the fp32 bits; zero it first)
};
cudaError_t attention_bwd(const AttnBwdDesc& d, int* status, cudaStream_t stream);

}  // namespace nc
