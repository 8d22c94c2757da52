// Python bindings: unpack torch tensors into raw pointers / strides and call the launchers.
// No math happens here and nothing is allocated except the one status word.
#include <torch/extension.h>
#include <atomic>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "attention.h"
#include "comm.h"
#include "fused.h"
#include "decode.h"
#include "gemm.h"
#include "optim.h"

namespace {

using at::Tensor;
using c10::optional;

static std::atomic<long long> g_launches{0};   // kernels of this extension launched so far

#define NC_CHECK(expr)                                                                         \
  do {                                                                                         \
    ++g_launches;                                                                              \
    cudaError_t _e = (expr);                                                                   \
    TORCH_CHECK(_e == cudaSuccess, "nanochat_b200 kernel launch failed: ", cudaGetErrorString(_e), \
                " at " #expr);                                                                 \
  } while (0)

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

Tensor& status_tensor(const at::Device& dev) {
  static std::vector<Tensor> per_dev(64);
  Tensor& t = per_dev[dev.index()];
  if (!t.defined()) t = torch::zeros({4}, torch::dtype(torch::kInt32).device(dev));
  return t;
}
int* status_ptr(const Tensor& like) { return status_tensor(like.device()).data_ptr<int>(); }

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, " must be a CUDA bf16 tensor");
}
const void* optptr(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
float* opt_scalar(const optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->numel() == 1, "expected a CUDA fp32 scalar");
  return t->data_ptr<float>();
}

// ------------------------------------------------------------------------------ GEMM
// Operands are bf16, or 8-bit floats (e4m3 / e5m2, both operands) with optional per-tensor scales.
void gemm(const Tensor& A, const Tensor& B, Tensor& C, const optional<Tensor>& aux, bool a_mn, bool b_mn,
          double alpha, double beta, int64_t epi, int64_t bn, int64_t pair, const optional<Tensor>& scale_a,
          const optional<Tensor>& scale_b, const optional<Tensor>& amax_out, bool symmetric) {
  const bool fp8 = A.scalar_type() == at::kFloat8_e4m3fn || A.scalar_type() == at::kFloat8_e5m2;
  if (fp8) {
    TORCH_CHECK(A.is_cuda() && B.is_cuda(), "fp8 operands must be CUDA tensors");
    TORCH_CHECK(B.scalar_type() == at::kFloat8_e4m3fn || B.scalar_type() == at::kFloat8_e5m2, "B must be fp8 like A");
  } else {
    check_bf16(A, "A");
    check_bf16(B, "B");
  }
  TORCH_CHECK(C.is_cuda() && (C.scalar_type() == at::kBFloat16 || C.scalar_type() == at::kFloat), "C dtype");
  TORCH_CHECK(A.dim() == B.dim() && A.dim() == C.dim() && (A.dim() == 2 || A.dim() == 3), "gemm rank");
  const c10::cuda::CUDAGuard guard(A.device());
  const int nd = A.dim();
  auto chk = [&](const Tensor& t, const char* n) {
    TORCH_CHECK(t.stride(nd - 1) == 1, n, ": innermost dim must be contiguous");
  };
  chk(A, "A"); chk(B, "B"); chk(C, "C");
  nc::GemmDesc d{};
  d.batch = nd == 3 ? (int)C.size(0) : 1;
  d.M = (int)C.size(nd - 2);
  d.N = (int)C.size(nd - 1);
  d.K = (int)(a_mn ? A.size(nd - 2) : A.size(nd - 1));
  TORCH_CHECK((a_mn ? A.size(nd - 1) : A.size(nd - 2)) == d.M, "A shape does not match C");
  TORCH_CHECK((b_mn ? B.size(nd - 1) : B.size(nd - 2)) == d.N, "B shape does not match C");
  TORCH_CHECK((b_mn ? B.size(nd - 2) : B.size(nd - 1)) == d.K, "A/B reduction dims differ");
  d.A = A.data_ptr(); d.a_mn = a_mn; d.lda = A.stride(nd - 2); d.bsa = nd == 3 ? A.stride(0) : 0;
  d.B = B.data_ptr(); d.b_mn = b_mn; d.ldb = B.stride(nd - 2); d.bsb = nd == 3 ? B.stride(0) : 0;
  d.C = C.data_ptr(); d.c_f32 = C.scalar_type() == at::kFloat; d.ldc = C.stride(nd - 2);
  d.bsc = nd == 3 ? C.stride(0) : 0;
  if (aux.has_value() && aux->defined()) {
    TORCH_CHECK(aux->scalar_type() == C.scalar_type() && aux->stride(nd - 1) == 1, "aux must match C");
    d.aux = aux->data_ptr(); d.ldaux = aux->stride(nd - 2); d.bsaux = nd == 3 ? aux->stride(0) : 0;
  }
  d.alpha = (float)alpha; d.beta = (float)beta; d.epi = (int)epi; d.bn = (int)bn; d.pair = (int)pair;
  d.symmetric = symmetric ? 1 : 0;
  auto scalar = [&](const optional<Tensor>& t, const char* n) -> float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->numel() == 1, n, " must be a CUDA fp32 scalar");
    return t->data_ptr<float>();
  };
  d.scale_a = scalar(scale_a, "scale_a");
  d.scale_b = scalar(scale_b, "scale_b");
  d.amax_out = scalar(amax_out, "amax_out");
  if (fp8) {
    d.a_e5m2 = A.scalar_type() == at::kFloat8_e5m2;
    d.b_e5m2 = B.scalar_type() == at::kFloat8_e5m2;
    NC_CHECK(nc::gemm_fp8(d, status_ptr(A), cur_stream()));
  } else {
    NC_CHECK(nc::gemm_bf16(d, status_ptr(A), cur_stream()));
  }
}

// Copies the upper triangle of every (n, n) matrix of a bf16 (n, n) or (batch, n, n) tensor over its lower triangle.
void symmetrize(Tensor& C) {
  check_bf16(C, "C");
  const int nd = C.dim();
  TORCH_CHECK((nd == 2 || nd == 3) && C.size(nd - 1) == C.size(nd - 2) && C.stride(nd - 1) == 1, "symmetrize: square matrices");
  const c10::cuda::CUDAGuard guard(C.device());
  NC_CHECK(nc::symmetrize_bf16(C.data_ptr(), (int)C.size(nd - 1), C.stride(nd - 2), nd == 3 ? C.stride(0) : 0,
                               nd == 3 ? (int)C.size(0) : 1, cur_stream()));
}

// MXFP8: A (M, K) and B (N, K) row-major fp8, sfa / sfb uint8 in the blocked scale layout (see gemm.h), C (M, N).
void gemm_mx(const Tensor& A, const Tensor& sfa, const Tensor& B, const Tensor& sfb, Tensor& C, const optional<Tensor>& aux,
             double alpha, double beta, int64_t epi, int64_t bn) {
  auto is8 = [](const Tensor& t) { return t.scalar_type() == at::kFloat8_e4m3fn || t.scalar_type() == at::kFloat8_e5m2; };
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && is8(A) && is8(B) && A.dim() == 2 && B.dim() == 2, "gemm_mx: 2-D fp8 operands");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && C.stride(1) == 1 && A.size(1) == B.size(1), "gemm_mx: K-major A, B");
  TORCH_CHECK(C.scalar_type() == at::kBFloat16 || C.scalar_type() == at::kFloat, "gemm_mx: C bf16 or fp32");
  TORCH_CHECK(C.size(0) == A.size(0) && C.size(1) == B.size(0), "gemm_mx: C shape");
  const int64_t M = A.size(0), N = B.size(0), K = A.size(1);
  TORCH_CHECK(K % 128 == 0, "gemm_mx: K must be a multiple of 128");
  auto chunks = [&](int64_t rows) { return ((rows + 127) / 128) * (K / 128) * 512; };
  TORCH_CHECK(sfa.scalar_type() == at::kByte && sfa.is_contiguous() && sfa.numel() >= chunks(M), "gemm_mx: sfa too small");
  TORCH_CHECK(sfb.scalar_type() == at::kByte && sfb.is_contiguous() && sfb.numel() >= chunks(N), "gemm_mx: sfb too small");
  const c10::cuda::CUDAGuard guard(A.device());
  nc::GemmDesc d{};
  d.batch = 1; d.M = (int)M; d.N = (int)N; d.K = (int)K;
  d.A = A.data_ptr(); d.lda = A.stride(0); d.B = B.data_ptr(); d.ldb = B.stride(0);
  d.C = C.data_ptr(); d.c_f32 = C.scalar_type() == at::kFloat; d.ldc = C.stride(0);
  if (aux.has_value() && aux->defined()) {
    TORCH_CHECK(aux->scalar_type() == C.scalar_type() && aux->stride(1) == 1, "aux must match C");
    d.aux = aux->data_ptr(); d.ldaux = aux->stride(0);
  }
  d.alpha = (float)alpha; d.beta = (float)beta; d.epi = (int)epi; d.bn = (int)bn;
  d.a_e5m2 = A.scalar_type() == at::kFloat8_e5m2;
  d.b_e5m2 = B.scalar_type() == at::kFloat8_e5m2;
  nc::MxScales sf{sfa.data_ptr<uint8_t>(), sfb.data_ptr<uint8_t>()};
  NC_CHECK(nc::gemm_mxfp8(d, sf, status_ptr(A), cur_stream()));
}
// x (R, K) bf16 rows -> q (R, K) fp8 (its dtype picks the format) + blocked E8M0 scales (pre-filled by the caller).
void mx_quantize(const Tensor& x, Tensor& q, Tensor& sf) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && q.is_contiguous() && q.sizes() == x.sizes(), "mx_quantize: shapes");
  TORCH_CHECK(q.scalar_type() == at::kFloat8_e4m3fn || q.scalar_type() == at::kFloat8_e5m2, "mx_quantize: q fp8");
  const int64_t R = x.size(0), K = x.size(1);
  TORCH_CHECK(K % 128 == 0, "mx_quantize: K must be a multiple of 128");
  TORCH_CHECK(sf.scalar_type() == at::kByte && sf.is_contiguous() && sf.numel() >= ((R + 127) / 128) * (K / 128) * 512,
              "mx_quantize: scale buffer too small");
  const c10::cuda::CUDAGuard guard(x.device());
  NC_CHECK(nc::mx_quantize_bf16(x.data_ptr(), x.stride(0), (int)R, (int)K, q.data_ptr(), sf.data_ptr<uint8_t>(),
                                q.scalar_type() == at::kFloat8_e5m2, cur_stream()));
}

int64_t gemm_pick_bn(int64_t M, int64_t N, int64_t batch) { return nc::gemm_pick_bn((int)M, (int)N, (int)batch); }

std::vector<int64_t> read_status(const Tensor& like) {
  Tensor h = status_tensor(like.device()).cpu();
  status_tensor(like.device()).zero_();
  auto a = h.accessor<int, 1>();
  return {a[0], a[1], a[2], a[3]};
}

// --------------------------------------------------------------------- layer kernels
void mixnorm_fwd(const Tensor& x, const Tensor& x0, const Tensor& lam_r, const Tensor& lam_0, int64_t layer,
                 Tensor& xm, Tensor& xn, const optional<Tensor>& amax) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  NC_CHECK(nc::mixnorm_fwd(x.data_ptr(), x0.data_ptr(), lam_r.data_ptr<float>(), lam_0.data_ptr<float>(), (int)layer,
                           xm.data_ptr(), xn.data_ptr(), opt_scalar(amax), M, C, cur_stream()));
}
void norm_fwd(const Tensor& x, Tensor& y, const optional<Tensor>& amax) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  NC_CHECK(nc::norm_fwd(x.data_ptr(), y.data_ptr(), opt_scalar(amax), M, C, cur_stream()));
}
void normadd_bwd(const Tensor& dy, const Tensor& x, const optional<Tensor>& dres, Tensor& dx,
                 const optional<Tensor>& amax) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  NC_CHECK(nc::normadd_bwd(dy.data_ptr(), x.data_ptr(), optptr(dres), dx.data_ptr(), opt_scalar(amax), M, C,
                           cur_stream()));
}
void mixnorm_bwd(const Tensor& dxn, const Tensor& dres, const optional<Tensor>& dgate, const Tensor& xm,
                 const Tensor& x, const Tensor& x0, const Tensor& lam_r, const Tensor& lam_0, int64_t layer,
                 Tensor& dx, Tensor& dx0, bool accumulate_dx0, Tensor& dlam_r, Tensor& dlam_0,
                 const optional<Tensor>& amax) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  NC_CHECK(nc::mixnorm_bwd(dxn.data_ptr(), dres.data_ptr(), (const float*)optptr(dgate), xm.data_ptr(), x.data_ptr(),
                           x0.data_ptr(), lam_r.data_ptr<float>(), lam_0.data_ptr<float>(), (int)layer, dx.data_ptr(),
                           dx0.data_ptr(), accumulate_dx0, dlam_r.data_ptr<float>(), dlam_0.data_ptr<float>(),
                           opt_scalar(amax), M, C, cur_stream()));
}
void backout_norm_fwd(const Tensor& x, const optional<Tensor>& xb, const Tensor& lam, Tensor& y) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  NC_CHECK(nc::backout_norm_fwd(x.data_ptr(), optptr(xb), lam.data_ptr<float>(), y.data_ptr(), M, C, cur_stream()));
}
void backout_norm_bwd(const Tensor& dy, const Tensor& x, const optional<Tensor>& xb, const Tensor& lam, Tensor& dx,
                      const optional<Tensor>& dxb, Tensor& dlam) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  NC_CHECK(nc::backout_norm_bwd(dy.data_ptr(), x.data_ptr(), optptr(xb), lam.data_ptr<float>(), dx.data_ptr(),
                                const_cast<void*>(optptr(dxb)), dlam.data_ptr<float>(), M, C, cur_stream()));
}
void qkv_post_fwd(Tensor& qkv, int64_t H, int64_t Hkv, const Tensor& cos_t, const Tensor& sin_t, int64_t T,
                  Tensor& rstd, const optional<Tensor>& xn, const optional<Tensor>& wg, const optional<Tensor>& ve,
                  const optional<Tensor>& idx) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int M = (int)(qkv.numel() / qkv.size(-1));
  const bool has_ve = ve.has_value() && ve->defined();
  NC_CHECK(nc::qkv_post_fwd(qkv.data_ptr(), qkv.stride(-2), (int)H, (int)Hkv, cos_t.data_ptr(), sin_t.data_ptr(),
                            (int)T, rstd.data_ptr<float>(), has_ve ? xn->data_ptr() : nullptr,
                            has_ve ? xn->stride(-2) : 0, has_ve ? wg->data_ptr<float>() : nullptr,
                            has_ve ? ve->data_ptr() : nullptr, has_ve ? (const long long*)idx->data_ptr<int64_t>() : nullptr,
                            M, cur_stream()));
}
void qkv_post_bwd(Tensor& dqkv, const Tensor& qkv, int64_t H, int64_t Hkv, const Tensor& cos_t, const Tensor& sin_t,
                  int64_t T, const Tensor& rstd, const optional<Tensor>& xn, const optional<Tensor>& wg,
                  const optional<Tensor>& ve, const optional<Tensor>& idx, const optional<Tensor>& dve,
                  const optional<Tensor>& dwg, const optional<Tensor>& dgate_x, const optional<Tensor>& amax_qk) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int M = (int)(qkv.numel() / qkv.size(-1));
  const bool has_ve = ve.has_value() && ve->defined();
  TORCH_CHECK(dqkv.stride(-2) == qkv.stride(-2), "dqkv/qkv pitch mismatch");
  NC_CHECK(nc::qkv_post_bwd(dqkv.data_ptr(), qkv.data_ptr(), qkv.stride(-2), (int)H, (int)Hkv, cos_t.data_ptr(),
                            sin_t.data_ptr(), (int)T, rstd.data_ptr<float>(), has_ve ? xn->data_ptr() : nullptr,
                            has_ve ? xn->stride(-2) : 0, has_ve ? wg->data_ptr<float>() : nullptr,
                            has_ve ? ve->data_ptr() : nullptr,
                            has_ve ? (const long long*)idx->data_ptr<int64_t>() : nullptr,
                            has_ve ? dve->data_ptr<float>() : nullptr, has_ve ? dwg->data_ptr<float>() : nullptr,
                            has_ve ? dgate_x->data_ptr<float>() : nullptr, opt_scalar(amax_qk), M, cur_stream()));
}
void embed_fwd(const Tensor& idx, const Tensor& wte, const Tensor& gate_w, const Tensor& lam, Tensor& x,
               const optional<Tensor>& e_last) {
  const c10::cuda::CUDAGuard guard(wte.device());
  const int C = (int)wte.size(1), T = (int)idx.size(1), M = (int)idx.numel();
  NC_CHECK(nc::embed_fwd((const long long*)idx.data_ptr<int64_t>(), wte.data_ptr(), gate_w.data_ptr<float>(),
                         lam.data_ptr<float>(), x.data_ptr(), const_cast<void*>(optptr(e_last)), M, T, C, cur_stream()));
}
void embed_bwd(const Tensor& dx, const Tensor& idx, const Tensor& wte, const Tensor& gate_w, const Tensor& lam,
               Tensor& dwte, Tensor& dgate_w, Tensor& dlam) {
  const c10::cuda::CUDAGuard guard(wte.device());
  const int C = (int)wte.size(1), T = (int)idx.size(1), M = (int)idx.numel();
  NC_CHECK(nc::embed_bwd(dx.data_ptr(), (const long long*)idx.data_ptr<int64_t>(), wte.data_ptr(),
                         gate_w.data_ptr<float>(), lam.data_ptr<float>(), dwte.data_ptr<float>(),
                         dgate_w.data_ptr<float>(), dlam.data_ptr<float>(), M, T, C, cur_stream()));
}
// x: bf16 (rows, cols), rows may be strided. amax: fp32 scalar (accumulates a max; zero it first).
void amax_bf16(const Tensor& x, Tensor& amax) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "amax: 2-D, innermost contiguous");
  TORCH_CHECK(amax.is_cuda() && amax.scalar_type() == at::kFloat && amax.numel() == 1, "amax scalar");
  const c10::cuda::CUDAGuard guard(x.device());
  NC_CHECK(nc::amax_bf16(x.data_ptr(), x.stride(0), (int)x.size(0), (int)x.size(1), amax.data_ptr<float>(), cur_stream()));
}
// q: fp8 (e4m3fn or e5m2) dense (rows, cols); inv_scale: fp32 scalar that receives the de-quantisation factor.
// square: quantise x^2 instead of x, `amax` holding max|x|.
void quantize_bf16(const Tensor& x, const Tensor& amax, Tensor& q, Tensor& inv_scale, bool square) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "quantize: 2-D, innermost contiguous");
  const bool e5 = q.scalar_type() == at::kFloat8_e5m2;
  TORCH_CHECK(q.is_cuda() && (e5 || q.scalar_type() == at::kFloat8_e4m3fn) && q.is_contiguous() &&
              q.numel() == x.numel(), "q must be a dense fp8 tensor of x's size");
  TORCH_CHECK(amax.scalar_type() == at::kFloat && inv_scale.scalar_type() == at::kFloat && amax.numel() == 1 &&
              inv_scale.numel() == 1, "scalars");
  const c10::cuda::CUDAGuard guard(x.device());
  NC_CHECK(nc::quantize_bf16(x.data_ptr(), x.stride(0), (int)x.size(0), (int)x.size(1), amax.data_ptr<float>(),
                             q.data_ptr(), inv_scale.data_ptr<float>(), e5 ? 1 : 0, square ? 1 : 0, cur_stream()));
}

void cast_f32_bf16(const Tensor& src, Tensor& dst) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel(), "cast shapes");
  NC_CHECK(nc::cast_f32_bf16(src.data_ptr<float>(), dst.data_ptr(), (size_t)src.numel(), cur_stream()));
}

// ------------------------------------------------------------------------------ loss
void softcap_ce_fwd(const Tensor& logits, const Tensor& targets, Tensor& loss, Tensor& lse, int64_t V, double cap) {
  const c10::cuda::CUDAGuard guard(logits.device());
  NC_CHECK(nc::softcap_ce_fwd(logits.data_ptr(), logits.stride(0), (const long long*)targets.data_ptr<int64_t>(),
                              loss.data_ptr<float>(), lse.data_ptr<float>(), (int)logits.size(0), (int)V, (float)cap,
                              cur_stream()));
}
void softcap_ce_bwd(Tensor& logits, const Tensor& targets, const Tensor& lse, const Tensor& gscale, int64_t V,
                    double cap) {
  const c10::cuda::CUDAGuard guard(logits.device());
  NC_CHECK(nc::softcap_ce_bwd(logits.data_ptr(), logits.stride(0), (const long long*)targets.data_ptr<int64_t>(),
                              lse.data_ptr<float>(), gscale.data_ptr<float>(), gscale.numel() > 1 ? 1 : 0,
                              (int)logits.size(0), (int)V, (int)logits.size(1), (float)cap, cur_stream()));
}
void softcap_ce_bwd_fp8(const Tensor& logits, const Tensor& targets, const Tensor& lse, const Tensor& gscale,
                        const Tensor& amax, Tensor& out, Tensor& inv_scale, int64_t V, double cap) {
  const c10::cuda::CUDAGuard guard(logits.device());
  check_bf16(logits, "logits");
  TORCH_CHECK(out.scalar_type() == at::kFloat8_e5m2 && out.is_contiguous() && out.sizes() == logits.sizes(),
              "out: contiguous e5m2 shaped like the logits");
  TORCH_CHECK(amax.scalar_type() == at::kFloat && amax.numel() == 1 && inv_scale.scalar_type() == at::kFloat &&
              inv_scale.numel() == 1, "amax / inv_scale: fp32 device scalars");
  NC_CHECK(nc::softcap_ce_bwd_fp8(logits.data_ptr(), logits.stride(0), (const long long*)targets.data_ptr<int64_t>(),
                                  lse.data_ptr<float>(), gscale.data_ptr<float>(), gscale.numel() > 1 ? 1 : 0,
                                  amax.data_ptr<float>(), out.data_ptr(), inv_scale.data_ptr<float>(),
                                  (int)logits.size(0), (int)V, (int)logits.size(1), (float)cap, cur_stream()));
}
void softcap_logits(const Tensor& logits, Tensor& out, int64_t V, double cap) {
  const c10::cuda::CUDAGuard guard(logits.device());
  NC_CHECK(nc::softcap_logits(logits.data_ptr(), logits.stride(0), out.data_ptr<float>(), (int)logits.size(0), (int)V,
                              (float)cap, cur_stream()));
}

// ---------------------------------------------------------------------------- decode
static std::pair<const void*, long long> next_weights(const optional<Tensor>& t) {
  if (!t.has_value() || !t->defined() || !t->is_contiguous()) return {nullptr, 0};
  return {t->data_ptr(), (long long)t->numel() * (long long)t->element_size()};
}

void gemv_rows(const Tensor& x, const Tensor& W, Tensor& out, const optional<Tensor>& aux, int64_t epi,
               bool norm_input, const optional<Tensor>& next_w) {
  check_bf16(x, "x"); check_bf16(W, "W"); check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && W.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && W.stride(1) == 1 &&
              out.stride(1) == 1, "gemv: 2-D row-major tensors");
  TORCH_CHECK(x.size(1) == W.size(1) && out.size(0) == x.size(0) && out.size(1) == W.size(0), "gemv shapes");
  const c10::cuda::CUDAGuard guard(x.device());
  const void* ap = nullptr; long long lda = 0;
  if (aux.has_value() && aux->defined()) {
    check_bf16(*aux, "aux");
    TORCH_CHECK(aux->sizes() == out.sizes() && aux->stride(1) == 1, "aux must match out");
    ap = aux->data_ptr(); lda = aux->stride(0);
  }
  NC_CHECK(nc::gemv_rows(x.data_ptr(), x.stride(0), W.data_ptr(), W.stride(0), out.data_ptr(), out.stride(0), ap, lda,
                         (int)x.size(0), (int)W.size(0), (int)x.size(1), (int)epi, norm_input ? 1 : 0,
                         next_weights(next_w).first, next_weights(next_w).second, cur_stream()));
}

// x, x0, xm, xn: (B, K) bf16 (xn: only its first 16 channels are written); lam_r, lam_0: fp32 (layers); W: (N, K); out: (B, N).
void gemv_rows_mix(const Tensor& x, const Tensor& x0, const Tensor& lam_r, const Tensor& lam_0, int64_t layer,
                   const Tensor& W, Tensor& out, Tensor& xm, Tensor& xn, const optional<Tensor>& next_w) {
  check_bf16(x, "x"); check_bf16(x0, "x0"); check_bf16(W, "W"); check_bf16(out, "out"); check_bf16(xm, "xm"); check_bf16(xn, "xn");
  TORCH_CHECK(x.dim() == 2 && W.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && x0.stride(1) == 1 && W.stride(1) == 1 &&
              out.stride(1) == 1 && xm.stride(1) == 1 && xn.stride(1) == 1, "gemv_rows_mix: 2-D row-major tensors");
  TORCH_CHECK(x.size(1) == W.size(1) && out.size(0) == x.size(0) && out.size(1) == W.size(0) && x0.sizes() == x.sizes() &&
              xm.sizes() == x.sizes() && xn.sizes() == x.sizes() && x.size(1) >= 16, "gemv_rows_mix shapes");
  TORCH_CHECK(lam_r.is_cuda() && lam_0.is_cuda() && lam_r.scalar_type() == at::kFloat && lam_0.scalar_type() == at::kFloat &&
              lam_r.is_contiguous() && lam_0.is_contiguous() && layer >= 0 && layer < lam_r.numel() && layer < lam_0.numel(),
              "lambdas: fp32 (layers)");
  const c10::cuda::CUDAGuard guard(x.device());
  NC_CHECK(nc::gemv_rows_mix(x.data_ptr(), x.stride(0), x0.data_ptr(), x0.stride(0), lam_r.data_ptr<float>(),
                             lam_0.data_ptr<float>(), (int)layer, W.data_ptr(), W.stride(0), out.data_ptr(), out.stride(0),
                             xm.data_ptr(), xm.stride(0), xn.data_ptr(), xn.stride(0), 16, (int)x.size(0), (int)W.size(0),
                             (int)x.size(1), next_weights(next_w).first, next_weights(next_w).second, cur_stream()));
}

// ids: int64 (B) or (B, 1); wte: (V, C) bf16; gate_w: fp32 (n_gate); lam: fp32 (1); prev, out: (B, C) bf16.
void decode_embed(const Tensor& ids, const Tensor& wte, const Tensor& gate_w, const Tensor& lam, Tensor& prev, Tensor& out) {
  check_bf16(wte, "wte"); check_bf16(prev, "prev"); check_bf16(out, "out");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.numel() == out.size(0), "ids int64 (B)");
  TORCH_CHECK(wte.dim() == 2 && wte.stride(1) == 1 && out.dim() == 2 && out.stride(1) == 1 && prev.dim() == 2 &&
              prev.stride(1) == 1 && out.size(1) == wte.size(1) && prev.sizes() == out.sizes(), "embedding shapes");
  TORCH_CHECK(gate_w.is_cuda() && gate_w.scalar_type() == at::kFloat && gate_w.is_contiguous() && lam.is_cuda() &&
              lam.scalar_type() == at::kFloat && lam.numel() == 1, "gate weights fp32, lambda fp32 (1)");
  const c10::cuda::CUDAGuard guard(out.device());
  NC_CHECK(nc::decode_embed(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), wte.data_ptr(), wte.stride(0),
                            (int)wte.size(0), gate_w.data_ptr<float>(), (int)gate_w.numel(), lam.data_ptr<float>(),
                            prev.data_ptr(), prev.stride(0), out.data_ptr(), out.stride(0), (int)out.size(0),
                            (int)out.size(1), cur_stream()));
}

// qkv: (B, (H+2Hkv)*128); cos/sin: (Tmax, 64); seqlens: int32 (B); k_cache/v_cache: (B, Tmax, Hkv, 128) of one layer.
// Paged store: k_cache/v_cache are one layer's pool (n_pages, page_tokens, Hkv, 128), `table` int32 (B, max_pages),
// `t_max` the per-row capacity in tokens.
static nc::KvPages kv_pages(const optional<Tensor>& table, const Tensor& cache, int64_t B) {
  nc::KvPages pg;
  if (!table.has_value() || !table->defined()) return pg;
  TORCH_CHECK(table->is_cuda() && table->scalar_type() == at::kInt && table->dim() == 2 && table->is_contiguous() &&
              table->size(0) == B, "page table: contiguous int32 (B, max_pages)");
  const int64_t tokens = cache.size(1);
  TORCH_CHECK(tokens > 0 && (tokens & (tokens - 1)) == 0, "page size must be a power of two");
  int shift = 0;
  while ((int64_t(1) << shift) < tokens) ++shift;
  pg.table = table->data_ptr<int>();
  pg.max_pages = (int)table->size(1);
  pg.page_shift = shift;
  return pg;
}

void decode_qkv_post(Tensor& qkv, int64_t H, int64_t Hkv, const Tensor& cos_t, const Tensor& sin_t, const Tensor& seqlens,
                     const optional<Tensor>& xn, const optional<Tensor>& wg, const optional<Tensor>& ve,
                     const optional<Tensor>& idx, Tensor& k_cache, Tensor& v_cache, const optional<Tensor>& table,
                     int64_t t_max) {
  check_bf16(qkv, "qkv"); check_bf16(cos_t, "cos"); check_bf16(sin_t, "sin"); check_bf16(k_cache, "k_cache");
  check_bf16(v_cache, "v_cache");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (H + 2 * Hkv) * 128, "qkv shape");
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(-1) == 64, "rotary tables (T, 64)");
  TORCH_CHECK(seqlens.scalar_type() == at::kInt && seqlens.numel() == qkv.size(0), "seqlens int32 (B)");
  const bool paged = table.has_value() && table->defined();
  TORCH_CHECK(k_cache.dim() == 4 && (paged || k_cache.size(0) == qkv.size(0)) && k_cache.size(2) == Hkv &&
              k_cache.size(3) == 128 && k_cache.stride(3) == 1 && k_cache.stride(2) == 128 &&
              v_cache.strides() == k_cache.strides(), "cache layout");
  const nc::KvPages pages = kv_pages(table, k_cache, qkv.size(0));
  const int64_t cap = paged ? t_max : k_cache.size(1);
  const bool has_ve = ve.has_value() && ve->defined();
  if (has_ve) {
    check_bf16(*ve, "ve"); check_bf16(*xn, "xn");
    TORCH_CHECK(wg->scalar_type() == at::kFloat && wg->is_contiguous() && idx->scalar_type() == at::kLong, "ve gate args");
  }
  const c10::cuda::CUDAGuard guard(qkv.device());
  NC_CHECK(nc::decode_qkv_post(qkv.data_ptr(), qkv.stride(0), (int)H, (int)Hkv, cos_t.data_ptr(), sin_t.data_ptr(),
                               seqlens.data_ptr<int>(), has_ve ? xn->data_ptr() : nullptr, has_ve ? xn->stride(0) : 0,
                               has_ve ? wg->data_ptr<float>() : nullptr, has_ve ? ve->data_ptr() : nullptr,
                               has_ve ? ve->stride(0) : 0, has_ve ? reinterpret_cast<const long long*>(idx->data_ptr<int64_t>()) : nullptr,
                               k_cache.data_ptr(), v_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1),
                               (int)cap, (int)qkv.size(0), status_ptr(qkv), pages, cur_stream()));
}

// q: (B, H*128) view (row pitch free); y: (B, H*128); scratch fp32 with at least decode_attn_scratch(B, H) elements.
void decode_attn(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& seqlens, int64_t H,
                 int64_t Hkv, int64_t window, double scale, Tensor& scratch, Tensor& y, const optional<Tensor>& table) {
  check_bf16(q, "q"); check_bf16(y, "y");
  TORCH_CHECK(scratch.scalar_type() == at::kFloat &&
              (size_t)scratch.numel() >= nc::decode_attn_scratch_floats((int)q.size(0), (int)H), "scratch too small");
  const c10::cuda::CUDAGuard guard(q.device());
  NC_CHECK(nc::decode_attn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.stride(0),
                           k_cache.stride(1), seqlens.data_ptr<int>(), (int)q.size(0), (int)H, (int)Hkv, (int)window,
                           (float)scale, scratch.data_ptr<float>(), y.data_ptr(), y.stride(0),
                           kv_pages(table, k_cache, q.size(0)), cur_stream()));
}
int64_t decode_attn_scratch(int64_t B, int64_t H) { return (int64_t)nc::decode_attn_scratch_floats((int)B, (int)H); }

void sample_next_token(const Tensor& logits, const Tensor& u, double temperature, int64_t top_k, Tensor& out) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1,
              "logits: CUDA fp32 (B, V)");
  TORCH_CHECK(u.is_cuda() && u.scalar_type() == at::kFloat && u.is_contiguous() && u.numel() == logits.size(0), "u: fp32 (B)");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kLong && out.is_contiguous() && out.numel() == logits.size(0),
              "out: int64 (B)");
  const c10::cuda::CUDAGuard guard(logits.device());
  NC_CHECK(nc::sample_next_token(logits.data_ptr<float>(), logits.stride(0), (int)logits.size(0), (int)logits.size(1),
                                 u.data_ptr<float>(), (float)temperature, (int)top_k,
                                 reinterpret_cast<long long*>(out.data_ptr<int64_t>()), cur_stream()));
}

// ------------------------------------------------------------------------- optimizer
void adamw_step(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const optional<Tensor>& shadow, double lr,
                double beta1, double beta2, double eps, double wd, int64_t step, double grad_scale) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw: contiguous");
  TORCH_CHECK(m.scalar_type() == p.scalar_type() && v.scalar_type() == p.scalar_type(), "adamw: state dtype");
  nc::AdamWArgs a;
  a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2; a.eps = (float)eps; a.wd = (float)wd;
  a.bias1 = (float)(1.0 - std::pow(beta1, (double)step));
  a.bias2 = (float)(1.0 - std::pow(beta2, (double)step));
  a.grad_scale = (float)grad_scale;
  NC_CHECK(nc::adamw_step(p.data_ptr(), p.scalar_type() == at::kBFloat16, g.data_ptr(),
                          g.scalar_type() == at::kBFloat16, m.data_ptr(), v.data_ptr(),
                          const_cast<void*>(optptr(shadow)), (size_t)p.numel(), a, cur_stream()));
}
void muon_momentum(const Tensor& g, Tensor& buf, Tensor& X, Tensor& rowss, Tensor& total, double mu,
                   double grad_scale) {
  const c10::cuda::CUDAGuard guard(g.device());
  NC_CHECK(nc::muon_momentum(g.data_ptr<float>(), buf.data_ptr<float>(), X.data_ptr(), rowss.data_ptr<float>(),
                             total.data_ptr<float>(), (float)mu, (float)grad_scale, (int)g.size(0), (int)g.size(1),
                             (int)g.size(2), cur_stream()));
  g_launches += 1;   // momentum + per-matrix total
}
void muon_equilibrate(Tensor& X, const Tensor& rowss, const Tensor& total, Tensor& rowss2, Tensor& total2) {
  const c10::cuda::CUDAGuard guard(X.device());
  NC_CHECK(nc::muon_equilibrate(X.data_ptr(), rowss.data_ptr<float>(), total.data_ptr<float>(),
                                rowss2.data_ptr<float>(), total2.data_ptr<float>(), (int)X.size(0), (int)X.size(1),
                                (int)X.size(2), cur_stream()));
  g_launches += 2;   // equilibrate + total + scale
}
void muon_finish(Tensor& p, const Tensor& X, Tensor& second_buf, Tensor& ss, Tensor& scale,
                 const optional<Tensor>& shadow, double lr, double wd, double beta2) {
  const c10::cuda::CUDAGuard guard(X.device());
  NC_CHECK(nc::muon_finish(p.data_ptr<float>(), X.data_ptr(), second_buf.data_ptr<float>(), ss.data_ptr<float>(),
                           scale.data_ptr<float>(), const_cast<void*>(optptr(shadow)), (int)X.size(0), (int)X.size(1),
                           (int)X.size(2), (float)lr, (float)wd, (float)beta2, cur_stream()));
  g_launches += 2;   // sumsq + stats + apply
}
int64_t launch_count() { return (int64_t)g_launches.load(); }

// ------------------------------------------------------------------------- attention
void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& o, Tensor& lse, int64_t window,
              double scale, const optional<Tensor>& amax_o) {
  const c10::cuda::CUDAGuard guard(q.device());
  nc::AttnDesc d{};
  d.B = (int)q.size(0); d.Tq = (int)q.size(1); d.H = (int)q.size(2); d.D = (int)q.size(3);
  d.Tk = (int)k.size(1); d.Hkv = (int)k.size(2);
  d.q = q.data_ptr(); d.k = k.data_ptr(); d.v = v.data_ptr(); d.o = o.data_ptr(); d.lse = lse.data_ptr<float>();
  d.q_tok = q.stride(1); d.k_tok = k.stride(1); d.v_tok = v.stride(1); d.o_tok = o.stride(1);
  d.q_bat = q.stride(0); d.k_bat = k.stride(0); d.v_bat = v.stride(0); d.o_bat = o.stride(0);
  d.q_head = q.stride(2); d.k_head = k.stride(2); d.v_head = v.stride(2); d.o_head = o.stride(2);
  d.window = (int)window; d.scale = (float)scale;
  d.amax_o = opt_scalar(amax_o);
  NC_CHECK(nc::attention_fwd(d, status_ptr(q), cur_stream()));
}

void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& lse,
              const Tensor& d_o, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& delta, int64_t window, double scale,
              const optional<Tensor>& amax_dv) {
  const c10::cuda::CUDAGuard guard(q.device());
  nc::AttnBwdDesc d{};
  nc::AttnDesc& f = d.fwd;
  f.B = (int)q.size(0); f.Tq = (int)q.size(1); f.H = (int)q.size(2); f.D = (int)q.size(3);
  f.Tk = (int)k.size(1); f.Hkv = (int)k.size(2);
  f.q = q.data_ptr(); f.k = k.data_ptr(); f.v = v.data_ptr(); f.o = const_cast<void*>(o.data_ptr());
  f.lse = const_cast<float*>(lse.data_ptr<float>());
  f.q_tok = q.stride(1); f.k_tok = k.stride(1); f.v_tok = v.stride(1); f.o_tok = o.stride(1);
  f.q_bat = q.stride(0); f.k_bat = k.stride(0); f.v_bat = v.stride(0); f.o_bat = o.stride(0);
  f.q_head = q.stride(2); f.k_head = k.stride(2); f.v_head = v.stride(2); f.o_head = o.stride(2);
  f.window = (int)window; f.scale = (float)scale;
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && o.stride(3) == 1 && d_o.stride(3) == 1 &&
              dq.stride(3) == 1 && dk.stride(3) == 1 && dv.stride(3) == 1, "attention: head dim must be contiguous");
  d.d_o = d_o.data_ptr(); d.do_bat = d_o.stride(0); d.do_tok = d_o.stride(1); d.do_head = d_o.stride(2);
  d.dq = dq.data_ptr(); d.dq_bat = dq.stride(0); d.dq_tok = dq.stride(1); d.dq_head = dq.stride(2);
  d.dk = dk.data_ptr(); d.dk_bat = dk.stride(0); d.dk_tok = dk.stride(1); d.dk_head = dk.stride(2);
  d.dv = dv.data_ptr(); d.dv_bat = dv.stride(0); d.dv_tok = dv.stride(1); d.dv_head = dv.stride(2);
  d.delta = delta.data_ptr<float>();
  d.amax_dv = opt_scalar(amax_dv);
  NC_CHECK(nc::attention_bwd(d, status_ptr(q), cur_stream()));
  g_launches += 2;   // delta pre-pass + dK/dV kernel + dQ kernel
}

// ------------------------------------------------------------------ peer-to-peer optimizer
nc::PeerPtrs peer_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK((int)v.size() <= nc::MAX_RANKS, "too many ranks");
  nc::PeerPtrs p{};
  for (size_t i = 0; i < v.size(); ++i) p.p[i] = reinterpret_cast<void*>(v[i]);
  return p;
}
nc::AdamWArgs adamw_args(double lr, double beta1, double beta2, double eps, double wd, int64_t step) {
  nc::AdamWArgs a;
  a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2; a.eps = (float)eps; a.wd = (float)wd;
  a.bias1 = (float)(1.0 - std::pow(beta1, (double)step));
  a.bias2 = (float)(1.0 - std::pow(beta2, (double)step));
  a.grad_scale = 1.f;
  return a;
}
void p2p_barrier(const std::vector<int64_t>& pads, int64_t rank, int64_t epoch, const Tensor& like) {
  const c10::cuda::CUDAGuard guard(like.device());
  NC_CHECK(nc::p2p_barrier(peer_ptrs(pads), (int)rank, (int)pads.size(), (int)epoch, status_ptr(like), cur_stream()));
}
void p2p_adamw(const std::vector<int64_t>& grads, int64_t grad_off, int64_t rank, Tensor& p, Tensor& m, Tensor& v,
               const std::vector<int64_t>& out, int64_t out_off, bool write_local_out, double lr, double beta1,
               double beta2, double eps, double wd, int64_t step, int64_t max_ctas) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "p2p_adamw: contiguous slices");
  NC_CHECK(nc::p2p_adamw(peer_ptrs(grads), (size_t)grad_off, (int)grads.size(), (int)rank, p.data_ptr(),
                         p.scalar_type() == at::kBFloat16, m.data_ptr(), v.data_ptr(), peer_ptrs(out), (size_t)out_off,
                         write_local_out, (size_t)p.numel(), adamw_args(lr, beta1, beta2, eps, wd, step), (int)max_ctas,
                         cur_stream()));
  ++g_launches;
}
void p2p_muon_momentum(const std::vector<int64_t>& grads, int64_t grad_off, Tensor& buf, Tensor& X, Tensor& rowss,
                       Tensor& total, double mu, int64_t max_ctas) {
  const c10::cuda::CUDAGuard guard(buf.device());
  NC_CHECK(nc::p2p_muon_momentum(peer_ptrs(grads), (size_t)grad_off, (int)grads.size(), buf.data_ptr<float>(),
                                 X.data_ptr(), rowss.data_ptr<float>(), (float)mu, (int)X.size(0), (int)X.size(1),
                                 (int)X.size(2), (int)max_ctas, cur_stream()));
  // per-matrix totals of the row sums (the reduction the single-GPU path uses)
  NC_CHECK(nc::muon_total(rowss.data_ptr<float>(), total.data_ptr<float>(), (int)X.size(0), (int)X.size(1), cur_stream()));
  g_launches += 2;
}
// Statistics + parameter update of this rank's chunk; the bf16 result goes to every rank's shadow stack.
void p2p_muon_finish(Tensor& p, const Tensor& X, Tensor& second_buf, Tensor& ss, Tensor& scale,
                     const std::vector<int64_t>& out, int64_t out_off, double lr, double wd, double beta2) {
  const c10::cuda::CUDAGuard guard(X.device());
  TORCH_CHECK(p.is_contiguous() && X.is_contiguous() && p.scalar_type() == at::kFloat && X.scalar_type() == at::kBFloat16,
              "p2p_muon_finish: contiguous fp32 masters and bf16 update");
  const int k = (int)X.size(0), r = (int)X.size(1), c = (int)X.size(2);
  NC_CHECK(nc::muon_stats(X.data_ptr(), second_buf.data_ptr<float>(), ss.data_ptr<float>(), scale.data_ptr<float>(), k, r,
                          c, (float)beta2, cur_stream()));
  NC_CHECK(nc::p2p_muon_apply(p.data_ptr<float>(), X.data_ptr(), scale.data_ptr<float>(), peer_ptrs(out), (size_t)out_off,
                              (int)out.size(), k, r, c, (float)lr, (float)wd, cur_stream()));
  g_launches += 3;
}
void p2p_bcast_bf16(const Tensor& src, const std::vector<int64_t>& dst, int64_t dst_off, int64_t rank) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == at::kBFloat16, "p2p_bcast: contiguous bf16");
  NC_CHECK(nc::p2p_bcast_bf16(src.data_ptr(), peer_ptrs(dst), (size_t)dst_off, (int)dst.size(), (int)rank,
                              (size_t)src.numel(), cur_stream()));
}
void p2p_push_slices(const Tensor& src, int64_t slice, const std::vector<int64_t>& stage, int64_t dst_off, int64_t rank,
                     int64_t max_ctas) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == at::kFloat, "p2p_push_slices: contiguous fp32 gradient");
  NC_CHECK(nc::p2p_push_slices(src.data_ptr<float>(), (size_t)src.numel(), (size_t)slice, peer_ptrs(stage),
                               (size_t)dst_off, (int)rank, (int)max_ctas, cur_stream()));
  ++g_launches;
}
void p2p_copy_f32(const Tensor& src, int64_t dst_ptr) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == at::kFloat, "p2p_copy_f32: contiguous fp32 source");
  NC_CHECK(nc::p2p_copy_f32(src.data_ptr<float>(), reinterpret_cast<float*>(dst_ptr), (size_t)src.numel(), cur_stream()));
  ++g_launches;
}
void p2p_small_adamw(const std::vector<int64_t>& grads, int64_t grad_off, Tensor& p, Tensor& m, Tensor& v, double lr,
                     double beta1, double beta2, double eps, double wd, int64_t step) {
  const c10::cuda::CUDAGuard guard(p.device());
  NC_CHECK(nc::p2p_small_adamw(peer_ptrs(grads), (size_t)grad_off, (int)grads.size(), p.data_ptr<float>(),
                               m.data_ptr<float>(), v.data_ptr<float>(), (int)p.numel(),
                               adamw_args(lr, beta1, beta2, eps, wd, step), cur_stream()));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, py::arg("A"), py::arg("B"), py::arg("C"), py::arg("aux"), py::arg("a_mn"), py::arg("b_mn"),
        py::arg("alpha"), py::arg("beta"), py::arg("epi"), py::arg("bn"), py::arg("pair"), py::arg("scale_a"),
        py::arg("scale_b"), py::arg("amax_out"), py::arg("symmetric") = false);
  m.def("symmetrize", &symmetrize);
  m.def("gemm_pick_bn", &gemm_pick_bn);
  m.def("sample_next_token", &sample_next_token);
  m.def("gemv_rows", &gemv_rows, py::arg("x"), py::arg("W"), py::arg("out"), py::arg("aux"), py::arg("epi"),
        py::arg("norm_input"), py::arg("next_w") = py::none());
  m.def("gemv_rows_mix", &gemv_rows_mix, py::arg("x"), py::arg("x0"), py::arg("lam_r"), py::arg("lam_0"), py::arg("layer"),
        py::arg("W"), py::arg("out"), py::arg("xm"), py::arg("xn"), py::arg("next_w") = py::none());
  m.def("decode_embed", &decode_embed);
  m.def("decode_qkv_post", &decode_qkv_post, py::arg("qkv"), py::arg("H"), py::arg("Hkv"), py::arg("cos"), py::arg("sin"),
        py::arg("seqlens"), py::arg("xn"), py::arg("wg"), py::arg("ve"), py::arg("idx"), py::arg("k_cache"),
        py::arg("v_cache"), py::arg("table") = py::none(), py::arg("t_max") = 0);
  m.def("decode_attn", &decode_attn, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("seqlens"), py::arg("H"),
        py::arg("Hkv"), py::arg("window"), py::arg("scale"), py::arg("scratch"), py::arg("y"), py::arg("table") = py::none());
  m.def("decode_attn_scratch", &decode_attn_scratch);
  m.def("amax_bf16", &amax_bf16);
  m.def("quantize_bf16", &quantize_bf16, py::arg("x"), py::arg("amax"), py::arg("q"), py::arg("inv_scale"),
        py::arg("square") = false);
  m.def("gemm_mx", &gemm_mx);
  m.def("mx_quantize", &mx_quantize);
  m.def("read_status", &read_status);
  m.def("launch_count", &launch_count);
  m.def("mixnorm_fwd", &mixnorm_fwd);
  m.def("norm_fwd", &norm_fwd);
  m.def("normadd_bwd", &normadd_bwd);
  m.def("mixnorm_bwd", &mixnorm_bwd);
  m.def("backout_norm_fwd", &backout_norm_fwd);
  m.def("backout_norm_bwd", &backout_norm_bwd);
  m.def("qkv_post_fwd", &qkv_post_fwd);
  m.def("qkv_post_bwd", &qkv_post_bwd);
  m.def("embed_fwd", &embed_fwd);
  m.def("embed_bwd", &embed_bwd);
  m.def("cast_f32_bf16", &cast_f32_bf16);
  m.def("softcap_ce_fwd", &softcap_ce_fwd);
  m.def("softcap_ce_bwd", &softcap_ce_bwd);
  m.def("softcap_ce_bwd_fp8", &softcap_ce_bwd_fp8);
  m.def("softcap_logits", &softcap_logits);
  m.def("adamw_step", &adamw_step);
  m.def("muon_momentum", &muon_momentum);
  m.def("muon_equilibrate", &muon_equilibrate);
  m.def("muon_finish", &muon_finish);
  m.def("p2p_barrier", &p2p_barrier);
  m.def("p2p_adamw", &p2p_adamw);
  m.def("p2p_muon_momentum", &p2p_muon_momentum);
  m.def("p2p_muon_finish", &p2p_muon_finish);
  m.def("p2p_bcast_bf16", &p2p_bcast_bf16);
  m.def("p2p_small_adamw", &p2p_small_adamw);
  m.def("p2p_push_slices", &p2p_push_slices);
  m.def("p2p_copy_f32", &p2p_copy_f32);
  m.def("attn_fwd", &attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("lse"), py::arg("window"),
        py::arg("scale"), py::arg("amax_o") = py::none());
  m.def("attn_bwd", &attn_bwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("lse"), py::arg("d_o"),
        py::arg("dq"), py::arg("dk"), py::arg("dv"), py::arg("delta"), py::arg("window"), py::arg("scale"),
        py::arg("amax_dv") = py::none());
}
