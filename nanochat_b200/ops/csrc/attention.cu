// Flash attention forward for sm_100a (head dim 128, bf16, causal with optional left window).
//
// One CTA per (128-query block, head, batch). Per 128-key block:
//   S  = Q K^T        tcgen05.mma, both operands K-major from TMA-loaded 128B-swizzled tiles,
//                     fp32 scores in TMEM columns [0,128)
//   softmax           128 threads, one per query row: tcgen05.ld the row, running max / sum in
//                     registers (base-2 exponent), masked P written as bf16 into a swizzled
//                     shared-memory tile
//   PV = P V          tcgen05.mma, A = P (K-major), B = V read MN-major straight from the
//                     [key][dim] tile (no transpose), result in TMEM columns [128,256)
//   O  = O*alpha + PV accumulated in registers by the same 128 threads
// Key blocks entirely above the causal diagonal or entirely left of the window are never
// loaded: a query block costs ceil((window+128)/128)+1 key blocks at most.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2..5
// softmax / accumulate / store. K and V are double buffered. All waits are bounded.
#include "attention.h"
#include "host_utils.cuh"
#include "ptx.cuh"

namespace nc {

namespace attn {
constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int THREADS = 192;
constexpr int HALF_TILE = 128 * 64 * 2;          // one TMA box: 128 rows x 64 bf16 = 16 KB
constexpr int TILE = 2 * HALF_TILE;              // 128 x 128 bf16 = 32 KB
constexpr int KV_STAGES = 2;
constexpr int SMEM_BYTES = TILE /*Q*/ + TILE /*P*/ + KV_STAGES * 2 * TILE + 1024 + 256;
constexpr int TMEM_COLS = 256;
constexpr float NEG_BIG = -1.0e30f;
}  // namespace attn

struct AttnKernelArgs {
  void* o;
  float* lse;
  long long o_bat, o_tok, o_head;
  int Tq, Tk, H, Hkv;
  int window;           // < 0: unlimited
  float scale_log2;     // softmax scale * log2(e)
  int* status;
};

__global__ void __launch_bounds__(attn::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnKernelArgs args) {
  using namespace attn;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + TILE;
  uint8_t* sK = sP + TILE;                       // KV_STAGES tiles
  uint8_t* sV = sK + KV_STAGES * TILE;           // KV_STAGES tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KV_STAGES * TILE);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                   // [2]
  uint64_t* v_full = bars + 3;                   // [2]
  uint64_t* k_empty = bars + 5;                  // [2]
  uint64_t* v_empty = bars + 7;                  // [2]
  uint64_t* s_full = bars + 9;
  uint64_t* p_ready = bars + 10;
  uint64_t* pv_full = bars + 11;
  uint64_t* pv_free = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;     // heavy (late) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (args.H / args.Hkv);
  const int q0 = qb * BQ;
  const int off = args.Tk - args.Tq;             // query i sees keys <= i + off
  // key-block range for this query block
  int hi_key = q0 + BQ - 1 + off;
  if (hi_key > args.Tk - 1) hi_key = args.Tk - 1;
  const int j_hi = hi_key / BKV;
  int j_lo = 0;
  if (args.window >= 0) {
    const int lo_key = q0 + off - args.window;
    j_lo = lo_key > 0 ? lo_key / BKV : 0;
  }
  const int n_blocks = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1); mbar_init(p_ready, 4); mbar_init(pv_full, 1); mbar_init(pv_free, 4);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_PV = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(q_full, TILE);
      tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
      tma_load_4d(sQ + HALF_TILE, &tmQ, q_full, 64, q0, h, b);
      bool ok = true;
      for (int it = 0; it < n_blocks && ok; ++it) {
        const int s = it & 1; const uint32_t ph = (it >> 1) & 1;
        const int k0 = (j_lo + it) * BKV;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag, args.status, ST_WAIT_EMPTY, it)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[s], TILE);
        tma_load_4d(sK + s * TILE, &tmK, &k_full[s], 0, k0, hkv, b);
        tma_load_4d(sK + s * TILE + HALF_TILE, &tmK, &k_full[s], 64, k0, hkv, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag, args.status, ST_WAIT_EMPTY, it)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[s], TILE);
        tma_load_4d(sV + s * TILE, &tmV, &v_full[s], 0, k0, hkv, b);
        tma_load_4d(sV + s * TILE + HALF_TILE, &tmV, &v_full[s], 64, k0, hkv, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, false, false);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BQ, D, false, true);     // P (K-major) x V (MN-major)
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, ST_WAIT_FULL, 0xff);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      for (int it = 0; it < n_blocks && ok; ++it) {
        const int s = it & 1; const uint32_t ph = (it >> 1) & 1;
        const uint32_t k_addr = smem_u32(sK + s * TILE), v_addr = smem_u32(sV + s * TILE);
        if (!mbar_wait(&k_full[s], ph, abort_flag, args.status, ST_WAIT_FULL, it)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = (kk >> 2) * HALF_TILE + (kk & 3) * 32;
          mma_f16(tmem_S, umma_desc_sw128(q_addr + o, 16, 1024), umma_desc_sw128(k_addr + o, 16, 1024), idesc_s,
                  kk != 0);
        }
        mma_commit(s_full);
        mma_commit(&k_empty[s]);
        if (!mbar_wait(p_ready, it & 1, abort_flag, args.status, ST_WAIT_PEER, it)) { ok = false; break; }
        if (!mbar_wait(&v_full[s], ph, abort_flag, args.status, ST_WAIT_FULL, it)) { ok = false; break; }
        if (!mbar_wait(pv_free, (it & 1) ^ 1, abort_flag, args.status, ST_WAIT_TMEM_EMPTY, it)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t po = (kk >> 2) * HALF_TILE + (kk & 3) * 32;     // P: keys contiguous (K-major)
          const uint32_t vo = kk * (16 * 128);                          // V: 16 key rows per step (MN-major)
          mma_f16(tmem_PV, umma_desc_sw128(p_addr + po, 16, 1024), umma_desc_sw128(v_addr + vo, HALF_TILE, 1024),
                  idesc_pv, kk != 0);
        }
        mma_commit(pv_full);
        mma_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------------------------ softmax / accumulate / store
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // query row within the block
    const int qi = q0 + r;                          // query position
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    float o_acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o_acc[d] = 0.f;
    float m_run = NEG_BIG, l_run = 0.f;
    bool ok = true;
    for (int it = 0; it < n_blocks && ok; ++it) {
      const int k0 = (j_lo + it) * BKV;
      if (!mbar_wait(s_full, it & 1, abort_flag, args.status, ST_WAIT_TMEM_FULL, it)) { ok = false; break; }
      tc_fence_after();
      const int hi = qi + off;                      // last visible key
      const int lo = args.window >= 0 ? hi - args.window : -(1 << 30);
      const bool need_mask = (k0 + BKV - 1 > q0 + off) || (k0 + BKV > args.Tk) ||
                             (args.window >= 0 && k0 < q0 + BQ - 1 + off - args.window);
      // pass 1: row maximum
      float m_blk = NEG_BIG;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_S + lane_sel + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int kj = k0 + c * 32 + j;
          const bool valid = !need_mask || (kj <= hi && kj >= lo && kj < args.Tk);
          const float sv = __uint_as_float(v[j]) * args.scale_log2;
          m_blk = valid ? fmaxf(m_blk, sv) : m_blk;
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      const float alpha = exp2f(m_run - m_new);
      // pass 2: probabilities -> swizzled bf16 tile, row sum
      float l_blk = 0.f;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_S + lane_sel + c * 32, v);
        tmem_wait_ld();
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int kj = k0 + c * 32 + j;
          const bool v0 = !need_mask || (kj <= hi && kj >= lo && kj < args.Tk);
          const bool v1 = !need_mask || (kj + 1 <= hi && kj + 1 >= lo && kj + 1 < args.Tk);
          float p0 = v0 ? exp2f(__uint_as_float(v[j]) * args.scale_log2 - m_new) : 0.f;
          float p1 = v1 ? exp2f(__uint_as_float(v[j + 1]) * args.scale_log2 - m_new) : 0.f;
          const uint32_t pk = pack_bf16(p0, p1);
          float2 back = unpack_bf16(pk);          // sum what the tensor core will actually see
          l_blk += back.x + back.y;
          packed[j >> 1] = pk;
        }
        // 32 keys = 4 units of 16 bytes; unit index within the 64-key half tile, XOR-swizzled by row
        uint8_t* half = sP + (c >> 1) * HALF_TILE + r * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int unit = ((c & 1) * 4 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(half + unit * 16) =
              make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
        }
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      tc_fence_before();
      fence_proxy_async_smem();                     // make the P tile visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      // accumulate O
      if (!mbar_wait(pv_full, it & 1, abort_flag, args.status, ST_WAIT_TMEM_FULL, 0x100 + it)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_PV + lane_sel + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) o_acc[c * 32 + j] = o_acc[c * 32 + j] * alpha + __uint_as_float(v[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pv_free);
    }
    if (ok && qi < args.Tq) {
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(args.o) + (long long)b * args.o_bat +
                            (long long)qi * args.o_tok + (long long)h * args.o_head;
#pragma unroll
      for (int d = 0; d < D; d += 8) {
        uint4 w;
        w.x = pack_bf16(o_acc[d] * inv_l, o_acc[d + 1] * inv_l);
        w.y = pack_bf16(o_acc[d + 2] * inv_l, o_acc[d + 3] * inv_l);
        w.z = pack_bf16(o_acc[d + 4] * inv_l, o_acc[d + 5] * inv_l);
        w.w = pack_bf16(o_acc[d + 6] * inv_l, o_acc[d + 7] * inv_l);
        *reinterpret_cast<uint4*>(orow + d) = w;
      }
      if (args.lse)
        args.lse[((long long)b * args.H + h) * args.Tq + qi] = (m_run + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  __syncthreads();
  if (*abort_flag) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, attn::TMEM_COLS);
  }
}

static bool make_qkv_map(CUtensorMap* m, const void* base, int T, int Hn, int B, long long tok, long long head,
                         long long bat) {
  // dims innermost-first: (d, t, h, b)
  uint64_t dims[4] = {128, (uint64_t)T, (uint64_t)Hn, (uint64_t)B};
  uint64_t str[3] = {(uint64_t)tok * 2, (uint64_t)head * 2, (uint64_t)bat * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, str, box);
}

cudaError_t attention_fwd(const AttnDesc& d, int* status, cudaStream_t stream) {
  if (d.D != 128 || d.H % d.Hkv != 0 || d.Tq > d.Tk) return cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  CUtensorMap tmQ, tmK, tmV;
  if (!make_qkv_map(&tmQ, d.q, d.Tq, d.H, d.B, d.q_tok, d.q_head, d.q_bat)) return cudaErrorInvalidValue;
  if (!make_qkv_map(&tmK, d.k, d.Tk, d.Hkv, d.B, d.k_tok, d.k_head, d.k_bat)) return cudaErrorInvalidValue;
  if (!make_qkv_map(&tmV, d.v, d.Tk, d.Hkv, d.B, d.v_tok, d.v_head, d.v_bat)) return cudaErrorInvalidValue;
  AttnKernelArgs a;
  a.o = d.o; a.lse = d.lse; a.o_bat = d.o_bat; a.o_tok = d.o_tok; a.o_head = d.o_head;
  a.Tq = d.Tq; a.Tk = d.Tk; a.H = d.H; a.Hkv = d.Hkv;
  a.window = d.window;
  a.scale_log2 = d.scale * 1.4426950408889634f;
  a.status = status;
  dim3 grid((d.Tq + attn::BQ - 1) / attn::BQ, d.H, d.B);
  attn_fwd_kernel<<<grid, attn::THREADS, attn::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, a);
  return cudaGetLastError();
}

}  // namespace nc
