// Flash attention forward for sm_100a (head dim 128, bf16, causal with optional left window).
//
// One CTA per (256-query block, head, batch): two 128-query tiles share every K/V block that is
// loaded, and their softmax phases are staggered so the tensor core always has the other tile's
// products to run. Per 128-key block j and tile x:
//   S_x  = Q_x K_j^T   tcgen05.mma, both operands K-major from TMA-loaded 128B-swizzled tiles,
//                      fp32 scores in tensor memory (128 columns per tile)
//   softmax            one warpgroup per tile, one thread per query row: the row is read from
//                      tensor memory once, the probabilities are written back over it as packed
//                      bf16 (tcgen05.st), the running sum stays in a register
//   O_x += P_x V_j     tcgen05.mma with A = P_x read from tensor memory, B = V_j MN-major straight
//                      from the [key][dim] tile (no transpose), fp32 accumulator in tensor memory
// The exponent base of a row (its "used" maximum) only moves when the true maximum has grown by
// more than 2^8; then the row's warp rescales its 32 rows of O in tensor memory. After the first
// blocks of a row this is rare, so O is normally touched by the tensor core only.
// Issue order  PV_A(j) S_A(j+1) PV_B(j) S_B(j+1) ...  gives each softmax a full product pair of the
// other tile to hide behind. Key blocks outside a tile's causal / window band are skipped per tile.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2..5
// softmax of tile A, warps 6..9 softmax of tile B. K and V are double buffered. All waits are bounded.
#include "attention.h"
#include "host_utils.cuh"
#include "ptx.cuh"

namespace nc {

namespace attn {
constexpr int BQ = 128;                          // rows of one query tile
constexpr int TILES = 2;                         // query tiles per CTA
constexpr int BKV = 128, D = 128;
constexpr int THREADS = 320;
constexpr int HALF_TILE = 128 * 64 * 2;          // one TMA box: 128 rows x 64 bf16 = 16 KB
constexpr int TILE = 2 * HALF_TILE;              // 128 x 128 bf16 = 32 KB
constexpr int KV_STAGES = 2;
constexpr int SMEM_BYTES = TILES * TILE /*Q*/ + KV_STAGES * 2 * TILE + 1024 + 256;
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_O = 256;            // + 128 * tile
constexpr float NEG_BIG = -1.0e30f;
constexpr float RESCALE_STEP = 8.f;              // log2 units the row maximum may outgrow the exponent base
}  // namespace attn

struct AttnKernelArgs {
  void* o;
  float* lse;
  float* amax_o;        // optional max |o|
  long long o_bat, o_tok, o_head;
  int Tq, Tk, H, Hkv;
  int window;           // < 0: unlimited
  float scale_log2;     // softmax scale * log2(e)
  int* status;
};

// Key blocks [lo, hi] a 128-query tile starting at query q0x needs (empty when hi < lo).
struct BlockRange { int lo, hi; };
__device__ __forceinline__ BlockRange tile_blocks(int q0x, const AttnKernelArgs& a) {
  BlockRange r;
  r.lo = 0; r.hi = -1;
  if (q0x >= a.Tq) return r;
  const int off = a.Tk - a.Tq;                   // query i sees keys <= i + off
  int hi_key = q0x + attn::BQ - 1 + off;
  if (hi_key > a.Tk - 1) hi_key = a.Tk - 1;
  r.hi = hi_key / attn::BKV;
  if (a.window >= 0) {
    const int lo_key = q0x + off - a.window;
    r.lo = lo_key > 0 ? lo_key / attn::BKV : 0;
  }
  return r;
}

__global__ void __launch_bounds__(attn::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnKernelArgs args) {
  using namespace attn;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                            // TILES tiles
  uint8_t* sK = sQ + TILES * TILE;               // KV_STAGES tiles
  uint8_t* sV = sK + KV_STAGES * TILE;           // KV_STAGES tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KV_STAGES * TILE);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                   // [2]
  uint64_t* v_full = bars + 3;                   // [2]
  uint64_t* k_empty = bars + 5;                  // [2]
  uint64_t* v_empty = bars + 7;                  // [2]
  uint64_t* s_full = bars + 9;                   // [tile]
  uint64_t* p_ready = bars + 11;                 // [tile]
  uint64_t* pv_done = bars + 13;                 // [tile]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;     // heavy (late) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (args.H / args.Hkv);
  const int q0 = qb * (TILES * BQ);
  const int off = args.Tk - args.Tq;
  const BlockRange rng[2] = {tile_blocks(q0, args), tile_blocks(q0 + BQ, args)};
  const int j_first = rng[0].lo;                                   // tile A starts no later than tile B
  const int j_last = rng[1].hi > rng[0].hi ? rng[1].hi : rng[0].hi;
  const int n_blocks = j_last - j_first + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int x = 0; x < TILES; ++x) { mbar_init(&s_full[x], 1); mbar_init(&p_ready[x], 4); mbar_init(&pv_done[x], 1); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      // rows past the end of the sequence (second tile of a ragged block) are zero-filled by TMA
      mbar_arrive_expect_tx(q_full, TILES * TILE);
#pragma unroll
      for (int x = 0; x < TILES; ++x) {
        tma_load_4d(sQ + x * TILE, &tmQ, q_full, 0, q0 + x * BQ, h, b);
        tma_load_4d(sQ + x * TILE + HALF_TILE, &tmQ, q_full, 64, q0 + x * BQ, h, b);
      }
      bool ok = true;
      for (int it = 0; it < n_blocks && ok; ++it) {
        const int s = it & 1; const uint32_t ph = (it >> 1) & 1;
        const int k0 = (j_first + it) * BKV;
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
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, false, false);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BQ, D, false, true);     // P (TMEM)    x V (MN-major)
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, ST_WAIT_FULL, 0xff);
      // Descriptors are built once; a byte offset inside the tile adds offset/16 to the address field
      // (shared memory is smaller than the field's range, so the add never carries out of it).
      const uint64_t dq[2] = {umma_desc_sw128(smem_u32(sQ), 16, 1024), umma_desc_sw128(smem_u32(sQ + TILE), 16, 1024)};
      const uint64_t dk[2] = {umma_desc_sw128(smem_u32(sK), 16, 1024), umma_desc_sw128(smem_u32(sK + TILE), 16, 1024)};
      const uint64_t dv[2] = {umma_desc_sw128(smem_u32(sV), HALF_TILE, 1024),
                              umma_desc_sw128(smem_u32(sV + TILE), HALF_TILE, 1024)};
      int n_pv[2] = {0, 0};                        // products issued per tile (barrier parities are per tile)
      auto active = [&](int x, int j) { return j >= rng[x].lo && j <= rng[x].hi; };
      auto issue_s = [&](int x, int it) -> bool {
        const int s = it & 1; const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph, abort_flag, args.status, ST_WAIT_FULL, it)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t o = static_cast<uint64_t>(((kk >> 2) * HALF_TILE + (kk & 3) * 32) >> 4);
          mma_f16(tmem_base + COL_S + x * 128, dq[x] + o, dk[s] + o, idesc_s, kk != 0);
        }
        mma_commit(&s_full[x]);
        return true;
      };
      auto issue_pv = [&](int x, int it) -> bool {
        const int s = it & 1; const uint32_t ph = (it >> 1) & 1;
        const int n = n_pv[x]++;
        if (!mbar_wait(&p_ready[x], n & 1, abort_flag, args.status, ST_WAIT_PEER, it)) return false;
        if (!mbar_wait(&v_full[s], ph, abort_flag, args.status, ST_WAIT_FULL, 0x100 + it)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // A: 16 keys = 8 packed bf16 columns of the tile's score block; B: 16 key rows of V (MN-major)
          mma_f16_ts(tmem_base + COL_O + x * 128, tmem_base + COL_S + x * 128 + kk * 8,
                     dv[s] + static_cast<uint64_t>((kk * 16 * 128) >> 4), idesc_pv, (n | kk) != 0);
        }
        mma_commit(&pv_done[x]);
        return true;
      };
      if (ok && n_blocks > 0) {
        if (active(0, j_first)) ok = issue_s(0, 0);
        if (ok && active(1, j_first)) ok = issue_s(1, 0);
        mma_commit(&k_empty[0]);
      }
      for (int it = 0; it < n_blocks && ok; ++it) {
        const int j = j_first + it;
        const bool more = it + 1 < n_blocks;
        if (active(0, j)) ok = issue_pv(0, it);
        if (ok && more && active(0, j + 1)) ok = issue_s(0, it + 1);     // overwrites P_A(j): issued after PV_A(j)
        if (ok && active(1, j)) ok = issue_pv(1, it);
        if (!ok) break;
        mma_commit(&v_empty[it & 1]);
        if (more) {
          if (active(1, j + 1)) ok = issue_s(1, it + 1);
          mma_commit(&k_empty[(it + 1) & 1]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax
    const int x = (warp - 2) >> 2;                  // query tile of this warpgroup
    const int quad = warp & 3;                      // TMEM lane quadrant this warp can access
    const int r = quad * 32 + lane;                 // query row within the tile
    const int q0x = q0 + x * BQ;
    const int qi = q0x + r;                         // query position
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_sel + COL_S + x * 128;
    const uint32_t t_o = tmem_base + lane_sel + COL_O + x * 128;
    const int hi = qi + off;                        // last visible key
    const int lo = args.window >= 0 ? hi - args.window : -(1 << 30);
    const float sc = args.scale_log2;
    float m_used = NEG_BIG, l_run = 0.f;
    int n = 0;                                      // blocks this tile has processed
    bool ok = true;
    for (int j = rng[x].lo; j <= rng[x].hi && ok; ++j, ++n) {
      const int k0 = j * BKV;
      if (!mbar_wait(&s_full[x], n & 1, abort_flag, args.status, ST_WAIT_TMEM_FULL, j)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) tmem_ld32(t_s + c * 32, reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
      tmem_wait_ld();
      const bool need_mask = (k0 + BKV - 1 > q0x + off) || (k0 + BKV > args.Tk) ||
                             (args.window >= 0 && k0 < q0x + BQ - 1 + off - args.window);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BKV; ++c) {
          const int kj = k0 + c;
          if (!(kj <= hi && kj >= lo && kj < args.Tk)) sv[c] = 0xff800000u;      // -inf
        }
      }
      float mx[4] = {__uint_as_float(sv[0]), __uint_as_float(sv[1]), __uint_as_float(sv[2]), __uint_as_float(sv[3])};
#pragma unroll
      for (int c = 4; c < BKV; c += 4) {
        mx[0] = fmaxf(mx[0], __uint_as_float(sv[c]));     mx[1] = fmaxf(mx[1], __uint_as_float(sv[c + 1]));
        mx[2] = fmaxf(mx[2], __uint_as_float(sv[c + 2])); mx[3] = fmaxf(mx[3], __uint_as_float(sv[c + 3]));
      }
      const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sc);
      // move the exponent base only when the maximum outgrew it by 2^RESCALE_STEP (always on the first block)
      if (__any_sync(0xffffffffu, m_new > m_used + RESCALE_STEP)) {
        const float alpha = exp2f(m_used - m_new);
        l_run *= alpha;
        m_used = m_new;
        if (n > 0) {
          // O of this tile is complete up to the previous block and not yet touched by this one
          if (!mbar_wait(&pv_done[x], (n - 1) & 1, abort_flag, args.status, ST_WAIT_TMEM_FULL, 0x200 + j)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(t_o + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
            tmem_st16(t_o + c * 32, reinterpret_cast<uint32_t(&)[16]>(v[0]));
            tmem_st16(t_o + c * 32 + 16, reinterpret_cast<uint32_t(&)[16]>(v[16]));
          }
        }
      }
      // probabilities, packed to bf16 over the first 64 columns of the score block
      const float neg_m = -m_used;
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[c * 32 + 2 * e]), sc, neg_m));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[c * 32 + 2 * e + 1]), sc, neg_m));
          ls[e & 3] += p0 + p1;
          pk[e] = pack_bf16(p0, p1);
        }
        tmem_st16(t_s + c * 16, pk);
      }
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[x]);
    }
    // ---------------------------------------------------------------- write-out
    if (ok && n > 0) ok = mbar_wait(&pv_done[x], (n - 1) & 1, abort_flag, args.status, ST_WAIT_TMEM_FULL, 0x300);
    tc_fence_after();
    // tcgen05.ld is warp-collective: every lane runs the loads, only the stores are predicated
    if (__all_sync(0xffffffffu, ok) && n > 0) {
      const bool row_ok = qi < args.Tq;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      float mxo = 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(args.o) + (long long)b * args.o_bat +
                            (long long)qi * args.o_tok + (long long)h * args.o_head;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(t_o + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(v[e]) * inv_l, __uint_as_float(v[e + 1]) * inv_l);
          w.y = pack_bf16(__uint_as_float(v[e + 2]) * inv_l, __uint_as_float(v[e + 3]) * inv_l);
          w.z = pack_bf16(__uint_as_float(v[e + 4]) * inv_l, __uint_as_float(v[e + 5]) * inv_l);
          w.w = pack_bf16(__uint_as_float(v[e + 6]) * inv_l, __uint_as_float(v[e + 7]) * inv_l);
          if (row_ok) *reinterpret_cast<uint4*>(orow + c * 32 + e) = w;
        }
        if (args.amax_o && row_ok) {
#pragma unroll
          for (int e = 0; e < 32; ++e) mxo = fmaxf(mxo, fabsf(__uint_as_float(v[e])));
        }
      }
      if (args.amax_o) {
        mxo *= inv_l * 1.00390625f;                   // bf16 rounding may push a stored value up by one part in 256
#pragma unroll
        for (int w = 16; w > 0; w >>= 1) mxo = fmaxf(mxo, __shfl_xor_sync(0xffffffffu, mxo, w));
        if (lane == 0 && mxo > 0.f) atomicMax(reinterpret_cast<unsigned int*>(args.amax_o), __float_as_uint(mxo));
      }
      if (row_ok && args.lse)
        args.lse[((long long)b * args.H + h) * args.Tq + qi] = (m_used + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
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
  static PerDeviceOnce configured;
  cudaError_t ce = configured.once([] {
    return cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_BYTES);
  });
  if (ce != cudaSuccess) return ce;
  CUtensorMap tmQ, tmK, tmV;
  if (!make_qkv_map(&tmQ, d.q, d.Tq, d.H, d.B, d.q_tok, d.q_head, d.q_bat)) return cudaErrorInvalidValue;
  if (!make_qkv_map(&tmK, d.k, d.Tk, d.Hkv, d.B, d.k_tok, d.k_head, d.k_bat)) return cudaErrorInvalidValue;
  if (!make_qkv_map(&tmV, d.v, d.Tk, d.Hkv, d.B, d.v_tok, d.v_head, d.v_bat)) return cudaErrorInvalidValue;
  AttnKernelArgs a;
  a.o = d.o; a.lse = d.lse; a.amax_o = d.amax_o; a.o_bat = d.o_bat; a.o_tok = d.o_tok; a.o_head = d.o_head;
  a.Tq = d.Tq; a.Tk = d.Tk; a.H = d.H; a.Hkv = d.Hkv;
  a.window = d.window;
  a.scale_log2 = d.scale * 1.4426950408889634f;
  a.status = status;
  dim3 grid((d.Tq + attn::TILES * attn::BQ - 1) / (attn::TILES * attn::BQ), d.H, d.B);
  attn_fwd_kernel<<<grid, attn::THREADS, attn::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, a);
  return cudaGetLastError();
}

}  // namespace nc
