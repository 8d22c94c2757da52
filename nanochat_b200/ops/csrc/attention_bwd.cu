// Flash attention backward for sm_100a (head dim 128, bf16, causal + optional left window).
//
// Two launches of one kernel template share a pipeline skeleton:
//
//   MODE_DKV  CTA = (128-key block, kv head, batch). Outer tiles X1 = K, X2 = V stay resident;
//             the inner loop walks 64-query blocks (Y1 = Q, Y2 = dO) of every query head that
//             shares the kv head. Scores are kept transposed (rows = keys):
//               S'  = K Q^T,  dP' = V dO^T                      (tcgen05, TMEM 2 x 64 columns, double buffered)
//               P'  = exp2(S' * c - lse_q),  dS' = P' * (dP' - delta_q)   (two threads per key row, 32 columns each)
//               dV += P' dO,  dK += dS' Q                        (A = bf16 P'/dS' in TMEM, B = Y tile MN-major)
//   MODE_DQ   CTA = (128-query block, head, batch). X1 = Q, X2 = dO resident, inner 64-key blocks
//             (Y1 = K, Y2 = V): S = Q K^T, dP = dO V^T, dS = P (dP - delta),  dQ += dS K.
//
// P' and dS' never touch shared memory: the compute threads write them as packed bf16 over the fp32
// S' / dP' columns they were computed from (tcgen05.st) and the accumulate products read their A
// operand from tensor memory. That leaves room for a four-deep ring of inner tiles, enough to cover
// the latency of the TMA loads (a stage is only released when the accumulate products that read it
// have completed).
//
// Recomputing S and dP in both launches costs 7 tile products instead of 5 but keeps every
// accumulator in TMEM (no atomics, deterministic) and every operand in its natural layout.
// delta = rowsum(dO * O) comes from a small pre-pass. All waits are bounded.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..9 =
// two compute warpgroups. Both warpgroups work on the same 128 x 64 score block, one per 32-column
// half, so the exp2 / dS arithmetic of a block takes half as long and each scheduler has two
// resident warps to overlap TMEM loads with math. Blocks that lie entirely inside the causal /
// window band skip the per-element mask.
#include "attention.h"
#include "host_utils.cuh"
#include "ptx.cuh"

#include <type_traits>

namespace nc {

namespace ab {
constexpr int BX = 128;                  // outer rows per CTA
constexpr int BY = 64;                   // inner block
constexpr int D = 128;
constexpr int THREADS = 320;
constexpr int COMPUTE_WARPS = 8;
constexpr int X_HALF = 128 * 64 * 2;     // 16 KB box of an outer tile
constexpr int X_TILE = 2 * X_HALF;       // 32 KB
constexpr int Y_HALF = 64 * 64 * 2;      // 8 KB box of an inner tile
constexpr int Y_TILE = 2 * Y_HALF;       // 16 KB
constexpr int NS = 4;                    // inner-tile ring depth
// smem: X1, X2 | NS stages x (Y1, Y2) | column vectors | barriers
constexpr int SMEM_BYTES = 2 * X_TILE + NS * 2 * Y_TILE + 1024 /*col vectors*/ + 1024 + 256;
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_DP = 128, COL_ACC1 = 256, COL_ACC2 = 384;
}  // namespace ab

// Optional timeline of one CTA (build with -DNC_ATTN_TRACE): SM clock at pipeline events of the first 32
// inner items, read back with nc_attn_trace_read(). Used to see which role the others wait for.
#ifdef NC_ATTN_TRACE
__device__ long long g_attn_trace[16 * 32];
#define NC_TRACE(ev, it) do { if (trace_on && (it) < 32) g_attn_trace[(ev) * 32 + (it)] = clock64(); } while (0)
#else
#define NC_TRACE(ev, it) do { } while (0)
#endif

struct AttnBwdArgs {
  const float* lse;      // (B, H, Tq)
  const float* delta;    // (B, H, Tq)
  void* out1;            // MODE_DKV: dV ; MODE_DQ: dQ
  void* out2;            // MODE_DKV: dK ; MODE_DQ: unused
  float* amax1;          // optional max |out1| (used for dV)
  long long o1_bat, o1_tok, o1_head, o2_bat, o2_tok, o2_head;
  int Tq, Tk, H, Hkv;
  int window;
  float scale, scale_log2;
  int* status;
};

template <bool DKV>
__global__ void __launch_bounds__(ab::THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2,
                const AttnBwdArgs args) {
  using namespace ab;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX1 = smem;
  uint8_t* sX2 = sX1 + X_TILE;
  uint8_t* sY = sX2 + X_TILE;                     // stage s: Y1 at s*2*Y_TILE, Y2 right after
  float* col_vec = reinterpret_cast<float*>(sY + NS * 2 * Y_TILE);   // [2 buffers][2 (lse, delta)][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(col_vec) + 1024);
  uint64_t* out_full = bars;
  uint64_t* in_full = bars + 1;       // [NS]
  uint64_t* in_empty = bars + 5;      // [NS]
  uint64_t* s_full = bars + 9;        // [2]
  uint64_t* p_ready = bars + 11;      // [2]
  uint64_t* done = bars + 13;
  uint64_t* cv_ready = bars + 14;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef NC_ATTN_TRACE
  const bool trace_on = DKV && blockIdx.x == 2 && blockIdx.y == 0 && blockIdx.z == 0 && (lane == 0) && (warp < 3);
#endif
  const int xb = DKV ? blockIdx.x : (gridDim.x - 1 - blockIdx.x);
  const int hx = blockIdx.y, b = blockIdx.z;       // DKV: kv head ; DQ: q head
  const int group = args.H / args.Hkv;
  const int x0 = xb * BX;
  const int off = args.Tk - args.Tq;

  // inner range [y_lo, y_hi] in 64-blocks, and the heads the inner loop covers
  int lo, hi;
  if (DKV) {
    lo = x0 - off; if (lo < 0) lo = 0;
    hi = args.window < 0 ? args.Tq - 1 : min(args.Tq - 1, x0 + BX - 1 + args.window - off);
  } else {
    lo = args.window < 0 ? 0 : max(0, x0 + off - args.window);
    hi = min(args.Tk - 1, x0 + BX - 1 + off);
  }
  const int y_lo = lo / BY;
  const int per_head = hi >= lo ? (hi / BY - y_lo + 1) : 0;
  const int n_heads_inner = DKV ? group : 1;
  const int n_items = per_head * n_heads_inner;
  const int hkv = DKV ? hx : hx / group;

  if (threadIdx.x == 0) {
    mbar_init(out_full, 1);
    for (int s = 0; s < NS; ++s) { mbar_init(&in_full[s], 1); mbar_init(&in_empty[s], 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1); mbar_init(&p_ready[s], COMPUTE_WARPS); mbar_init(&cv_ready[s], 4);
    }
    mbar_init(done, 1);
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
      tma_prefetch_desc(&tmX1); tma_prefetch_desc(&tmX2); tma_prefetch_desc(&tmY1); tma_prefetch_desc(&tmY2);
      const int head_x = DKV ? hkv : hx;
      mbar_arrive_expect_tx(out_full, 2 * X_TILE);
      tma_load_4d(sX1, &tmX1, out_full, 0, x0, head_x, b);
      tma_load_4d(sX1 + X_HALF, &tmX1, out_full, 64, x0, head_x, b);
      tma_load_4d(sX2, &tmX2, out_full, 0, x0, head_x, b);
      tma_load_4d(sX2 + X_HALF, &tmX2, out_full, 64, x0, head_x, b);
      for (int it = 0; it < n_items; ++it) {
        const int s = it % NS; const uint32_t ph = (it / NS) & 1;
        const int hi_idx = it / per_head;
        const int y0 = (y_lo + it - hi_idx * per_head) * BY;
        const int head_y = DKV ? hkv * group + hi_idx : hkv;
        if (!mbar_wait(&in_empty[s], ph ^ 1, abort_flag, args.status, ST_WAIT_EMPTY, it)) break;
        uint8_t* y1 = sY + s * 2 * Y_TILE;
        uint8_t* y2 = y1 + Y_TILE;
        NC_TRACE(7, it);
        mbar_arrive_expect_tx(&in_full[s], 2 * Y_TILE);
        tma_load_4d(y1, &tmY1, &in_full[s], 0, y0, head_y, b);
        tma_load_4d(y1 + Y_HALF, &tmY1, &in_full[s], 64, y0, head_y, b);
        tma_load_4d(y2, &tmY2, &in_full[s], 0, y0, head_y, b);
        tma_load_4d(y2 + Y_HALF, &tmY2, &in_full[s], 64, y0, head_y, b);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BX, BY, false, false);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(BX, D, false, true);
      // Descriptors are built once per tile; a byte offset inside a tile adds offset/16 to the address field
      // (shared memory is smaller than the field's range, so the add never carries out of it).
      const uint64_t dx1 = umma_desc_sw128(smem_u32(sX1), 16, 1024), dx2 = umma_desc_sw128(smem_u32(sX2), 16, 1024);
      // inner tiles of ring stage 0 viewed K-major (scores) and MN-major (accumulate); stage st adds st * stride
      const uint64_t dyk0 = umma_desc_sw128(smem_u32(sY), 16, 1024), dym0 = umma_desc_sw128(smem_u32(sY), Y_HALF, 1024);
      constexpr uint64_t STAGE_STEP = (2 * Y_TILE) >> 4, Y2_STEP = Y_TILE >> 4;
      bool ok = mbar_wait(out_full, 0, abort_flag, args.status, ST_WAIT_FULL, 0xfff);
      auto accumulate = [&](int i) -> bool {
        const int bfr = i & 1; const uint32_t ph = (i >> 1) & 1;
        const int st = i % NS;
        if (!mbar_wait(&p_ready[bfr], ph, abort_flag, args.status, ST_WAIT_PEER, i)) return false;
        NC_TRACE(1, i);
        tc_fence_after();
        const uint64_t m1 = dym0 + st * STAGE_STEP, m2 = m1 + Y2_STEP;
#pragma unroll
        for (int kk = 0; kk < BY / 16; ++kk) {
          // A: 16 reduction elements = 8 packed columns; each warpgroup wrote its 32 elements at the start of
          // its own 32-column half of the fp32 block
          const uint32_t acol = bfr * BY + (kk >> 1) * 32 + (kk & 1) * 8;
          const uint64_t bdesc1 = m1 + static_cast<uint64_t>((kk * 2048) >> 4);   // Y1 as [red 64][out 128]
          if (DKV) {
            const uint64_t bdesc2 = m2 + static_cast<uint64_t>((kk * 2048) >> 4);
            mma_f16_ts(tmem_base + COL_ACC1, tmem_base + COL_S + acol, bdesc2, idesc_acc, (i | kk) != 0);
            mma_f16_ts(tmem_base + COL_ACC2, tmem_base + COL_DP + acol, bdesc1, idesc_acc, (i | kk) != 0);
          } else {
            mma_f16_ts(tmem_base + COL_ACC1, tmem_base + COL_DP + acol, bdesc1, idesc_acc, (i | kk) != 0);
          }
        }
        mma_commit(&in_empty[st]);
        return true;
      };
      for (int it = 0; it < n_items && ok; ++it) {
        // S'/dP' buffer it&1 still holds P'/dS' of item it-2: its accumulate products were issued in the
        // previous iteration and the tensor pipe runs this thread's instructions in order
        const int s = it & 1;
        const int st = it % NS; const uint32_t ph = (it / NS) & 1;
        if (!mbar_wait(&in_full[st], ph, abort_flag, args.status, ST_WAIT_FULL, it)) { ok = false; break; }
        NC_TRACE(8, it);
        tc_fence_after();
        const uint64_t k1 = dyk0 + st * STAGE_STEP, k2 = k1 + Y2_STEP;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t xo = static_cast<uint64_t>(((kk >> 2) * X_HALF + (kk & 3) * 32) >> 4);
          const uint64_t yo = static_cast<uint64_t>(((kk >> 2) * Y_HALF + (kk & 3) * 32) >> 4);
          mma_f16(tmem_base + COL_S + s * BY, dx1 + xo, k1 + yo, idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t xo = static_cast<uint64_t>(((kk >> 2) * X_HALF + (kk & 3) * 32) >> 4);
          const uint64_t yo = static_cast<uint64_t>(((kk >> 2) * Y_HALF + (kk & 3) * 32) >> 4);
          mma_f16(tmem_base + COL_DP + s * BY, dx2 + xo, k2 + yo, idesc_s, kk != 0);
        }
        mma_commit(&s_full[s]);
        NC_TRACE(0, it);
        if (it > 0 && !accumulate(it - 1)) { ok = false; break; }
      }
      if (ok && n_items > 0) ok = accumulate(n_items - 1);
      mma_commit(done);
    }
  } else {
    // ------------------------------------------------------------------ compute
    const int quad = warp & 3;                      // TMEM lane quadrant this warp can read
    const int half = (warp - 2) >> 2;               // which 32-column half of the 64-wide block
    const int r = quad * 32 + lane;
    const int tid_c = (quad * 32 + lane);           // 0..127 inside a warpgroup
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const int xi = x0 + r;                          // DKV: key index ; DQ: query index
    float row_lse = 0.f, row_delta = 0.f;
    if (!DKV && xi < args.Tq) {
      const long long o = ((long long)b * args.H + hx) * args.Tq + xi;
      row_lse = args.lse[o] * 1.4426950408889634f;
      row_delta = args.delta[o];
    }
    bool ok = true;
    for (int it = 0; it < n_items && ok; ++it) {
      const int s = it & 1; const uint32_t ph = (it >> 1) & 1;
      const int hi_idx = it / per_head;
      const int y0 = (y_lo + it - hi_idx * per_head) * BY;
      float* cv = col_vec + s * 128;
      float col_stat = 0.f;
      if (DKV && half == 0) {
        // per-query (column) statistics of this inner block: fetched early, published to smem below
        const int hq = hkv * group + hi_idx;
        const int qi = y0 + (tid_c & 63);
        if (qi < args.Tq) {
          const long long o = ((long long)b * args.H + hq) * args.Tq + qi;
          col_stat = tid_c < 64 ? args.lse[o] * 1.4426950408889634f : args.delta[o];
        }
      }
      if (!mbar_wait(&s_full[s], ph, abort_flag, args.status, ST_WAIT_TMEM_FULL, it)) { ok = false; break; }
      NC_TRACE(2, it);
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld32(tmem_base + lane_sel + COL_S + s * BY + half * 32, sv);
      tmem_ld32(tmem_base + lane_sel + COL_DP + s * BY + half * 32, dv);
      tmem_wait_ld();
      NC_TRACE(3, it);
      // column vectors of buffer s were last read for item it-2; every compute warp finished that item before
      // its accumulate products (and therefore this item's S'/dP') could be issued
      if (DKV) {
        if (half == 0) {
          cv[tid_c] = col_stat;
          __syncwarp();
          if (lane == 0) mbar_arrive(&cv_ready[s]);
        }
        if (!mbar_wait(&cv_ready[s], ph, abort_flag, args.status, ST_WAIT_PEER, 0x400 + it)) { ok = false; break; }
      }
      NC_TRACE(4, it);
      // a block needs the element mask only if the causal diagonal, the window edge or the end of the
      // sequence passes through it
      const bool interior =
          DKV ? (x0 + BX - 1 <= y0 + off) && (args.window < 0 || y0 + BY - 1 + off - x0 <= args.window) &&
                    (x0 + BX - 1 < args.Tk) && (y0 + BY - 1 < args.Tq)
              : (y0 + BY - 1 <= x0 + off) && (args.window < 0 || x0 + BX - 1 + off - y0 <= args.window) &&
                    (y0 + BY - 1 < args.Tk) && (x0 + BX - 1 < args.Tq);
      uint32_t pp[16], dd[16];
      auto block = [&](auto masked_tag) {
        constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cbase = half * 32 + u * 8;      // first of 8 columns, within the 64-wide block
          float l8[8], d8[8];
          if (DKV) {
            const float4 la = *reinterpret_cast<const float4*>(cv + cbase);
            const float4 lb = *reinterpret_cast<const float4*>(cv + cbase + 4);
            const float4 da = *reinterpret_cast<const float4*>(cv + 64 + cbase);
            const float4 db = *reinterpret_cast<const float4*>(cv + 64 + cbase + 4);
            l8[0] = la.x; l8[1] = la.y; l8[2] = la.z; l8[3] = la.w; l8[4] = lb.x; l8[5] = lb.y; l8[6] = lb.z; l8[7] = lb.w;
            d8[0] = da.x; d8[1] = da.y; d8[2] = da.z; d8[3] = da.w; d8[4] = db.x; d8[5] = db.y; d8[6] = db.z; d8[7] = db.w;
          }
          float pv[8], dsv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int j = u * 8 + e;                // index into this thread's 32 loaded columns
            const float lse2 = DKV ? l8[e] : row_lse;
            const float dl = DKV ? d8[e] : row_delta;
            float pe = exp2f(__uint_as_float(sv[j]) * args.scale_log2 - lse2);
            if (MASKED) {
              const int yi = y0 + cbase + e;
              const int qi = DKV ? yi : xi;
              const int kj = DKV ? xi : yi;
              const bool valid = (kj <= qi + off) && (args.window < 0 || qi + off - kj <= args.window) &&
                                 (kj < args.Tk) && (qi < args.Tq);
              pe = valid ? pe : 0.f;
            }
            pv[e] = pe;
            dsv[e] = pe * (__uint_as_float(dv[j]) - dl);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (DKV) pp[u * 4 + e] = pack_bf16(pv[2 * e], pv[2 * e + 1]);
            dd[u * 4 + e] = pack_bf16(dsv[2 * e], dsv[2 * e + 1]);
          }
        }
      };
      if (interior) block(std::false_type{}); else block(std::true_type{});
      NC_TRACE(5, it);
      // packed bf16 over the first 16 of this warp's own 32 fp32 columns (already in registers)
      if (DKV) tmem_st16(tmem_base + lane_sel + COL_S + s * BY + half * 32, pp);
      tmem_st16(tmem_base + lane_sel + COL_DP + s * BY + half * 32, dd);
      tmem_wait_st();
      NC_TRACE(6, it);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[s]);
    }
    // -------------------------------------------------------------- write-out
    if (ok) ok = mbar_wait(done, 0, abort_flag, args.status, ST_WAIT_TMEM_FULL, 0x300);
    tc_fence_after();
    const int limit = DKV ? args.Tk : args.Tq;
    // tcgen05.ld is warp-collective: every lane of the warp runs the loads, only the stores are predicated
    const bool warp_ok = __all_sync(0xffffffffu, ok);
    const bool store_row_ok = xi < limit;
    if (warp_ok) {
      // DKV: warpgroup 0 writes dV, warpgroup 1 writes dK. DQ: each warpgroup writes half of the head dim.
      {
        const int which = DKV ? half : 0;
        const int c_lo = DKV ? 0 : half * (D / 64), c_hi = DKV ? D / 32 : c_lo + D / 64;
        const float mul = (DKV && which == 0) ? 1.f : args.scale;
        __nv_bfloat16* orow =
            which == 0 ? reinterpret_cast<__nv_bfloat16*>(args.out1) + (long long)b * args.o1_bat +
                             (long long)xi * args.o1_tok + (long long)hx * args.o1_head
                       : reinterpret_cast<__nv_bfloat16*>(args.out2) + (long long)b * args.o2_bat +
                             (long long)xi * args.o2_tok + (long long)hx * args.o2_head;
        const uint32_t col0 = which == 0 ? COL_ACC1 : COL_ACC2;
        const bool track = DKV && which == 0 && args.amax1 != nullptr;
        float mx1 = 0.f;
#pragma unroll 1
        for (int c = c_lo; c < c_hi; ++c) {
          uint32_t v[32];
          if (n_items > 0) {
            tmem_ld32(tmem_base + lane_sel + col0 + c * 32, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[j]) * mul, __uint_as_float(v[j + 1]) * mul);
            w.y = pack_bf16(__uint_as_float(v[j + 2]) * mul, __uint_as_float(v[j + 3]) * mul);
            w.z = pack_bf16(__uint_as_float(v[j + 4]) * mul, __uint_as_float(v[j + 5]) * mul);
            w.w = pack_bf16(__uint_as_float(v[j + 6]) * mul, __uint_as_float(v[j + 7]) * mul);
            if (store_row_ok) *reinterpret_cast<uint4*>(orow + c * 32 + j) = w;
          }
          if (track && store_row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) mx1 = fmaxf(mx1, fabsf(__uint_as_float(v[j])));
          }
        }
        if (track) {                                  // warp-uniform: every lane takes part in the shuffles
          mx1 *= mul * 1.00390625f;                   // bf16 rounding may push a stored value up by one part in 256
#pragma unroll
          for (int w = 16; w > 0; w >>= 1) mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, w));
          if (lane == 0 && mx1 > 0.f) atomicMax(reinterpret_cast<unsigned int*>(args.amax1), __float_as_uint(mx1));
        }
      }
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
    tmem_dealloc(tmem_base, ab::TMEM_COLS);
  }
}

// delta[b,h,t] = sum_d dO * O. A warp owns 32 consecutive tokens of one (b, h): a row (128 values = 256 B of each
// tensor) is read by a half-warp with 16-byte loads, eight rows' loads are in flight per warp, and the 32 sums leave as
// one 128-byte store (delta is (B, H, T), so a warp per token would scatter 4-byte writes T apart).
constexpr int DELTA_WARPS = 4;
__global__ void __launch_bounds__(DELTA_WARPS * 32)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                  long long o_bat, long long o_tok, long long o_head, long long g_bat, long long g_tok,
                  long long g_head, float* __restrict__ delta, int B, int T, int H) {
  const int lane = threadIdx.x & 31, half = lane >> 4, sub = lane & 15;
  const int t_blocks = (T + 31) / 32;
  const long long units = (long long)B * H * t_blocks;
  for (long long u = blockIdx.x * (long long)DELTA_WARPS + (threadIdx.x >> 5); u < units;
       u += gridDim.x * (long long)DELTA_WARPS) {
    const int tb = (int)(u % t_blocks);
    const long long bh = u / t_blocks;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const int t0 = tb * 32;
    const __nv_bfloat16* op = o + b * o_bat + h * o_head + sub * 8;
    const __nv_bfloat16* gp = d_o + b * g_bat + h * g_head + sub * 8;
    float mine = 0.f;
#pragma unroll
    for (int i0 = 0; i0 < 16; i0 += 4) {
      uint4 a[4], g[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = t0 + 2 * (i0 + j) + half;
        a[j] = g[j] = make_uint4(0, 0, 0, 0);
        if (t < T) {
          a[j] = *reinterpret_cast<const uint4*>(op + t * o_tok);
          g[j] = *reinterpret_cast<const uint4*>(gp + t * g_tok);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t aw[4] = {a[j].x, a[j].y, a[j].z, a[j].w}, gw[4] = {g[j].x, g[j].y, g[j].z, g[j].w};
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 x = unpack_bf16(aw[q]), y = unpack_bf16(gw[q]);
          s += x.x * y.x + x.y * y.y;
        }
#pragma unroll
        for (int w = 8; w > 0; w >>= 1) s += __shfl_xor_sync(0xffffffffu, s, w);
        const float other = __shfl_xor_sync(0xffffffffu, s, 16);
        // lower half holds the sum of token 2i, upper half of token 2i + 1; lane r keeps token t0 + r
        const int i = i0 + j;
        if (lane == 2 * i) mine = half ? other : s;
        if (lane == 2 * i + 1) mine = half ? s : other;
      }
    }
    if (t0 + lane < T) delta[((long long)b * H + h) * T + t0 + lane] = mine;
  }
}

static bool map4(CUtensorMap* m, const void* base, int T, int Hn, int B, long long tok, long long head,
                 long long bat, int box_rows) {
  uint64_t dims[4] = {128, (uint64_t)T, (uint64_t)Hn, (uint64_t)B};
  uint64_t str[3] = {(uint64_t)tok * 2, (uint64_t)head * 2, (uint64_t)bat * 2};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, str, box);
}

cudaError_t attention_bwd(const AttnBwdDesc& d, int* status, cudaStream_t stream) {
  const AttnDesc& f = d.fwd;
  if (f.D != 128 || f.H % f.Hkv != 0 || f.Tq > f.Tk) return cudaErrorInvalidValue;
  static PerDeviceOnce configured;
  cudaError_t ce = configured.once([] {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ab::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ab::SMEM_BYTES);
  });
  if (ce != cudaSuccess) return ce;
  // The tensor maps are encoded before anything is launched: the encoder rejects misaligned bases and strides,
  // so a bad layout is an error return here, not a fault in the pre-pass below.
  CUtensorMap q128, do128, k128, v128, q64, do64, k64, v64;
  bool okm = map4(&q128, f.q, f.Tq, f.H, f.B, f.q_tok, f.q_head, f.q_bat, 128) &&
             map4(&do128, d.d_o, f.Tq, f.H, f.B, d.do_tok, d.do_head, d.do_bat, 128) &&
             map4(&k128, f.k, f.Tk, f.Hkv, f.B, f.k_tok, f.k_head, f.k_bat, 128) &&
             map4(&v128, f.v, f.Tk, f.Hkv, f.B, f.v_tok, f.v_head, f.v_bat, 128) &&
             map4(&q64, f.q, f.Tq, f.H, f.B, f.q_tok, f.q_head, f.q_bat, 64) &&
             map4(&do64, d.d_o, f.Tq, f.H, f.B, d.do_tok, d.do_head, d.do_bat, 64) &&
             map4(&k64, f.k, f.Tk, f.Hkv, f.B, f.k_tok, f.k_head, f.k_bat, 64) &&
             map4(&v64, f.v, f.Tk, f.Hkv, f.B, f.v_tok, f.v_head, f.v_bat, 64);
  if (!okm) return cudaErrorInvalidValue;
  // the pre-pass reads O with 16-byte loads (dO has passed the encoder's checks above)
  if ((reinterpret_cast<uintptr_t>(f.o) & 15) || (f.o_tok & 7) || (f.o_head & 7) || (f.o_bat & 7)) return cudaErrorInvalidValue;
  {
    const long long units = (long long)f.B * f.H * ((f.Tq + 31) / 32);
    const long long blocks = (units + DELTA_WARPS - 1) / DELTA_WARPS;
    const int grid = (int)(blocks < 148 * 16 ? blocks : 148 * 16);
    attn_delta_kernel<<<grid, DELTA_WARPS * 32, 0, stream>>>((const __nv_bfloat16*)f.o, (const __nv_bfloat16*)d.d_o, f.o_bat,
                                                f.o_tok, f.o_head, d.do_bat, d.do_tok, d.do_head, d.delta, f.B,
                                                f.Tq, f.H);
  }
  AttnBwdArgs a;
  a.lse = f.lse; a.delta = d.delta;
  a.Tq = f.Tq; a.Tk = f.Tk; a.H = f.H; a.Hkv = f.Hkv; a.window = f.window;
  a.scale = f.scale; a.scale_log2 = f.scale * 1.4426950408889634f;
  a.status = status;
  // dK, dV
  a.out1 = d.dv; a.o1_bat = d.dv_bat; a.o1_tok = d.dv_tok; a.o1_head = d.dv_head;
  a.out2 = d.dk; a.o2_bat = d.dk_bat; a.o2_tok = d.dk_tok; a.o2_head = d.dk_head;
  a.amax1 = d.amax_dv;
  dim3 grid_kv((f.Tk + ab::BX - 1) / ab::BX, f.Hkv, f.B);
  attn_bwd_kernel<true><<<grid_kv, ab::THREADS, ab::SMEM_BYTES, stream>>>(k128, v128, q64, do64, a);
  // dQ
  a.out1 = d.dq; a.o1_bat = d.dq_bat; a.o1_tok = d.dq_tok; a.o1_head = d.dq_head;
  a.out2 = nullptr;
  a.amax1 = nullptr;
  dim3 grid_q((f.Tq + ab::BX - 1) / ab::BX, f.H, f.B);
  attn_bwd_kernel<false><<<grid_q, ab::THREADS, ab::SMEM_BYTES, stream>>>(q128, do128, k64, v64, a);
  return cudaGetLastError();
}

}  // namespace nc

#ifdef NC_ATTN_TRACE
extern "C" int nc_attn_trace_read(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, nc::g_attn_trace, sizeof(long long) * 16 * 32);
}
#endif
