// bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma
// (cta_group::1, 128 x BN x 16 per instruction) -> fp32 accumulators in TMEM ->
// tcgen05.ld epilogue. One persistent CTA per SM walks a grouped tile order; two
// TMEM accumulator stages let the epilogue of tile i overlap the main loop of
// tile i+1.
//
//   C[b] (M x N) = epi( alpha * A[b] * B[b]^T , aux[b] )
//
// Operand storage is described per operand ("K-major" = reduction dim contiguous,
// "MN-major" = output dim contiguous), which covers the three GEMMs of a linear
// layer without any transposed copies:
//   forward  y  = x  W^T : A = x  (K-major),   B = W  (K-major)
//   dgrad    dx = dy W   : A = dy (K-major),   B = W  (MN-major)
//   wgrad    dW = dy^T x : A = dy (MN-major),  B = x  (MN-major), fp32 accumulate
// and the Newton-Schulz products of the Muon optimizer (X X^T, A A, B X, X^T X).
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer
// (one elected lane), warps 2..9 = epilogue (a warp may read the TMEM lane quadrant
// warp_id % 4; the two warps of a quadrant take one half of the tile's columns each). All waits are bounded (ptx.cuh); a failed wait raises the CTA abort
// flag, records a status word and the kernel drains and exits normally.
#include "gemm.h"
#include "host_utils.cuh"
#include "ptx.cuh"

#include <stdlib.h>

namespace nc {

constexpr int BM = 128;
constexpr int GEMM_THREADS = 320;        // producer warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int ROW_BYTES = 128;   // one swizzle row: 64 bf16 or 128 fp8 values along the contiguous dim

struct GemmKernelArgs {
  int M, N, K, batch;
  void* C;
  long long ldc, bsc;
  const void* aux;
  long long ldaux, bsaux;
  float alpha, beta;
  const float* scale_a;     // optional device scalars multiplied into alpha (fp8 de-quantisation)
  const float* scale_b;
  float* amax_out;          // optional: max |C| over everything this launch stores (atomic, fp32 bits)
  int epi;
  int c_f32;
  int f32_staged;           // fp32 output through the staging tile (whole 128-byte lines) instead of per-row pieces
  int c_tma;                // bf16 output leaves the staging tile as TMA stores (the kernel's third tensor map covers C)
  int m_blocks, n_blocks, group_m;
  int tiles_per_batch;      // m_blocks * n_blocks, or the tiles on and above the diagonal of a symmetric output
  int symmetric;            // C = C^T by construction (X X^T, A A): tiles below the diagonal are skipped, the caller mirrors
  uint32_t idesc;
  int* status;
};

constexpr int next_pow2_cols(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : 256; }

// FP8 = operands are 1-byte (e4m3 / e5m2, kind::f8f6f4), else bf16 (kind::f16). A k-block is always one
// 128-byte swizzle row deep along K for K-major operands, and BK rows of 128 bytes for MN-major ones.
template <int BN, bool A_MN, bool B_MN, bool FP8>
struct Cfg {
  static constexpr int ELT = FP8 ? 1 : 2;
  static constexpr int BK = ROW_BYTES / ELT;            // elements of K per k-block (64 bf16 / 128 fp8)
  static constexpr int UMMA_K = 32 / ELT;               // K per tcgen05.mma (16 bf16 / 32 fp8)
  static constexpr int MN_CHUNK = ROW_BYTES / ELT;      // MN elements per MN-major TMA box
  static constexpr int CHUNK_BYTES = BK * ROW_BYTES;    // one MN-major box: BK k-rows x 128 B
  static constexpr int A_CHUNKS = BM / MN_CHUNK;        // 2 (bf16) / 1 (fp8)
  static constexpr int B_CHUNKS = (BN + MN_CHUNK - 1) / MN_CHUNK;
  static constexpr int A_BYTES = BM * ROW_BYTES;        // 16 KB either way
  static constexpr int B_ROWS_ALLOC = (BN + 127) / 128 * 128;
  static constexpr int B_BYTES = B_ROWS_ALLOC * ROW_BYTES;
  static constexpr int B_TX = B_MN ? B_CHUNKS * CHUNK_BYTES : BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = 8 * 32 * 128;   // staging tiles of the eight epilogue warps
  static constexpr int MAX_STAGES = (227 * 1024 - 2048 - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int ACC_STRIDE = next_pow2_cols(BN);
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/ + EPI_BYTES;
  static_assert(!B_MN || B_CHUNKS * CHUNK_BYTES <= B_BYTES, "MN-major B boxes must fit the stage");
};

__device__ __forceinline__ void tile_coords(int t, const GemmKernelArgs& a, int& b, int& mb, int& nb) {
  int per_batch = a.tiles_per_batch;
  b = t / per_batch;
  int r = t - b * per_batch;
  if (a.symmetric) {          // square tiles, row by row over the upper triangle: (0,0..T-1), (1,1..T-1), ...
    int row_len = a.n_blocks;
    mb = 0;
    while (r >= row_len) { r -= row_len; ++mb; --row_len; }
    nb = mb + r;
    return;
  }
  int group_tiles = a.group_m * a.n_blocks;
  int g = r / group_tiles;
  int first_m = g * a.group_m;
  int gm = min(a.group_m, a.m_blocks - first_m);
  int in_g = r - g * group_tiles;
  mb = first_m + in_g % gm;
  nb = in_g / gm;
}

// Epilogue of one accumulator tile for one thread: its row of 128 x BN fp32 values comes out of tensor memory
// 16 columns at a time, goes through the fused epilogue and is stored as bf16 or fp32.
template <int BN>
__device__ __forceinline__ void store_tile_row(const GemmKernelArgs& args, uint32_t taddr, int b, int row, int n0,
                                               float alpha, float beta, float& amax, int c_begin, int c_end) {
  const bool row_ok = row < args.M;
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
    uint32_t r[16];
    tmem_ld16(taddr + c * 16, r);
    tmem_wait_ld();
    const int col = n0 + c * 16;
    if (row_ok && col < args.N) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) * alpha;
      if (args.c_f32) {
        float* crow = reinterpret_cast<float*>(args.C) + b * args.bsc + static_cast<long long>(row) * args.ldc + col;
        const float* xrow = args.aux ? reinterpret_cast<const float*>(args.aux) + b * args.bsaux +
                                           static_cast<long long>(row) * args.ldaux + col
                                     : nullptr;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          if (col + q4 * 4 + 4 <= args.N) {
            float4 o = make_float4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
            if (xrow) {
              float4 x = *reinterpret_cast<const float4*>(xrow + q4 * 4);
              o.x += beta * x.x; o.y += beta * x.y; o.z += beta * x.z; o.w += beta * x.w;
            }
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w))));
            *reinterpret_cast<float4*>(crow + q4 * 4) = o;
          }
        }
      } else {
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(args.C) + b * args.bsc +
                              static_cast<long long>(row) * args.ldc + col;
        const __nv_bfloat16* xrow = args.aux ? reinterpret_cast<const __nv_bfloat16*>(args.aux) + b * args.bsaux +
                                                   static_cast<long long>(row) * args.ldaux + col
                                             : nullptr;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (col + h * 8 + 8 <= args.N) {
            float* vv = v + h * 8;
            if (args.epi == EPI_RELU2) {
#pragma unroll
              for (int j = 0; j < 8; ++j) { float tpos = fmaxf(vv[j], 0.f); vv[j] = tpos * tpos; }
            } else if (args.epi == EPI_RELU) {
#pragma unroll
              for (int j = 0; j < 8; ++j) vv[j] = fmaxf(vv[j], 0.f);
            } else if (xrow) {
              uint4 xa = *reinterpret_cast<const uint4*>(xrow + h * 8);
              const uint32_t xs[4] = {xa.x, xa.y, xa.z, xa.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16(xs[j]);
                if (args.epi == EPI_MUL2SQRT) {
                  vv[2 * j] *= 2.f * sqrtf(f.x);
                  vv[2 * j + 1] *= 2.f * sqrtf(f.y);
                } else if (args.epi == EPI_MULAUX) {
                  vv[2 * j] *= f.x;
                  vv[2 * j + 1] *= f.y;
                } else {
                  vv[2 * j] += beta * f.x;
                  vv[2 * j + 1] += beta * f.y;
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vv[j]));
            uint4 o;
            o.x = pack_bf16(vv[0], vv[1]); o.y = pack_bf16(vv[2], vv[3]);
            o.z = pack_bf16(vv[4], vv[5]); o.w = pack_bf16(vv[6], vv[7]);
            *reinterpret_cast<uint4*>(crow + h * 8) = o;
          }
        }
      }
    }
  }
}

// bf16 epilogue through a per-warp staging tile in shared memory. A thread owns one accumulator row, so storing it
// directly makes every warp-wide store touch 32 different rows (32 partial sectors per instruction), and for short
// reductions that store traffic, not the tensor core, sets the tile time. Here the warp converts 64 columns of its 32
// rows at a time into a 32 x 128 B tile (16-byte units XOR-swizzled by row, so the row-wise writes and the
// 4-rows-per-instruction reads are both conflict free) and writes it out as whole 128-byte lines. The auxiliary operand
// (residual, relu^2 derivative input) comes in the same way, through the same tile.
constexpr int EPI_STAGE_BYTES = 32 * 128;          // per epilogue warp

// The auxiliary loads run one group ahead of their use: the 32 x 128 B of the NEXT group (of this tile, or the first group
// of the warp's next tile) are requested into registers before the current group is converted, so their DRAM latency
// passes under the tensor-memory reads, the conversion and the stores instead of in front of them. With a short reduction
// (K = 1664) the epilogue sets the tile time, and a load waited for at the head of every group more than doubled it.
struct AuxAhead {
  uint4 v[8];
};

struct TileAt {
  int b, row0, n0;
  bool valid;
};

__device__ __forceinline__ bool aux_bf16_used(const GemmKernelArgs& args) {
  return args.aux != nullptr && !args.c_f32 && args.epi != EPI_RELU2 && args.epi != EPI_RELU;
}

__device__ __forceinline__ void aux_request(const GemmKernelArgs& args, AuxAhead& ahead, const TileAt& at, int g, int c_end,
                                            int lane) {
  const __nv_bfloat16* xbase = reinterpret_cast<const __nv_bfloat16*>(args.aux) + at.b * args.bsaux;
  const int sub_r = lane >> 3, unit = lane & 7;
  const int nch = min(4, c_end - g);
  const int col = at.n0 + g * 16 + unit * 8;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + sub_r;
    ahead.v[it] = make_uint4(0, 0, 0, 0);
    if (at.row0 + r < args.M && unit < nch * 2 && col + 8 <= args.N)
      ahead.v[it] = *reinterpret_cast<const uint4*>(xbase + static_cast<long long>(at.row0 + r) * args.ldaux + col);
  }
}

// One line of the next tile's auxiliary operand per lane goes to L2 ahead of time (the warp's 32 rows x its columns).
__device__ __forceinline__ void aux_prefetch_l2(const GemmKernelArgs& args, const TileAt& at, int c_begin, int c_end, int lane) {
  const int col = at.n0 + c_begin * 16;
  const int cols = min((c_end - c_begin) * 16, args.N - col);
  if (at.valid && at.row0 + lane < args.M && cols >= 8) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(args.aux) + at.b * args.bsaux +
                             static_cast<long long>(at.row0 + lane) * args.ldaux + col;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(static_cast<uint32_t>((cols & ~7) * 2)) : "memory");
  }
}

template <int BN, bool AHEAD>
__device__ __forceinline__ void store_tile_bf16_staged(const GemmKernelArgs& args, uint32_t taddr, int b, int row0, int n0,
                                                       float alpha, float beta, float& amax, int c_begin, int c_end,
                                                       uint8_t* stage, int lane, AuxAhead& ahead, const TileAt& next,
                                                       const CUtensorMap* tmC) {
  __nv_bfloat16* cbase = reinterpret_cast<__nv_bfloat16*>(args.C) + b * args.bsc;
  const __nv_bfloat16* xbase = args.aux ? reinterpret_cast<const __nv_bfloat16*>(args.aux) + b * args.bsaux : nullptr;
  const bool use_aux = aux_bf16_used(args);
  const int sub_r = lane >> 3, unit = lane & 7;     // coalesced phase: 4 rows x 8 units (16 B) per instruction
#pragma unroll 1
  for (int g = c_begin; g < c_end; g += 4) {
    const int nch = min(4, c_end - g);              // 16-column chunks in this group
    const int col0 = n0 + g * 16;
    if (tmC) {                                      // the previous group's TMA store has read the tile
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
    }
    if (use_aux) {
      if constexpr (AHEAD) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + sub_r;
          *reinterpret_cast<uint4*>(stage + r * 128 + ((unit ^ (r & 7)) << 4)) = ahead.v[it];
        }
        __syncwarp();
        if (g + 4 < c_end) aux_request(args, ahead, TileAt{b, row0, n0, true}, g + 4, c_end, lane);
        else if (next.valid) aux_request(args, ahead, next, c_begin, c_end, lane);
      } else {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + sub_r;
          const int col = col0 + unit * 8;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (row0 + r < args.M && unit < nch * 2 && col + 8 <= args.N)
            v = *reinterpret_cast<const uint4*>(xbase + static_cast<long long>(row0 + r) * args.ldaux + col);
          *reinterpret_cast<uint4*>(stage + r * 128 + ((unit ^ (r & 7)) << 4)) = v;
        }
        __syncwarp();
      }
    }
    // Accumulator columns come out of tensor memory 64 at a time; with loads in flight for the next group only 32 at a
    // time, so that the registers holding those loads are not spilled (a spill waits for the load it was meant to hide).
    constexpr int BATCH = AHEAD ? 2 : 4;
#pragma unroll 1
    for (int c0 = 0; c0 < 4; c0 += BATCH) {
    uint32_t acc[BATCH][16];
#pragma unroll
    for (int ci = 0; ci < BATCH; ++ci)
      if (c0 + ci < nch) tmem_ld16(taddr + (g + c0 + ci) * 16, acc[ci]);
    tmem_wait_ld();
#pragma unroll
    for (int ci = 0; ci < BATCH; ++ci) {
      const int cc = c0 + ci;
      if (cc < nch) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float vv[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) vv[j] = __uint_as_float(acc[ci][h * 8 + j]) * alpha;
          uint8_t* slot = stage + lane * 128 + (((cc * 2 + h) ^ (lane & 7)) << 4);
          if (args.epi == EPI_RELU2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float tpos = fmaxf(vv[j], 0.f); vv[j] = tpos * tpos; }
          } else if (args.epi == EPI_RELU) {
#pragma unroll
            for (int j = 0; j < 8; ++j) vv[j] = fmaxf(vv[j], 0.f);
          } else if (use_aux) {
            const uint4 xa = *reinterpret_cast<const uint4*>(slot);
            const uint32_t xs[4] = {xa.x, xa.y, xa.z, xa.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16(xs[j]);
              if (args.epi == EPI_MUL2SQRT) {
                vv[2 * j] *= 2.f * sqrtf(f.x);
                vv[2 * j + 1] *= 2.f * sqrtf(f.y);
              } else if (args.epi == EPI_MULAUX) {
                vv[2 * j] *= f.x;
                vv[2 * j + 1] *= f.y;
              } else {
                vv[2 * j] += beta * f.x;
                vv[2 * j + 1] += beta * f.y;
              }
            }
          }
          if (row0 + lane < args.M && col0 + (cc * 2 + h) * 8 + 8 <= args.N) {
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vv[j]));
          }
          *reinterpret_cast<uint4*>(slot) = make_uint4(pack_bf16(vv[0], vv[1]), pack_bf16(vv[2], vv[3]),
                                                       pack_bf16(vv[4], vv[5]), pack_bf16(vv[6], vv[7]));
        }
      }
    }
    }
    if (tmC && nch == 4) {
      // The tile's layout (16-byte units XOR-ed with the row index) is the 128-byte TMA swizzle: one lane hands all 4 KB to
      // the copy engine, which clips rows beyond M and columns beyond N; the warp goes on to the next group meanwhile.
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { tma_store_3d(tmC, stage, col0, row0, b); tma_store_commit(); }
      continue;
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + sub_r;
      const int col = col0 + unit * 8;
      if (row0 + r < args.M && unit < nch * 2 && col + 8 <= args.N)
        *reinterpret_cast<uint4*>(cbase + static_cast<long long>(row0 + r) * args.ldc + col) =
            *reinterpret_cast<const uint4*>(stage + r * 128 + ((unit ^ (r & 7)) << 4));
    }
    __syncwarp();                                   // the tile is reused by the next group
  }
}

// fp32 epilogue through the same per-warp staging tile: 32 columns (128 B of fp32) of the warp's 32 rows per pass, written
// out as whole 128-byte lines. Weight gradients are the fp32 outputs; on several GPUs the last micro-batch writes them
// into another rank's memory over NVLink, where a warp-wide store of 32 scattered 16-byte pieces (one per row) costs a
// packet each while a 128-byte line travels as one. The auxiliary operand (the gradient accumulated so far) is read
// the same way.
template <int BN>
__device__ __forceinline__ void store_tile_f32_staged(const GemmKernelArgs& args, uint32_t taddr, int b, int row0, int n0,
                                                      float alpha, float beta, float& amax, int c_begin, int c_end,
                                                      uint8_t* stage, int lane) {
  float* cbase = reinterpret_cast<float*>(args.C) + b * args.bsc;
  const float* xbase = args.aux ? reinterpret_cast<const float*>(args.aux) + b * args.bsaux : nullptr;
  const int sub_r = lane >> 3, unit = lane & 7;     // coalesced phase: 4 rows x 8 units (16 B = 4 floats) per instruction
#pragma unroll 1
  for (int g = c_begin; g < c_end; g += 2) {
    const int nch = min(2, c_end - g);              // 16-column chunks in this pass
    const int col0 = n0 + g * 16;
    if (xbase) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + sub_r;
        const int col = col0 + unit * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < args.M && unit < nch * 4 && col + 4 <= args.N)
          v = *reinterpret_cast<const float4*>(xbase + static_cast<long long>(row0 + r) * args.ldaux + col);
        *reinterpret_cast<float4*>(stage + r * 128 + ((unit ^ (r & 7)) << 4)) = v;
      }
      __syncwarp();
    }
    uint32_t acc[2][16];
#pragma unroll
    for (int cc = 0; cc < 2; ++cc)
      if (cc < nch) tmem_ld16(taddr + (g + cc) * 16, acc[cc]);
    tmem_wait_ld();
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      if (cc < nch) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint8_t* slot = stage + lane * 128 + (((cc * 4 + q) ^ (lane & 7)) << 4);
          float4 o = make_float4(__uint_as_float(acc[cc][q * 4]) * alpha, __uint_as_float(acc[cc][q * 4 + 1]) * alpha,
                                 __uint_as_float(acc[cc][q * 4 + 2]) * alpha, __uint_as_float(acc[cc][q * 4 + 3]) * alpha);
          if (xbase) {
            const float4 x = *reinterpret_cast<const float4*>(slot);
            o.x += beta * x.x; o.y += beta * x.y; o.z += beta * x.z; o.w += beta * x.w;
          }
          if (row0 + lane < args.M && col0 + (cc * 4 + q) * 4 + 4 <= args.N)
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w))));
          *reinterpret_cast<float4*>(slot) = o;
        }
      }
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + sub_r;
      const int col = col0 + unit * 4;
      if (row0 + r < args.M && unit < nch * 4 && col + 4 <= args.N)
        *reinterpret_cast<float4*>(cbase + static_cast<long long>(row0 + r) * args.ldc + col) =
            *reinterpret_cast<const float4*>(stage + r * 128 + ((unit ^ (r & 7)) << 4));
    }
    __syncwarp();                                   // the tile is reused by the next pass
  }
}

template <int BN, bool A_MN, bool B_MN, bool FP8, bool AHEAD = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const GemmKernelArgs args) {
  using C = Cfg<BN, A_MN, B_MN, FP8>;
  constexpr int BK = C::BK;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* epi_stage = smem + C::STAGES * C::STAGE_BYTES;            // 8 x 4 KB, 1024-byte aligned (TMA swizzle atom)
  uint64_t* full = reinterpret_cast<uint64_t*>(epi_stage + C::EPI_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (args.K + BK - 1) / BK;
  const int total_tiles = args.tiles_per_batch * args.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], EPI_WARPS); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); if (args.c_tma) tma_prefetch_desc(&tmC); }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, mb, nb; tile_coords(t, args, b, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, args.status, ST_WAIT_EMPTY, t)) { ok = false; break; }
          uint8_t* sA = tiles + stage * C::STAGE_BYTES;
          uint8_t* sB = sA + C::A_BYTES;
          mbar_arrive_expect_tx(&full[stage], C::A_BYTES + C::B_TX);
          const int k0 = kb * BK;
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < C::A_CHUNKS; ++j)
              tma_load_3d(sA + j * C::CHUNK_BYTES, &tmA, &full[stage], m0 + C::MN_CHUNK * j, k0, b);
          } else {
            tma_load_3d(sA, &tmA, &full[stage], k0, m0, b);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < C::B_CHUNKS; ++j)
              tma_load_3d(sB + j * C::CHUNK_BYTES, &tmB, &full[stage], n0 + C::MN_CHUNK * j, k0, b);
          } else {
            tma_load_3d(sB, &tmB, &full[stage], k0, n0, b);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = args.idesc;
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, args.status, ST_WAIT_TMEM_EMPTY, t)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, args.status, ST_WAIT_FULL, t)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / C::UMMA_K; ++k) {
            // one instruction consumes 32 bytes of K: 32 B along a K-major row, or UMMA_K rows of 128 B
            const uint64_t a_desc = A_MN ? umma_desc_sw128(a_addr + k * (C::UMMA_K * ROW_BYTES), C::CHUNK_BYTES, 1024)
                                         : umma_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t b_desc = B_MN ? umma_desc_sw128(b_addr + k * (C::UMMA_K * ROW_BYTES), C::CHUNK_BYTES, 1024)
                                         : umma_desc_sw128(b_addr + k * 32, 16, 1024);
            if (FP8) mma_f8(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0);
            else     mma_f16(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0);
          }
          mma_commit(&empty[stage]);   // frees the smem stage once these MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&acc_full[acc]);    // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;
    constexpr int CHUNKS = BN / 16, SPLIT = (CHUNKS + 1) / 2;
    // with TMA stores a warp's columns are split into whole 64-column groups where possible (a partial group is stored by hand)
    const int split = (args.c_tma && CHUNKS > 8) ? (SPLIT + 3) / 4 * 4 : SPLIT;
    const int c_begin = (warp - 2) < 4 ? 0 : split, c_end = (warp - 2) < 4 ? split : CHUNKS;
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    float amax = 0.f;
    float alpha = args.alpha;
    if (args.scale_a) alpha *= __ldg(args.scale_a);
    if (args.scale_b) alpha *= __ldg(args.scale_b);
    const float beta = args.beta;
    const bool use_aux = AHEAD && aux_bf16_used(args);     // auxiliary loads run ahead of their use (see AuxAhead)
    AuxAhead ahead;
    auto tile_at = [&](int t) {
      TileAt at{0, 0, 0, t < total_tiles};
      if (at.valid) {
        int tb, tmb, tnb; tile_coords(t, args, tb, tmb, tnb);
        at.b = tb; at.row0 = tmb * BM + quad * 32; at.n0 = tnb * BN;
      }
      return at;
    };
    if (use_aux && blockIdx.x < total_tiles) aux_request(args, ahead, tile_at(blockIdx.x), c_begin, c_end, lane);
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int b, mb, nb; tile_coords(t, args, b, mb, nb);
      const TileAt next = use_aux ? tile_at(t + gridDim.x) : TileAt{0, 0, 0, false};
      if (use_aux) aux_prefetch_l2(args, next, c_begin, c_end, lane);
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, args.status, ST_WAIT_TMEM_FULL, t)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * BM + quad * 32 + lane;
      const int n0 = nb * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * C::ACC_STRIDE;
      if (args.c_f32 && args.f32_staged && args.epi == EPI_LINEAR)
        store_tile_f32_staged<BN>(args, taddr, b, mb * BM + quad * 32, n0, alpha, beta, amax, c_begin, c_end,
                                  epi_stage + (warp - 2) * EPI_STAGE_BYTES, lane);
      else if (args.c_f32)
        store_tile_row<BN>(args, taddr, b, row, n0, alpha, beta, amax, c_begin, c_end);
      else
        store_tile_bf16_staged<BN, AHEAD>(args, taddr, b, mb * BM + quad * 32, n0, alpha, beta, amax, c_begin, c_end,
                                          epi_stage + (warp - 2) * EPI_STAGE_BYTES, lane, ahead, next,
                                          args.c_tma ? &tmC : nullptr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (args.c_tma && lane == 0) tma_store_wait<0>();     // the warp's last stores have left shared memory and landed
    if (args.amax_out) {
      // non-negative floats order like their bit patterns
#pragma unroll
      for (int w = 16; w > 0; w >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, w));
      if (lane == 0 && amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(args.amax_out), __float_as_uint(amax));
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ block-scaled (MXFP8) kernel
// kind::mxf8f6f4.block_scale: A (M x K) and B (N x K) K-major 8-bit floats, one E8M0 scale per 32 elements of K.
// The pipeline is the single-CTA one above plus the scale factors: each k-block (128 elements of K = four MMAs of
// K = 32) brings one 512-byte chunk of A scales (128 rows x 4 K blocks) and BN/128 chunks of B scales into shared memory
// with untiled bulk copies on the stage's barrier; the MMA thread moves them into tensor memory with tcgen05.cp (32 rows
// x 16 bytes, replicated over the four lane quadrants: lane l holds the scales of rows l % 32 + 32 g in column g, one
// byte per K block) and issues the four MMAs with the scale-factor id of their K block. tcgen05.cp and tcgen05.mma of
// one thread execute in order, so the same scale columns are reused by every k-block. Tensor memory: accumulators in
// columns [0, 256) (two stages of 128 columns, or one of 256), scales from column 256 on.
template <int BN>
struct MxCfg {
  static_assert(BN == 128 || BN == 256, "MXFP8 tiles are 128 x 128 or 128 x 256");
  static constexpr int BK = 128;
  static constexpr int A_BYTES = BM * ROW_BYTES;
  static constexpr int B_BYTES = BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SF_CHUNK = 512;
  static constexpr int SFB_CHUNKS = BN / 128;
  static constexpr int SF_STAGE = SF_CHUNK * (1 + SFB_CHUNKS);
  static constexpr int EPI_BYTES = 8 * 32 * 128;
  static constexpr int MAX_STAGES = (227 * 1024 - 2048 - EPI_BYTES) / (STAGE_BYTES + SF_STAGE);
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int ACC_STAGES = BN == 256 ? 1 : 2;
  static constexpr int ACC_STRIDE = BN;
  static constexpr int SF_COL = 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_BYTES = STAGES * (STAGE_BYTES + SF_STAGE) + 1024 /*align*/ + 512 /*barriers*/ + EPI_BYTES;
};

struct MxKernelScales {
  const unsigned char* sfa;
  const unsigned char* sfb;
  int k_blocks;        // K / 128
  int sfb_row_blocks;  // ceil(N / 128): chunks beyond it do not exist and are not fetched
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmKernelArgs args, const MxKernelScales sf) {
  using C = MxCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_stage = smem + C::STAGES * C::STAGE_BYTES + 512;      // 8 x 4 KB, 128-byte aligned
  uint8_t* sf_smem = epi_stage + C::EPI_BYTES;                       // STAGES x (A chunk | B chunks), 512-byte chunks

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = sf.k_blocks;
  const int total_tiles = args.tiles_per_batch * args.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], EPI_WARPS); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer: operand tiles + scale chunks
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, mb, nb; tile_coords(t, args, b, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        int sfb_have = sf.sfb_row_blocks - nb * C::SFB_CHUNKS;          // B scale chunks that exist for this tile
        sfb_have = sfb_have < 0 ? 0 : (sfb_have > C::SFB_CHUNKS ? C::SFB_CHUNKS : sfb_have);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, args.status, ST_WAIT_EMPTY, t)) { ok = false; break; }
          uint8_t* sA = tiles + stage * C::STAGE_BYTES;
          uint8_t* sB = sA + C::A_BYTES;
          uint8_t* sS = sf_smem + stage * C::SF_STAGE;
          mbar_arrive_expect_tx(&full[stage], C::A_BYTES + C::B_BYTES + C::SF_CHUNK * (1 + sfb_have));
          tma_load_3d(sA, &tmA, &full[stage], kb * C::BK, m0, b);
          tma_load_3d(sB, &tmB, &full[stage], kb * C::BK, n0, b);
          bulk_load_1d(sS, sf.sfa + (static_cast<size_t>(mb) * num_kb + kb) * C::SF_CHUNK, C::SF_CHUNK, &full[stage]);
          for (int j = 0; j < sfb_have; ++j)
            bulk_load_1d(sS + C::SF_CHUNK * (1 + j),
                         sf.sfb + (static_cast<size_t>(nb * C::SFB_CHUNKS + j) * num_kb + kb) * C::SF_CHUNK, C::SF_CHUNK,
                         &full[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t acc_phase = 0;
      const uint32_t sfa_tmem = tmem_base + C::SF_COL, sfb_tmem = tmem_base + C::SF_COL + 4;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, args.status, ST_WAIT_TMEM_EMPTY, t)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, args.status, ST_WAIT_FULL, t)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
          const uint32_t s_addr = smem_u32(sf_smem + stage * C::SF_STAGE);
          tmem_cp_32x128b_warpx4(sfa_tmem, umma_desc_noswizzle(s_addr, 128, 128));
#pragma unroll
          for (int j = 0; j < C::SFB_CHUNKS; ++j)
            tmem_cp_32x128b_warpx4(sfb_tmem + 4 * j, umma_desc_noswizzle(s_addr + C::SF_CHUNK * (1 + j), 128, 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t a_desc = umma_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t b_desc = umma_desc_sw128(b_addr + k * 32, 16, 1024);
            const uint32_t idesc = args.idesc | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4);
            mma_mxf8(d_tmem, a_desc, b_desc, idesc, sfa_tmem, sfb_tmem, (kb | k) != 0);
          }
          mma_commit(&empty[stage]);   // frees the stage (tiles and scale chunks) once the copies and MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&acc_full[acc]);
        if (++acc == C::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;
    constexpr int CHUNKS = BN / 16, SPLIT = (CHUNKS + 1) / 2;
    const int c_begin = (warp - 2) < 4 ? 0 : SPLIT, c_end = (warp - 2) < 4 ? SPLIT : CHUNKS;
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    float amax = 0.f;
    const float alpha = args.alpha, beta = args.beta;
    AuxAhead ahead;                                         // this kernel reads its auxiliary operand in place
    const TileAt next{0, 0, 0, false};
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int b, mb, nb; tile_coords(t, args, b, mb, nb);
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, args.status, ST_WAIT_TMEM_FULL, t)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * BM + quad * 32 + lane;
      const int n0 = nb * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * C::ACC_STRIDE;
      if (args.c_f32 && args.f32_staged && args.epi == EPI_LINEAR)
        store_tile_f32_staged<BN>(args, taddr, b, mb * BM + quad * 32, n0, alpha, beta, amax, c_begin, c_end,
                                  epi_stage + (warp - 2) * EPI_STAGE_BYTES, lane);
      else if (args.c_f32)
        store_tile_row<BN>(args, taddr, b, row, n0, alpha, beta, amax, c_begin, c_end);
      else
        store_tile_bf16_staged<BN, false>(args, taddr, b, mb * BM + quad * 32, n0, alpha, beta, amax, c_begin, c_end,
                                          epi_stage + (warp - 2) * EPI_STAGE_BYTES, lane, ahead, next, nullptr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == C::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
    if (args.amax_out) {
#pragma unroll
      for (int w = 16; w > 0; w >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, w));
      if (lane == 0 && amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(args.amax_out), __float_as_uint(amax));
    }
  }

  __syncthreads();
  if (*abort_flag) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ CTA-pair kernel
// Same pipeline with cta_group::2: a cluster of two CTAs computes one 256 x BN tile. Each CTA loads its
// own 128 rows of A and its own half (BN/2 columns) of B, so a k-block costs each SM 16 KB + BN/2 * 128 B
// of shared-memory fill instead of 16 KB + BN * 128 B, and each tensor core reads half of B from its
// partner. With one CTA per tile the fill plus the operand reads exceed what shared memory can deliver
// while the tensor core runs; the pair brings the two into balance.
//
// Only the even CTA ("leader") issues MMAs. Barriers: full[s] lives in the leader and counts the bytes of
// all four copies (the partner's TMA signals it through its cluster address); empty[s] and acc_full[a]
// exist in both CTAs and the leader's MMA thread commits to each of them; acc_empty[a] lives in the
// leader and collects the arrivals of the sixteen epilogue warps of the pair.
template <int BN, bool A_MN, bool B_MN, bool FP8>
struct PairCfg {
  using Base = Cfg<BN, A_MN, B_MN, FP8>;
  static constexpr int BK = Base::BK;
  static constexpr int UMMA_K = Base::UMMA_K;
  static constexpr int MN_CHUNK = Base::MN_CHUNK;
  static constexpr int CHUNK_BYTES = Base::CHUNK_BYTES;
  static constexpr int A_CHUNKS = Base::A_CHUNKS;
  static constexpr int BNH = BN / 2;                                   // B columns held by one CTA
  static constexpr int B_CHUNKS = (BNH + MN_CHUNK - 1) / MN_CHUNK;
  static constexpr int A_BYTES = BM * ROW_BYTES;
  static constexpr int B_TX = B_MN ? B_CHUNKS * CHUNK_BYTES : BNH * ROW_BYTES;
  static constexpr int B_BYTES = (B_TX + 1023) / 1024 * 1024;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = Base::EPI_BYTES;
  static constexpr int MAX_STAGES = (227 * 1024 - 2048 - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int ACC_STRIDE = next_pow2_cols(BN);
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/ + EPI_BYTES;
  static_assert(BN % 32 == 0 || BN == 208, "pair tiles: N/2 must stay a multiple of 8");
};

template <int BN, bool A_MN, bool B_MN, bool FP8, bool AHEAD = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmKernelArgs args) {
  using C = PairCfg<BN, A_MN, B_MN, FP8>;
  constexpr int BK = C::BK;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* epi_stage = smem + C::STAGES * C::STAGE_BYTES;            // 8 x 4 KB, 1024-byte aligned (TMA swizzle atom)
  uint64_t* full = reinterpret_cast<uint64_t*>(epi_stage + C::EPI_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader, 1 = partner
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int num_kb = (args.K + BK - 1) / BK;
  const int total_tiles = args.tiles_per_batch * args.batch;   // m_blocks counts 256-row blocks

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 2 * EPI_WARPS); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); if (args.c_tma) tma_prefetch_desc(&tmC); }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, C::TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  cluster_sync_all();                               // both CTAs' barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += n_pairs) {
        int b, mb, nb; tile_coords(t, args, b, mb, nb);
        const int m0 = mb * (2 * BM) + rank * BM;
        const int n0 = nb * BN + rank * C::BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, args.status, ST_WAIT_EMPTY, t)) { ok = false; break; }
          uint8_t* sA = tiles + stage * C::STAGE_BYTES;
          uint8_t* sB = sA + C::A_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_arrive_expect_tx(&full[stage], 2 * (C::A_BYTES + C::B_TX));
          const int k0 = kb * BK;
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < C::A_CHUNKS; ++j)
              tma_load_3d_pair(sA + j * C::CHUNK_BYTES, &tmA, bar, m0 + C::MN_CHUNK * j, k0, b);
          } else {
            tma_load_3d_pair(sA, &tmA, bar, k0, m0, b);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < C::B_CHUNKS; ++j)
              tma_load_3d_pair(sB + j * C::CHUNK_BYTES, &tmB, bar, n0 + C::MN_CHUNK * j, k0, b);
          } else {
            tma_load_3d_pair(sB, &tmB, bar, k0, n0, b);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = args.idesc;
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t acc_phase = 0;
      for (int t = pair; t < total_tiles && ok; t += n_pairs) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, args.status, ST_WAIT_TMEM_EMPTY, t)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, args.status, ST_WAIT_FULL, t)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
          const uint64_t a0 = A_MN ? umma_desc_sw128(a_addr, C::CHUNK_BYTES, 1024) : umma_desc_sw128(a_addr, 16, 1024);
          const uint64_t b0 = B_MN ? umma_desc_sw128(b_addr, C::CHUNK_BYTES, 1024) : umma_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / C::UMMA_K; ++k) {
            // one instruction consumes 32 bytes of K: 32 B along a K-major row, or UMMA_K rows of 128 B
            const uint64_t ao = static_cast<uint64_t>((A_MN ? k * (C::UMMA_K * ROW_BYTES) : k * 32) >> 4);
            const uint64_t bo = static_cast<uint64_t>((B_MN ? k * (C::UMMA_K * ROW_BYTES) : k * 32) >> 4);
            mma_pair<FP8>(d_tmem, a0 + ao, b0 + bo, idesc, (kb | k) != 0);
          }
          // frees the stage in both CTAs once these MMAs have read it
          mma_commit_pair(smem_u32(&empty[stage]));
          mma_commit_pair(map_to_cta(smem_u32(&empty[stage]), 1));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit_pair(smem_u32(&acc_full[acc]));
        mma_commit_pair(map_to_cta(smem_u32(&acc_full[acc]), 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int quad = warp & 3;
    constexpr int CHUNKS = BN / 16, SPLIT = (CHUNKS + 1) / 2;
    // with TMA stores a warp's columns are split into whole 64-column groups where possible (a partial group is stored by hand)
    const int split = (args.c_tma && CHUNKS > 8) ? (SPLIT + 3) / 4 * 4 : SPLIT;
    const int c_begin = (warp - 2) < 4 ? 0 : split, c_end = (warp - 2) < 4 ? split : CHUNKS;
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    float amax = 0.f;
    float alpha = args.alpha;
    if (args.scale_a) alpha *= __ldg(args.scale_a);
    if (args.scale_b) alpha *= __ldg(args.scale_b);
    const float beta = args.beta;
    const bool use_aux = AHEAD && aux_bf16_used(args);
    AuxAhead ahead;
    auto tile_at = [&](int t) {
      TileAt at{0, 0, 0, t < total_tiles};
      if (at.valid) {
        int tb, tmb, tnb; tile_coords(t, args, tb, tmb, tnb);
        at.b = tb; at.row0 = tmb * (2 * BM) + rank * BM + quad * 32; at.n0 = tnb * BN;
      }
      return at;
    };
    if (use_aux && pair < total_tiles) aux_request(args, ahead, tile_at(pair), c_begin, c_end, lane);
    for (int t = pair; t < total_tiles && ok; t += n_pairs) {
      int b, mb, nb; tile_coords(t, args, b, mb, nb);
      const TileAt next = use_aux ? tile_at(t + n_pairs) : TileAt{0, 0, 0, false};
      if (use_aux) aux_prefetch_l2(args, next, c_begin, c_end, lane);
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, args.status, ST_WAIT_TMEM_FULL, t)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * (2 * BM) + rank * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * C::ACC_STRIDE;
      if (args.c_f32 && args.f32_staged && args.epi == EPI_LINEAR)
        store_tile_f32_staged<BN>(args, taddr, b, mb * (2 * BM) + rank * BM + quad * 32, nb * BN, alpha, beta, amax,
                                  c_begin, c_end, epi_stage + (warp - 2) * EPI_STAGE_BYTES, lane);
      else if (args.c_f32)
        store_tile_row<BN>(args, taddr, b, row, nb * BN, alpha, beta, amax, c_begin, c_end);
      else
        store_tile_bf16_staged<BN, AHEAD>(args, taddr, b, mb * (2 * BM) + rank * BM + quad * 32, nb * BN, alpha, beta,
                                          amax, c_begin, c_end, epi_stage + (warp - 2) * EPI_STAGE_BYTES, lane, ahead, next,
                                          args.c_tma ? &tmC : nullptr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (args.c_tma && lane == 0) tma_store_wait<0>();     // the warp's last stores have left shared memory and landed
    if (args.amax_out) {
#pragma unroll
      for (int w = 16; w > 0; w >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, w));
      if (lane == 0 && amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(args.amax_out), __float_as_uint(amax));
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();       // the partner may still signal this CTA's barriers or read its operands until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------- host

// M-blocks per group of the tile order (tiles of one group run back to back so their B tiles stay in L2);
// NANOCHAT_GEMM_GROUP_M overrides the default for tuning.
static int group_m_override(int dflt) {
  static const int env = [] { const char* e = getenv("NANOCHAT_GEMM_GROUP_M"); return e ? atoi(e) : 0; }();
  return env > 0 ? env : dflt;
}

// NANOCHAT_F32_EPILOGUE=direct selects the per-row fp32 stores (A/B measurements); default: staged.
static int f32_staged_default() {
  static const int v = [] {
    const char* e = getenv("NANOCHAT_F32_EPILOGUE");
    return (e && e[0] == 'd') ? 0 : 1;
  }();
  return v;
}

// Tensor map over a bf16 output for the epilogue's TMA stores: boxes of 32 rows x 64 columns (one warp's staging tile).
// Returns false, and leaves a placeholder in *tm, where the output cannot be stored that way (fp32, unaligned base or
// pitch, narrower than a box); the kernel then writes it with ordinary stores.
static bool make_c_tmap(const GemmDesc& d, const CUtensorMap& placeholder, CUtensorMap* tm) {
  static const bool enabled = [] { const char* e = getenv("NANOCHAT_GEMM_TMA_STORE"); return !e || atoi(e) != 0; }();
  *tm = placeholder;
  if (!enabled || d.c_f32 || d.N < 64 || d.M < 32) return false;
  if ((reinterpret_cast<uintptr_t>(d.C) & 15) || (d.ldc & 7) || (d.batch > 1 && (d.bsc & 7))) return false;
  uint64_t dims[3] = {static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.M), static_cast<uint64_t>(d.batch)};
  uint64_t str[2] = {static_cast<uint64_t>(d.ldc) * 2,
                     d.batch > 1 ? static_cast<uint64_t>(d.bsc) * 2 : static_cast<uint64_t>(d.ldc) * 2 * dims[1]};
  uint32_t box[3] = {64, 32, 1};
  return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d.C, dims, str, box);
}

// bf16 output with an auxiliary operand that the epilogue combines with the product (not relu^2, which needs none)
static bool aux_ahead_wanted(const GemmDesc& d) {
  return d.aux != nullptr && !d.c_f32 && d.epi != EPI_RELU2 && d.epi != EPI_RELU;
}

template <int BN, bool A_MN, bool B_MN, bool FP8, bool AHEAD = false>
static cudaError_t launch_cfg(const GemmDesc& d, int* status, cudaStream_t stream) {
  using C = Cfg<BN, A_MN, B_MN, FP8>;
  constexpr int BK = C::BK;
  constexpr int ELT = C::ELT;
  static PerDeviceOnce configured;
  auto kern = gemm_kernel<BN, A_MN, B_MN, FP8, AHEAD>;
  cudaError_t ce = configured.once(
      [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES); });
  if (ce != cudaSuccess) return ce;
  const CUtensorMapDataType dt = FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA, tmB;
  const uint64_t batch = static_cast<uint64_t>(d.batch);
  {
    uint64_t dims[3], str[2]; uint32_t box[3];
    if (A_MN) { dims[0] = d.M; dims[1] = d.K; box[0] = C::MN_CHUNK; box[1] = BK; }
    else      { dims[0] = d.K; dims[1] = d.M; box[0] = BK; box[1] = BM; }
    dims[2] = batch; box[2] = 1;
    str[0] = static_cast<uint64_t>(d.lda) * ELT;
    str[1] = d.batch > 1 ? static_cast<uint64_t>(d.bsa) * ELT : str[0] * dims[1];
    if (!make_tmap(&tmA, dt, 3, d.A, dims, str, box)) return cudaErrorInvalidValue;
  }
  {
    uint64_t dims[3], str[2]; uint32_t box[3];
    if (B_MN) { dims[0] = d.N; dims[1] = d.K; box[0] = C::MN_CHUNK; box[1] = BK; }
    else      { dims[0] = d.K; dims[1] = d.N; box[0] = BK; box[1] = BN; }
    dims[2] = batch; box[2] = 1;
    str[0] = static_cast<uint64_t>(d.ldb) * ELT;
    str[1] = d.batch > 1 ? static_cast<uint64_t>(d.bsb) * ELT : str[0] * dims[1];
    if (!make_tmap(&tmB, dt, 3, d.B, dims, str, box)) return cudaErrorInvalidValue;
  }
  GemmKernelArgs a;
  a.M = d.M; a.N = d.N; a.K = d.K; a.batch = d.batch;
  a.C = d.C; a.ldc = d.ldc; a.bsc = d.bsc;
  a.aux = d.aux; a.ldaux = d.ldaux; a.bsaux = d.bsaux;
  a.alpha = d.alpha; a.beta = d.beta; a.epi = d.epi; a.c_f32 = d.c_f32; a.f32_staged = f32_staged_default();
  CUtensorMap tmC;
  a.c_tma = make_c_tmap(d, tmA, &tmC);
  a.scale_a = d.scale_a; a.scale_b = d.scale_b; a.amax_out = d.amax_out;
  a.m_blocks = (d.M + BM - 1) / BM;
  a.n_blocks = (d.N + BN - 1) / BN;
  a.group_m = group_m_override(16);
  a.symmetric = d.symmetric && BN == BM && d.M == d.N;          // square tiles only; otherwise every tile is computed
  a.tiles_per_batch = a.symmetric ? a.n_blocks * (a.n_blocks + 1) / 2 : a.m_blocks * a.n_blocks;
  a.idesc = FP8 ? umma_idesc_f8(BM, BN, A_MN, B_MN, d.a_e5m2, d.b_e5m2) : umma_idesc_bf16(BM, BN, A_MN, B_MN);
  a.status = status;
  const long long tiles = 1ll * a.tiles_per_batch * d.batch;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  kern<<<grid, GEMM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, tmC, a);
  return cudaGetLastError();
}

template <bool A_MN, bool B_MN, bool FP8>
static cudaError_t launch_bn(int bn, const GemmDesc& d, int* status, cudaStream_t s) {
  // forward and activation-gradient layouts with a bf16 auxiliary operand (residual add, the MLP's relu^2 derivative)
  // have kernels of their own, which request that operand ahead of its use
  if constexpr (!A_MN) {
    if (aux_ahead_wanted(d) && bn == 256) return launch_cfg<256, A_MN, B_MN, FP8, true>(d, status, s);
    if (aux_ahead_wanted(d) && bn == 208) return launch_cfg<208, A_MN, B_MN, FP8, true>(d, status, s);
    if (aux_ahead_wanted(d) && bn == 128) return launch_cfg<128, A_MN, B_MN, FP8, true>(d, status, s);
  }
  switch (bn) {
    case 256: return launch_cfg<256, A_MN, B_MN, FP8>(d, status, s);
    case 208: return launch_cfg<208, A_MN, B_MN, FP8>(d, status, s);
    case 128: return launch_cfg<128, A_MN, B_MN, FP8>(d, status, s);
    case 64:  return launch_cfg<64, A_MN, B_MN, FP8>(d, status, s);
    case 32:  return launch_cfg<32, A_MN, B_MN, FP8>(d, status, s);
    default:  return cudaErrorInvalidValue;
  }
}

template <int BN, bool A_MN, bool B_MN, bool FP8, bool AHEAD = false>
static cudaError_t launch_pair_cfg(const GemmDesc& d, int* status, cudaStream_t stream) {
  using C = PairCfg<BN, A_MN, B_MN, FP8>;
  constexpr int BK = C::BK;
  constexpr int ELT = Cfg<BN, A_MN, B_MN, FP8>::ELT;
  static PerDeviceOnce configured;
  auto kern = gemm_pair_kernel<BN, A_MN, B_MN, FP8, AHEAD>;
  cudaError_t ce = configured.once(
      [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES); });
  if (ce != cudaSuccess) return ce;
  const CUtensorMapDataType dt = FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA, tmB;
  const uint64_t batch = static_cast<uint64_t>(d.batch);
  {
    uint64_t dims[3], str[2]; uint32_t box[3];
    if (A_MN) { dims[0] = d.M; dims[1] = d.K; box[0] = C::MN_CHUNK; box[1] = BK; }
    else      { dims[0] = d.K; dims[1] = d.M; box[0] = BK; box[1] = BM; }
    dims[2] = batch; box[2] = 1;
    str[0] = static_cast<uint64_t>(d.lda) * ELT;
    str[1] = d.batch > 1 ? static_cast<uint64_t>(d.bsa) * ELT : str[0] * dims[1];
    if (!make_tmap(&tmA, dt, 3, d.A, dims, str, box)) return cudaErrorInvalidValue;
  }
  {
    uint64_t dims[3], str[2]; uint32_t box[3];
    if (B_MN) { dims[0] = d.N; dims[1] = d.K; box[0] = C::MN_CHUNK; box[1] = BK; }
    else      { dims[0] = d.K; dims[1] = d.N; box[0] = BK; box[1] = C::BNH; }      // each CTA loads half of the columns
    dims[2] = batch; box[2] = 1;
    str[0] = static_cast<uint64_t>(d.ldb) * ELT;
    str[1] = d.batch > 1 ? static_cast<uint64_t>(d.bsb) * ELT : str[0] * dims[1];
    if (!make_tmap(&tmB, dt, 3, d.B, dims, str, box)) return cudaErrorInvalidValue;
  }
  GemmKernelArgs a;
  a.M = d.M; a.N = d.N; a.K = d.K; a.batch = d.batch;
  a.C = d.C; a.ldc = d.ldc; a.bsc = d.bsc;
  a.aux = d.aux; a.ldaux = d.ldaux; a.bsaux = d.bsaux;
  a.alpha = d.alpha; a.beta = d.beta; a.epi = d.epi; a.c_f32 = d.c_f32; a.f32_staged = f32_staged_default();
  CUtensorMap tmC;
  a.c_tma = make_c_tmap(d, tmA, &tmC);
  a.scale_a = d.scale_a; a.scale_b = d.scale_b; a.amax_out = d.amax_out;
  a.m_blocks = (d.M + 2 * BM - 1) / (2 * BM);
  a.n_blocks = (d.N + BN - 1) / BN;
  a.group_m = group_m_override(8);
  a.symmetric = d.symmetric && BN == 2 * BM && d.M == d.N;      // 256 x 256 tiles only
  a.tiles_per_batch = a.symmetric ? a.n_blocks * (a.n_blocks + 1) / 2 : a.m_blocks * a.n_blocks;
  a.idesc = FP8 ? umma_idesc_f8(2 * BM, BN, A_MN, B_MN, d.a_e5m2, d.b_e5m2) : umma_idesc_bf16(2 * BM, BN, A_MN, B_MN);
  a.status = status;
  const long long tiles = 1ll * a.tiles_per_batch * d.batch;
  const int max_pairs = sm_count() / 2;
  const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, a);
}

template <bool A_MN, bool B_MN, bool FP8>
static cudaError_t launch_pair_bn(int bn, const GemmDesc& d, int* status, cudaStream_t s) {
  if constexpr (!A_MN) {
    if (aux_ahead_wanted(d) && bn == 256) return launch_pair_cfg<256, A_MN, B_MN, FP8, true>(d, status, s);
    if (aux_ahead_wanted(d) && bn == 208) return launch_pair_cfg<208, A_MN, B_MN, FP8, true>(d, status, s);
    if (aux_ahead_wanted(d) && bn == 128) return launch_pair_cfg<128, A_MN, B_MN, FP8, true>(d, status, s);
  }
  switch (bn) {
    case 256: return launch_pair_cfg<256, A_MN, B_MN, FP8>(d, status, s);
    case 208: return launch_pair_cfg<208, A_MN, B_MN, FP8>(d, status, s);
    case 128: return launch_pair_cfg<128, A_MN, B_MN, FP8>(d, status, s);
    default:  return cudaErrorInvalidValue;
  }
}

template <bool FP8>
static cudaError_t launch_major(int bn, bool pair, const GemmDesc& d, int* status, cudaStream_t stream) {
  if (pair) {
    if (d.a_mn && d.b_mn) return launch_pair_bn<true, true, FP8>(bn, d, status, stream);
    if (!d.a_mn && d.b_mn) return launch_pair_bn<false, true, FP8>(bn, d, status, stream);
    if (!d.a_mn && !d.b_mn) return launch_pair_bn<false, false, FP8>(bn, d, status, stream);
    return launch_pair_bn<true, false, FP8>(bn, d, status, stream);
  }
  if (d.a_mn && d.b_mn) return launch_bn<true, true, FP8>(bn, d, status, stream);
  if (!d.a_mn && d.b_mn) return launch_bn<false, true, FP8>(bn, d, status, stream);
  if (!d.a_mn && !d.b_mn) return launch_bn<false, false, FP8>(bn, d, status, stream);
  return launch_bn<true, false, FP8>(bn, d, status, stream);
}

int gemm_pick_bn(int M, int N, int batch) {
  // maximise (useful columns / padded columns) x (tiles / tiles rounded up to whole waves) x tile efficiency
  static const int cand[5] = {256, 208, 128, 64, 32};
  static const double eff[5] = {1.0, 0.98, 0.86, 0.62, 0.36};
  const int sms = sm_count();
  const long long mb = (M + BM - 1) / BM;
  double best = -1; int pick = 128;
  for (int i = 0; i < 5; ++i) {
    const int bn = cand[i];
    const long long nb = (N + bn - 1) / bn;
    const long long tiles = mb * nb * batch;
    const long long waves = (tiles + sms - 1) / sms;
    const double score = eff[i] * (double(N) / double(nb * bn)) * (double(tiles) / double(waves * sms));
    if (score > best + 1e-9) { best = score; pick = bn; }
  }
  return pick;
}

// Tile plan: N tile and kernel flavour. Scores are (relative tile efficiency) x (useful fraction of the padded
// tile grid) x (fill of the last wave); the efficiencies are measured rates of the d26 layer shapes relative to
// the single-CTA 128 x 256 tile. The CTA-pair kernel needs at least two 256-row blocks to be worth a cluster.
struct GemmPlan { int bn; bool pair; };
static bool best_is_invalid(const GemmPlan& p, const GemmDesc& d) {
  if (d.bn > 0 && p.bn != d.bn) return true;                  // the requested tile has no kernel of the requested flavour
  return p.pair && p.bn != 256 && p.bn != 208 && p.bn != 128;
}
static GemmPlan gemm_plan(const GemmDesc& d, bool fp8) {
  static const int env_pair = [] { const char* e = getenv("NANOCHAT_GEMM_PAIR"); return e ? atoi(e) : 1; }();
  const int sms = sm_count();
  auto score = [&](int bn, bool pair, double eff) {
    const long long rows = pair ? 2 * BM : BM;
    const long long mb = (d.M + rows - 1) / rows, nb = (d.N + bn - 1) / bn;
    const long long tiles = mb * nb * d.batch;
    const long long slots = pair ? sms / 2 : sms;
    const long long waves = (tiles + slots - 1) / slots;
    return eff * (double(d.N) / double(nb * bn)) * (double(d.M) / double(mb * rows)) *
           (double(tiles) / double(waves * slots));
  };
  GemmPlan best{128, false};
  double best_score = -1;
  const bool pair_ok = d.pair > 0 || (d.pair < 0 && env_pair > 0 && d.M > 2 * BM);
  const bool single_ok = d.pair <= 0;
  if (d.symmetric && d.M == d.N && d.bn == 0) return pair_ok ? GemmPlan{256, true} : GemmPlan{128, false};   // square tiles
  static const int cand[5] = {256, 208, 128, 64, 32};
  static const double eff1[5] = {1.0, 0.98, 0.86, 0.62, 0.36};
  static const double eff2[3] = {1.14, 1.08, 0.95};
  for (int i = 0; i < 5; ++i) {
    if (d.bn > 0 && cand[i] != d.bn) continue;
    if (single_ok) {
      const double sc = score(cand[i], false, eff1[i]);
      if (sc > best_score + 1e-9) { best_score = sc; best = {cand[i], false}; }
    }
    if (pair_ok && i < 3) {
      // fp8, MN-major B: the partner's half of a 208-wide tile would start a TMA copy off a 16-byte boundary
      if (fp8 && d.b_mn && cand[i] == 208) continue;
      // 8-bit operands halve the math time per byte fetched, which is where the pair's smaller shared-memory
      // traffic counts most (measured on the wgrad shapes: 2.3-2.5 vs 1.8 PFLOP/s)
      const double sc = score(cand[i], true, eff2[i] * (fp8 ? 1.2 : 1.0));
      if (sc > best_score + 1e-9) { best_score = sc; best = {cand[i], true}; }
    }
  }
  return best;
}

// Upper triangle -> lower triangle, 32 x 32 blocks transposed through shared memory. Block (bi, bj) with bj > bi is read
// from rows bi, columns bj and written to rows bj, columns bi; diagonal blocks mirror inside themselves.
__global__ void __launch_bounds__(256)
symmetrize_bf16_kernel(__nv_bfloat16* __restrict__ C, int n, long long ld, long long bs) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int bi = blockIdx.y, bj = blockIdx.x;
  if (bj < bi) return;
  __nv_bfloat16* base = C + static_cast<long long>(blockIdx.z) * bs;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8 threads
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int row = bi * 32 + r, col = bj * 32 + tx;
    if (row < n && col < n) tile[r][tx] = base[static_cast<long long>(row) * ld + col];
  }
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 32; r += 8) {
    const int row = bj * 32 + r, col = bi * 32 + tx;               // destination: transposed block
    if (row < n && col < n && row > col) base[static_cast<long long>(row) * ld + col] = tile[tx][r];
  }
}

cudaError_t symmetrize_bf16(void* C, int n, long long ld, long long bs, int batch, cudaStream_t stream) {
  if (n <= 0 || batch <= 0) return cudaErrorInvalidValue;
  const int blocks = (n + 31) / 32;
  if (batch > 65535 || blocks > 65535) return cudaErrorInvalidValue;
  symmetrize_bf16_kernel<<<dim3(blocks, blocks, batch), 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(C), n, ld, bs);
  return cudaGetLastError();
}

cudaError_t gemm_bf16(const GemmDesc& d, int* status, cudaStream_t stream) {
  if (d.M <= 0 || d.N <= 0 || d.K <= 0 || d.batch <= 0) return cudaErrorInvalidValue;
  if ((d.N & 7) || (d.lda & 7) || (d.ldb & 7) || (d.ldc & 3)) return cudaErrorInvalidValue;
  const GemmPlan p = gemm_plan(d, false);
  if (best_is_invalid(p, d)) return cudaErrorInvalidValue;
  return launch_major<false>(p.bn, p.pair, d, status, stream);
}

cudaError_t gemm_fp8(const GemmDesc& d, int* status, cudaStream_t stream) {
  if (d.M <= 0 || d.N <= 0 || d.K <= 0 || d.batch <= 0) return cudaErrorInvalidValue;
  // TMA strides are multiples of 16 bytes; output rows as for the bf16 kernel
  if ((d.N & 7) || (d.lda & 15) || (d.ldb & 15) || (d.ldc & 3)) return cudaErrorInvalidValue;
  const GemmPlan p = gemm_plan(d, true);
  if (best_is_invalid(p, d)) return cudaErrorInvalidValue;
  return launch_major<true>(p.bn, p.pair, d, status, stream);
}


template <int BN>
static cudaError_t launch_mx(const GemmDesc& d, const MxScales& sf, int* status, cudaStream_t stream) {
  using C = MxCfg<BN>;
  static PerDeviceOnce configured;
  auto kern = gemm_mx_kernel<BN>;
  cudaError_t ce = configured.once(
      [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES); });
  if (ce != cudaSuccess) return ce;
  CUtensorMap tmA, tmB;
  const uint64_t batch = 1;
  {
    uint64_t dims[3] = {(uint64_t)d.K, (uint64_t)d.M, batch}, str[2];
    uint32_t box[3] = {C::BK, BM, 1};
    str[0] = static_cast<uint64_t>(d.lda);
    str[1] = str[0] * dims[1];
    if (!make_tmap(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.A, dims, str, box)) return cudaErrorInvalidValue;
  }
  {
    uint64_t dims[3] = {(uint64_t)d.K, (uint64_t)d.N, batch}, str[2];
    uint32_t box[3] = {C::BK, BN, 1};
    str[0] = static_cast<uint64_t>(d.ldb);
    str[1] = str[0] * dims[1];
    if (!make_tmap(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.B, dims, str, box)) return cudaErrorInvalidValue;
  }
  GemmKernelArgs a;
  a.M = d.M; a.N = d.N; a.K = d.K; a.batch = 1;
  a.C = d.C; a.ldc = d.ldc; a.bsc = 0;
  a.aux = d.aux; a.ldaux = d.ldaux; a.bsaux = 0;
  a.alpha = d.alpha; a.beta = d.beta; a.epi = d.epi; a.c_f32 = d.c_f32; a.f32_staged = f32_staged_default();
  a.c_tma = 0;
  a.scale_a = nullptr; a.scale_b = nullptr; a.amax_out = d.amax_out;
  a.m_blocks = (d.M + BM - 1) / BM;
  a.n_blocks = (d.N + BN - 1) / BN;
  a.group_m = group_m_override(16);
  a.symmetric = 0;
  a.tiles_per_batch = a.m_blocks * a.n_blocks;
  a.idesc = umma_idesc_mxf8(BM, BN, d.a_e5m2, d.b_e5m2, 0, 0);
  a.status = status;
  MxKernelScales ks;
  ks.sfa = sf.sfa; ks.sfb = sf.sfb; ks.k_blocks = d.K / 128; ks.sfb_row_blocks = (d.N + 127) / 128;
  const long long tiles = 1ll * a.m_blocks * a.n_blocks;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  kern<<<grid, GEMM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, a, ks);
  return cudaGetLastError();
}

cudaError_t gemm_mxfp8(const GemmDesc& d, const MxScales& sf, int* status, cudaStream_t stream) {
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return cudaSuccess;
  if (d.a_mn || d.b_mn || d.batch != 1 || (d.K % 128) || (d.lda % 16) || (d.ldb % 16) || !sf.sfa || !sf.sfb ||
      (reinterpret_cast<uintptr_t>(sf.sfa) & 15) || (reinterpret_cast<uintptr_t>(sf.sfb) & 15))
    return cudaErrorInvalidValue;
  if (d.c_f32 ? (d.N % 4) : (d.N % 8)) return cudaErrorInvalidValue;
  const int bn = d.bn ? d.bn : (d.N > 128 ? 256 : 128);
  if (bn == 256) return launch_mx<256>(d, sf, status, stream);
  if (bn == 128) return launch_mx<128>(d, sf, status, stream);
  return cudaErrorInvalidValue;
}

}  // namespace nc
