// tcgen05 GEMM engine with fused bias + activation epilogue, and the xb_gemm
// dispatcher.
//
//   Y[b] = act(alpha * A[b] * B[b]^T + beta * bias[b])
//   A [M,K] row-major (K-major), B [N,K] row-major (K-major), fp16 or bf16,
//   fp32 accumulation in tensor memory.
//
// Persistent kernel, one CTA per SM, 128 x BLOCK_N output tiles. Warp 0 streams
// 128x64 A tiles (and BLOCK_Nx64 B tiles) through a shared-memory ring with TMA
// (as many stages as fit; 128-byte swizzle, out-of-range rows/columns zero-filled
// by the TMA unit, so M, N and K tails need no padding in HBM). When the whole
// B tile (all of K) is small and many m tiles share it, it is loaded once and stays
// resident while the CTA walks a contiguous run of tiles. Warp 1 issues
// tcgen05.mma (128 x BLOCK_N x 16 per instruction) into one of two TMEM
// accumulators and releases ring slots with tcgen05.commit. Warps 2-17 read the
// accumulator with tcgen05.ld (one output row per thread, a quarter of the
// columns per warpgroup), apply bias and activation and store with an arbitrary
// row stride, which is what lets parallel branches write side by side into one
// wide output (axis-1 concat) or stacked (axis 0).
#include <algorithm>
#include <mutex>
#include <cstring>

#include "xb_common.cuh"
#include "xb_umma.cuh"

namespace xb {

int gemm_simt(const xb_gemm_args& a, cudaStream_t stream);

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;
constexpr int MAX_STAGES = 8;       // the launch picks as many as fit in shared memory (at least 2)
constexpr int SMEM_BUDGET = 220 * 1024;
constexpr int A_STAGE_BYTES = BLOCK_M * BLOCK_K * 2;

struct UmmaGemmParams {
  int M, N, K, block_n, tmem_cols, tiles_m, tiles_n, batch, stages;
  int b_resident;        // the B tile (all of K) stays in shared memory while consecutive tiles share it
  uint32_t tiles_per_cta;
  float alpha, beta;
  int a_batched, b_batched;
  const void* bias; int64_t ldbias, stride_bias; int bias_kind, bias_dtype, bias_group;
  void* Y; int64_t ldy, stride_y; int y_dtype;
  EpiParams epi; int64_t stride_ep;
  uint32_t idesc;
};

template <typename TOut>
__device__ __forceinline__ void store_row16(TOut* dst, const float (&v)[16], int valid, bool vec_ok) {
  if (sizeof(TOut) == 2 && vec_ok && valid == 16) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      TOut lo = from_f32<TOut>(v[2 * i]), hi = from_f32<TOut>(v[2 * i + 1]);
      w[i] = (uint32_t)(*reinterpret_cast<uint16_t*>(&lo)) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&hi)) << 16);
    }
    uint4* d = reinterpret_cast<uint4*>(dst);
    d[0] = make_uint4(w[0], w[1], w[2], w[3]);
    d[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else if (sizeof(TOut) == 4 && vec_ok && valid == 16) {
    float4* d = reinterpret_cast<float4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    for (int i = 0; i < valid; ++i) dst[i] = from_f32<TOut>(v[i]);
  }
}

// 16 epilogue warps: four per TMEM lane quarter, each owning a quarter of the tile's columns, so every
// scheduler has four of them to hide the TMEM round trip and the store latency behind one another
constexpr int EPI_WARPS = 16;
constexpr int GEMM_THREADS = 64 + EPI_WARPS * 32;

// 16 results of one output row as one (fp32: four) 16-byte store(s)
template <typename TOut>
__device__ __forceinline__ void store16_vec(TOut* dst, const float (&v)[16]);
template <>
__device__ __forceinline__ void store16_vec<float>(float* dst, const float (&v)[16]) {
  float4* d = reinterpret_cast<float4*>(dst);
#pragma unroll
  for (int i = 0; i < 4; ++i) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}
template <>
__device__ __forceinline__ void store16_vec<__half>(__half* dst, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  uint4* d = reinterpret_cast<uint4*>(dst);
  d[0] = make_uint4(w[0], w[1], w[2], w[3]);
  d[1] = make_uint4(w[4], w[5], w[6], w[7]);
}
template <>
__device__ __forceinline__ void store16_vec<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  uint4* d = reinterpret_cast<uint4*>(dst);
  d[0] = make_uint4(w[0], w[1], w[2], w[3]);
  d[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Activation of 16 adjacent columns of one row; the per-column parameters sit in shared memory and are
// read as 16-byte vectors (all lanes read the same address: a broadcast).
template <int KIND>
__device__ __forceinline__ void epi_apply16(float (&v)[16], const float* s_a, const float* s_b, const float* s_c) {
  if constexpr (KIND != XB_EPI_NONE) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (KIND == XB_EPI_PRELU) {
      const float4 a = reinterpret_cast<const float4*>(s_a)[j];
      // x * (x < 0 ? w : 1): the same value as act_prelu for every x, signed zeros and NaN included
      v[4 * j] *= v[4 * j] < 0.f ? a.x : 1.f;
      v[4 * j + 1] *= v[4 * j + 1] < 0.f ? a.y : 1.f;
      v[4 * j + 2] *= v[4 * j + 2] < 0.f ? a.z : 1.f;
      v[4 * j + 3] *= v[4 * j + 3] < 0.f ? a.w : 1.f;
    } else if (KIND == XB_EPI_DICE) {
      const float4 g = reinterpret_cast<const float4*>(s_a)[j];
      const float4 b = reinterpret_cast<const float4*>(s_b)[j];
      const float4 c = reinterpret_cast<const float4*>(s_c)[j];
      const float gg[4] = {g.x, g.y, g.z, g.w}, bb[4] = {b.x, b.y, b.z, b.w}, cc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x = v[4 * j + i];
        const float pr = __fdividef(1.f, 1.f + __expf(-fmaf(x, cc[i], bb[i])));
        v[4 * j + i] = x * fmaf(pr, 1.f - gg[i], gg[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * j + i] = act_sigmoid(v[4 * j + i]);
    }
  }
  }
}

// 8 results as one 16-byte piece of 2-byte elements
template <typename TOut>
__device__ __forceinline__ uint4 pack8(const float* v);
template <>
__device__ __forceinline__ uint4 pack8<__half>(const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack8<float>(const float*) { return make_uint4(0, 0, 0, 0); }   // not used

constexpr int EPI_STAGE_BYTES = 32 * 64;      // per epilogue warp: 32 rows x 32 two-byte results

// Epilogue of a tile that lies fully inside the output, with a per-column bias (or none) and 16-byte
// aligned rows: this thread's row, columns [16 * c_begin, 16 * c_end) of the tile.
// Two-byte outputs go through a 2 KB staging area of the warp: a thread holds 64 contiguous bytes of its
// own row, and a store instruction of one piece per lane would touch 32 different lines; after the
// exchange the 32 lanes of an instruction write 8 rows x 64 contiguous bytes. Piece j of row l is kept at
// position j ^ ((l >> 1) & 3) of the row, which makes both the writes (lane = row) and the reads (four
// lanes per row) free of bank conflicts.
template <typename TOut, int KIND>
__device__ __forceinline__ void epi_tile_fast(uint32_t tmem_row, int c_begin, int c_end, float alpha,
                                              const float* s_bias, const float* s_a, const float* s_b,
                                              const float* s_c, TOut* yrow, int64_t ldy, uint4* stage, int lane) {
  using namespace umma;
  for (int cg = c_begin; cg < c_end; cg += 2) {
    // two chunks per TMEM round trip when the thread owns two more
    uint32_t raw[32];
    const bool two = cg + 1 < c_end;                                    // uniform across the CTA
    if (two) {
      tmem_ld32_nowait(tmem_row + (uint32_t)(cg * 16), raw);
    } else {
#pragma unroll
      for (int i = 16; i < 32; ++i) raw[i] = 0u;
      tmem_ld16_lo_nowait(tmem_row + (uint32_t)(cg * 16), raw);
    }
    tmem_wait_ld(raw);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !two) break;
      const int c = (cg + u) * 16;
      float v[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 b = reinterpret_cast<const float4*>(s_bias + c)[j];
        v[4 * j] = fmaf(alpha, __uint_as_float(raw[16 * u + 4 * j]), b.x);
        v[4 * j + 1] = fmaf(alpha, __uint_as_float(raw[16 * u + 4 * j + 1]), b.y);
        v[4 * j + 2] = fmaf(alpha, __uint_as_float(raw[16 * u + 4 * j + 2]), b.z);
        v[4 * j + 3] = fmaf(alpha, __uint_as_float(raw[16 * u + 4 * j + 3]), b.w);
      }
      epi_apply16<KIND>(v, s_a + c, s_b + c, s_c + c);
      if (sizeof(TOut) == 2 && two) {
        const int sw = (lane >> 1) & 3;
        stage[lane * 4 + ((2 * u) ^ sw)] = pack8<TOut>(v);
        stage[lane * 4 + ((2 * u + 1) ^ sw)] = pack8<TOut>(v + 8);
      } else {
        store16_vec<TOut>(yrow + c, v);
      }
    }
    if (sizeof(TOut) == 2 && two) {
      __syncwarp();
      TOut* base = yrow + cg * 16 + (lane & 3) * 8;          // this lane's 16-byte column slot, in its own row
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 8 * i + (lane >> 2);
        const uint4 x = stage[r * 4 + ((lane & 3) ^ ((r >> 1) & 3))];
        *reinterpret_cast<uint4*>(base + (int64_t)(r - lane) * ldy) = x;
      }
      __syncwarp();                                          // the next round overwrites the staging area
    }
  }
}

template <typename TOut>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ UmmaGemmParams p) {
  using namespace umma;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int b_stage_bytes = p.block_n * BLOCK_K * 2;
  uint8_t* smem_a = smem;
  const int STAGES = p.stages;
  uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;      // per-stage B tiles, or the resident B tile (all k blocks)
  __shared__ __align__(8) uint64_t b_full, b_free;
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
  // tile numbers fit 31 bits (checked by the host): 32-bit divisions, a few per tile and thread
  const uint32_t tiles_mn = (uint32_t)p.tiles_m * (uint32_t)p.tiles_n;
  const uint32_t total_tiles = tiles_mn * (uint32_t)p.batch;
  const uint32_t acc_stride = (uint32_t)p.tmem_cols / 2;
  // Tile sequence of this CTA, the same for every role. With a resident B tile each CTA takes a contiguous
  // run (m fastest), so that B changes once or twice per CTA; otherwise CTAs interleave, so that the CTAs
  // running at the same time read the same B tile from L2.
  const bool bres = p.b_resident != 0;
  const uint32_t tile_first = bres ? blockIdx.x * p.tiles_per_cta : blockIdx.x;
  const uint32_t tile_step = bres ? 1u : gridDim.x;
  const uint32_t tile_end = bres ? min(total_tiles, tile_first + p.tiles_per_cta) : total_tiles;
  const int b_bytes_per_load = bres ? 0 : b_stage_bytes;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&b_full), 1);
    mbar_init(smem_u32(&b_free), 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&acc_full[s]), 1); mbar_init(smem_u32(&acc_empty[s]), EPI_WARPS); }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), (uint32_t)p.tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;                 // stage and its phase: the stage counter wraps, the phase flips
      uint32_t b_loads = 0;
      int cur_n0 = -1, cur_b = -1;
      bool ok = true;
      for (uint32_t tile = tile_first; tile < tile_end && ok; tile += tile_step) {
        const int b = (int)(tile / tiles_mn);
        const uint32_t rem = tile - (uint32_t)b * tiles_mn, nt = rem / (uint32_t)p.tiles_m;
        const int m0 = (int)(rem - nt * (uint32_t)p.tiles_m) * BLOCK_M, n0 = (int)nt * p.block_n;
        if (bres && (n0 != cur_n0 || b != cur_b)) {
          cur_n0 = n0; cur_b = b;
          // the MMAs that read the previous B tile have completed (signalled after the last tile that used it)
          if (b_loads > 0) ok = mbar_wait(smem_u32(&b_free), (b_loads - 1) & 1u, 5);
          if (!ok) break;
          mbar_arrive_expect_tx(smem_u32(&b_full), (uint32_t)(num_kb * b_stage_bytes));
          for (int kb = 0; kb < num_kb; ++kb)
            tma_load_3d(smem_u32(smem_b + kb * b_stage_bytes), &map_b, smem_u32(&b_full), kb * BLOCK_K, n0,
                        p.b_batched ? b : 0);
          ++b_loads;
        }
        for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
          ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, 1);
          if (!ok) break;
          mbar_arrive_expect_tx(smem_u32(&full_bar[s]), (uint32_t)(A_STAGE_BYTES + b_bytes_per_load));
          tma_load_3d(smem_u32(smem_a + s * A_STAGE_BYTES), &map_a, smem_u32(&full_bar[s]), kb * BLOCK_K, m0,
                      p.a_batched ? b : 0);
          if (!bres)
            tma_load_3d(smem_u32(smem_b + s * b_stage_bytes), &map_b, smem_u32(&full_bar[s]), kb * BLOCK_K, n0,
                        p.b_batched ? b : 0);
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the issue loop in uniform control flow and one elected lane issues: the descriptors then
    // live in uniform registers, which is what the MMA instruction reads, and the issue cost per MMA drops to about
    // a third of what one thread under `if (lane == 0)` pays.
    {
      int s = 0, it = 0;
      uint32_t ph = 0;
      uint32_t b_loads = 0;
      uint32_t cur_bn = 0xffffffffu;             // (batch, n tile) of the resident B tile
      bool ok = true;
      for (uint32_t tile = tile_first; tile < tile_end && ok; tile += tile_step, ++it) {
        const int as = it & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc_empty[as]), ((uint32_t)(it >> 1) & 1u) ^ 1u, 4));   // epilogue drained it
        if (!ok) break;
        if (bres && tile / (uint32_t)p.tiles_m != cur_bn) {
          cur_bn = tile / (uint32_t)p.tiles_m;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&b_full), b_loads & 1u, 6));
          if (!ok) break;
          ++b_loads;
        }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + as * acc_stride;
        for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s]), ph, 2));
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + (bres ? kb : s) * b_stage_bytes);
#pragma unroll
          for (int k = 0; k < BLOCK_K / 16; ++k) {
            const uint64_t da = make_desc_sw128(a_addr + k * 32, 1024);
            const uint64_t db = make_desc_sw128(b_addr + k * 32, 1024);
            mma_f16_ss_elect(tmem_acc, da, db, p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit_elect(smem_u32(&empty_bar[s]));     // slot free once these MMAs have read it
        }
        mma_commit_elect(smem_u32(&acc_full[as]));       // accumulator complete
        // the next tile of this CTA needs another B tile: tell the producer when these MMAs are done with this one
        if (bres && ok && tile + tile_step < tile_end && (tile + tile_step) / (uint32_t)p.tiles_m != cur_bn)
          mma_commit_elect(smem_u32(&b_free));
      }
    }
  } else {
    // epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32); the four warpgroups split the columns.
    // Per-column operands (bias, activation parameters) are staged in shared memory once per (n tile,
    // batch) - a persistent CTA walks m tiles first, so that is rare - and each thread loads all the
    // accumulator chunks it owns before it waits, so one TMEM round trip is exposed per tile.
    const int ew = warp - 2;
    const int q = warp & 3;
    const int part = ew >> 2;
    const int row = q * 32 + lane;
    const int chunks = p.block_n / 16;
    const int c_begin = chunks * part / 4, c_end = chunks * (part + 1) / 4;
    const bool vec_base = ((reinterpret_cast<uintptr_t>(p.Y) & 15) == 0) && ((p.ldy * sizeof(TOut)) % 16 == 0) &&
                          ((p.stride_y * sizeof(TOut)) % 16 == 0);
    float* s_bias = reinterpret_cast<float*>(smem + STAGES * A_STAGE_BYTES +
                                             (bres ? num_kb : STAGES) * b_stage_bytes);           // [4][256]
    uint4* stage = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(s_bias + 4 * 256) + ew * EPI_STAGE_BYTES);
    float* s_a = s_bias + 256;
    float* s_b = s_a + 256;
    float* s_c = s_b + 256;
    int it = 0, cur_n0 = -1, cur_b = -1;
    bool ok = true;
    // A warp whose accumulator wait ran out keeps walking the tile sequence without touching tensor memory,
    // global memory or the acc_empty barrier: the other epilogue warps may have passed the same wait (each
    // lane keeps its own clock), and they still need this warp at the two named barriers below.
    for (uint32_t tile = tile_first; tile < tile_end; tile += tile_step, ++it) {
      const int b = (int)(tile / tiles_mn);
      const uint32_t rem = tile - (uint32_t)b * tiles_mn, nt = rem / (uint32_t)p.tiles_m;
      const int m0 = (int)(rem - nt * (uint32_t)p.tiles_m) * BLOCK_M, n0 = (int)nt * p.block_n;
      const int as = it & 1;
      const int gm = m0 + row;
      const int brow = p.bias_group > 1 ? (int)((uint32_t)gm / (uint32_t)p.bias_group) : gm;   // bias row of this output row
      if (n0 != cur_n0 || b != cur_b) {
        cur_n0 = n0; cur_b = b;
        asm volatile("bar.sync 2, 512;" ::: "memory");                  // everyone is done with the old columns
        const int e = ew * 32 + lane, gn = n0 + e;
        if (e < p.block_n) {
          const bool in = gn < p.N;
          float bv = 0.f, pa = 0.f, pb = 0.f, pc = 0.f;
          if (in && p.bias_kind == XB_BIAS_ROW) bv = p.beta * load_as_f32(p.bias, (int64_t)b * p.stride_bias + gn, p.bias_dtype);
          if (in && p.epi.kind == XB_EPI_PRELU) pa = p.epi.a[(int64_t)b * p.stride_ep + (p.epi.count == 1 ? 0 : gn)];
          if (in && p.epi.kind == XB_EPI_DICE) {
            const float var = p.epi.c[(int64_t)b * p.stride_ep + gn];
            pa = p.epi.a[(int64_t)b * p.stride_ep + gn];                            // gamma
            pc = p.epi.nosqrt ? 1.f / var : rsqrtf(var + 1e-8f);                    // 1/std
            pb = -p.epi.b[(int64_t)b * p.stride_ep + gn] * pc;                      // -mean/std
          }
          s_bias[e] = bv; s_a[e] = pa; s_b[e] = pb; s_c[e] = pc;
        }
        asm volatile("bar.sync 2, 512;" ::: "memory");
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc_full[as]), (uint32_t)(it >> 1) & 1u, 3));
      if (!ok) continue;
      tc_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + as * acc_stride + ((uint32_t)(q * 32) << 16);
      TOut* yrow = reinterpret_cast<TOut*>(p.Y) + (int64_t)b * p.stride_y + (int64_t)gm * p.ldy;
      if (vec_base && p.bias_kind != XB_BIAS_FULL && m0 + BLOCK_M <= p.M && n0 + p.block_n <= p.N &&
          (n0 * sizeof(TOut)) % 16 == 0) {
        // the common case, without the per-chunk edge and bias-matrix handling of the loop below
        switch (p.epi.kind) {
          case XB_EPI_PRELU:
            epi_tile_fast<TOut, XB_EPI_PRELU>(tmem_acc, c_begin, c_end, p.alpha, s_bias, s_a, s_b, s_c, yrow + n0, p.ldy, stage, lane); break;
          case XB_EPI_DICE:
            epi_tile_fast<TOut, XB_EPI_DICE>(tmem_acc, c_begin, c_end, p.alpha, s_bias, s_a, s_b, s_c, yrow + n0, p.ldy, stage, lane); break;
          case XB_EPI_SIGMOID:
            epi_tile_fast<TOut, XB_EPI_SIGMOID>(tmem_acc, c_begin, c_end, p.alpha, s_bias, s_a, s_b, s_c, yrow + n0, p.ldy, stage, lane); break;
          default:
            epi_tile_fast<TOut, XB_EPI_NONE>(tmem_acc, c_begin, c_end, p.alpha, s_bias, s_a, s_b, s_c, yrow + n0, p.ldy, stage, lane); break;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&acc_empty[as]));
        continue;
      }
      for (int cg = c_begin; cg < c_end; ++cg) {
        uint32_t raw[1][16];
        tmem_ld16_nowait(tmem_acc + (uint32_t)(cg * 16), raw[0]);
        tmem_wait_ld(raw[0]);
        for (int u = 0; u < 1; ++u) {
          const int c = (cg + u) * 16;
          const int gn0 = n0 + c;
          int valid = p.N - gn0;
          valid = valid > 16 ? 16 : valid;
          if (cg + u >= c_end || valid <= 0) continue;                   // uniform across the warp
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = fmaf(p.alpha, __uint_as_float(raw[u][i]), s_bias[c + i]);
          if (p.bias_kind == XB_BIAS_FULL && gm < p.M) {
            const int64_t base = (int64_t)b * p.stride_bias + (int64_t)brow * p.ldbias + gn0;
            const float* bf = reinterpret_cast<const float*>(p.bias) + base;
            if (p.bias_dtype == XB_F32 && valid == 16 && (reinterpret_cast<uintptr_t>(bf) & 15) == 0) {
              // fp32 rows (the per-group partial product of a pruned GEMM): four 16-byte loads, mostly one
              // address per warp since consecutive output rows share the bias row
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float4 t = __ldg(reinterpret_cast<const float4*>(bf) + i);
                v[4 * i] += p.beta * t.x; v[4 * i + 1] += p.beta * t.y;
                v[4 * i + 2] += p.beta * t.z; v[4 * i + 3] += p.beta * t.w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (i < valid) v[i] += p.beta * load_as_f32(p.bias, base + i, p.bias_dtype);
            }
          }
          if (p.epi.kind == XB_EPI_PRELU) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = act_prelu(v[i], s_a[c + i]);
          } else if (p.epi.kind == XB_EPI_DICE) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g = s_a[c + i];
              const float pr = __fdividef(1.f, 1.f + __expf(-fmaf(v[i], s_c[c + i], s_b[c + i])));
              v[i] = v[i] * fmaf(pr, 1.f - g, g);
            }
          } else if (p.epi.kind == XB_EPI_SIGMOID) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = act_sigmoid(v[i]);
          }
          if (gm < p.M) store_row16<TOut>(yrow + gn0, v, valid, vec_base && ((gn0 * sizeof(TOut)) % 16 == 0));
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[as]));              // one arrival per epilogue warp
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// [batch, rows, K] tensor of 2-byte elements, box {64, box_rows, 1}, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, int is_bf16, int64_t K, int64_t rows, int64_t ld, int64_t batch,
             int64_t batch_stride, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(XB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? batch_stride : ld * rows) * 2};
  if (strides[1] == 0) strides[1] = strides[0];
  cuuint32_t box[3] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(XB_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

int pick_block_n(int N) {
  if (N <= 256) return (N + 15) / 16 * 16;
  return (N % 256 == 0) ? 256 : 128;
}

bool umma_eligible(const xb_gemm_args& a) {
  if (a.ab_dtype != XB_F16 && a.ab_dtype != XB_BF16) return false;
  if (a.trans_a || !a.trans_b) return false;
  if (a.y_dtype != XB_F16 && a.y_dtype != XB_BF16 && a.y_dtype != XB_F32) return false;
  if (a.lda % 8 || a.ldb % 8 || a.stride_a % 8 || a.stride_b % 8) return false;
  if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15)) return false;
  if (a.lda < a.K || a.ldb < a.K) return false;
  return true;
}

template <typename TOut>
int launch_umma(const CUtensorMap& ma, const CUtensorMap& mb, const UmmaGemmParams& p, dim3 grid, size_t smem,
                cudaStream_t s) {
  static PerDeviceOnce attr_set;   // per instantiation
  XB_SET_MAX_SMEM_ONCE(attr_set, SMEM_BUDGET + 6 * 1024, (const void*)gemm_umma_kernel<TOut>);
  gemm_umma_kernel<TOut><<<grid, GEMM_THREADS, smem, s>>>(ma, mb, p);
  return check_launch("gemm_umma_kernel");
}

int gemm_umma(const xb_gemm_args& a, cudaStream_t stream) {
  UmmaGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.block_n = pick_block_n(a.N);
  p.tmem_cols = 64;                                      // two accumulator stages, each at least 32 columns
  while (p.tmem_cols < 2 * p.block_n) p.tmem_cols <<= 1;
  p.alpha = a.alpha; p.beta = a.beta;
  p.a_batched = a.stride_a != 0; p.b_batched = a.stride_b != 0;
  p.bias = a.bias; p.ldbias = a.ldbias; p.stride_bias = a.stride_bias;
  p.bias_group = a.bias_row_group > 1 ? (int)a.bias_row_group : 1;
  p.bias_kind = a.bias ? a.bias_kind : XB_BIAS_NONE; p.bias_dtype = a.bias_dtype;
  p.Y = a.Y; p.ldy = a.ldy; p.stride_y = a.stride_y; p.y_dtype = a.y_dtype;
  p.epi.kind = a.epilogue; p.epi.a = a.ep_a; p.epi.b = a.ep_b; p.epi.c = a.ep_c;
  p.epi.count = a.ep_count; p.epi.nosqrt = a.dice_nosqrt; p.stride_ep = a.stride_ep;
  const int is_bf16 = a.ab_dtype == XB_BF16;
  p.idesc = umma::make_idesc(BLOCK_M, p.block_n, is_bf16);
  CUtensorMap ma, mb;
  if (int rc = make_map(&ma, a.A, is_bf16, a.K, a.M, a.lda, p.a_batched ? a.batch : 1, a.stride_a, BLOCK_M)) return rc;
  if (int rc = make_map(&mb, a.B, is_bf16, a.K, a.N, a.ldb, p.b_batched ? a.batch : 1, a.stride_b, p.block_n)) return rc;
  p.tiles_m = (a.M + BLOCK_M - 1) / BLOCK_M;
  p.tiles_n = (a.N + p.block_n - 1) / p.block_n;
  p.batch = a.batch;
  const int64_t total = (int64_t)p.tiles_m * p.tiles_n * p.batch;
  XB_REQUIRE(total < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_gemm: %lld output tiles are too many for one call", (long long)total);
  // persistent: one CTA per SM walks the tiles; the accumulator is double-buffered in TMEM so the
  // epilogue of one tile overlaps the loads and MMAs of the next
  dim3 grid((unsigned)std::min<int64_t>(total, sm_count()));
  // When the whole B tile (all of K) is small and several m tiles share it, it is loaded once and stays in
  // shared memory: re-reading it from L2 for every tile doubles the L2-to-SM traffic of a thin GEMM, which
  // then bounds the kernel below the HBM rate.
  const int b_stage_bytes = p.block_n * BLOCK_K * 2;
  const int num_kb = (a.K + BLOCK_K - 1) / BLOCK_K;
  const int grid_ctas = (int)std::min<int64_t>(total, sm_count());
  p.tiles_per_cta = (uint32_t)((total + grid_ctas - 1) / grid_ctas);
  p.b_resident = (int64_t)num_kb * b_stage_bytes <= 96 * 1024 && p.tiles_m >= 4 && p.tiles_per_cta >= 2;
  // after the ring: per-column epilogue parameters [4][256] fp32, then the epilogue warps' staging areas
  const int tail = 4 * 256 * (int)sizeof(float) + (a.y_dtype == XB_F32 ? 0 : EPI_WARPS * EPI_STAGE_BYTES);
  size_t smem;
  if (p.b_resident) {
    const int b_bytes = num_kb * b_stage_bytes;
    p.stages = std::max(2, std::min(MAX_STAGES, (SMEM_BUDGET - tail - b_bytes) / A_STAGE_BYTES));
    smem = (size_t)p.stages * A_STAGE_BYTES + b_bytes + tail + 1024;
  } else {
    const int stage_bytes = A_STAGE_BYTES + b_stage_bytes;
    p.stages = std::max(2, std::min(MAX_STAGES, (SMEM_BUDGET - tail) / stage_bytes));
    smem = (size_t)p.stages * stage_bytes + tail + 1024;
  }
  switch (a.y_dtype) {
    case XB_F16: return launch_umma<__half>(ma, mb, p, grid, smem, stream);
    case XB_BF16: return launch_umma<__nv_bfloat16>(ma, mb, p, grid, smem, stream);
    default: return launch_umma<float>(ma, mb, p, grid, smem, stream);
  }
}

}  // namespace

int gemm_umma_status(int* out) { return umma::read_status_word(out); }
int gemm_umma_clear_status() { return umma::clear_status_word(); }

}  // namespace xb

using namespace xb;

namespace xb {
int att_status(int* out);
int att_clear_status();
int tower_status(int* out);
int tower_clear_status();
int att_set_status_mirror(int* p);
int tower_set_status_mirror(int* p);
int rnn_status(int* out);
int rnn_clear_status();
int rnn_set_status_mirror(int* p);

// Host-mapped copy of the status word, one per device: {host address, device address}.
struct StatusMirror { volatile int* host = nullptr; int* dev = nullptr; };
static StatusMirror g_mirror[64];
static std::mutex g_mirror_mu;
}  // namespace xb

// A wait that nothing will ever satisfy, with its own short limit: shows that a bounded wait gives up,
// records where, and leaves the context usable. Site code 99.
__global__ void wait_selftest_kernel(long long limit_cycles) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    umma::mbar_init(umma::smem_u32(&bar), 1);
    umma::fence_barrier_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  bool done = false;
  while (!(done = umma::mbar_try_wait(umma::smem_u32(&bar), 0))) {
    if (clock64() - t0 > limit_cycles) break;
  }
  if (!done && threadIdx.x == 0) umma::wait_gave_up(99);
}

extern "C" int xb_selftest_wait_timeout(int64_t limit_cycles, xb_stream_t stream) {
  XB_REQUIRE(limit_cycles > 0 && limit_cycles <= ((int64_t)1 << 31), XB_ERR_ARG,
             "xb_selftest_wait_timeout: limit of %lld cycles (1 .. 2^31)", (long long)limit_cycles);
  wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((long long)limit_cycles);
  return check_launch("wait_selftest_kernel");
}

extern "C" int xb_device_status(int* status) {
  XB_REQUIRE(status, XB_ERR_ARG, "xb_device_status: null pointer");
  int a = 0, b = 0, c = 0, d = 0;
  XB_REQUIRE(gemm_umma_status(&a) == 0 && att_status(&b) == 0 && tower_status(&c) == 0 && rnn_status(&d) == 0, XB_ERR_CUDA,
             "xb_device_status: read failed");
  *status = a ? a : (b ? b : (c ? c : d));
  return 0;
}

extern "C" int xb_device_status_clear(void) {
  XB_REQUIRE(gemm_umma_clear_status() == 0 && att_clear_status() == 0 && tower_clear_status() == 0 && rnn_clear_status() == 0, XB_ERR_CUDA,
             "xb_device_status_clear failed");
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lock(g_mirror_mu);
    if (g_mirror[dev].host) *g_mirror[dev].host = 0;
  }
  return 0;
}

extern "C" int xb_device_status_mirror(const volatile int** host_word) {
  XB_REQUIRE(host_word, XB_ERR_ARG, "xb_device_status_mirror: null pointer");
  int dev = 0;
  XB_CUDA(cudaGetDevice(&dev));
  XB_REQUIRE(dev >= 0 && dev < 64, XB_ERR_LIMIT, "xb_device_status_mirror: device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(g_mirror_mu);
  StatusMirror& m = g_mirror[dev];
  if (m.host == nullptr) {
    int* h = nullptr;
    int* d = nullptr;
    XB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped | cudaHostAllocPortable));
    *h = 0;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0) != cudaSuccess) {
      cudaFreeHost(h);
      return fail(XB_ERR_CUDA, "xb_device_status_mirror: cudaHostGetDevicePointer failed");
    }
    if (umma::set_status_mirror(d) != 0 || att_set_status_mirror(d) != 0 || tower_set_status_mirror(d) != 0 ||
        rnn_set_status_mirror(d) != 0) {
      umma::set_status_mirror(nullptr); att_set_status_mirror(nullptr); tower_set_status_mirror(nullptr);
      rnn_set_status_mirror(nullptr);
      cudaFreeHost(h);
      return fail(XB_ERR_CUDA, "xb_device_status_mirror: could not publish the mirror address");
    }
    // a wait may have run out before the mirror existed
    int now = 0;
    if (xb_device_status(&now) == 0) *h = now;
    m.host = h;
    m.dev = d;
  }
  *host_word = m.host;
  return 0;
}

static int validate_gemm(const xb_gemm_args* a) {
  XB_REQUIRE(a, XB_ERR_ARG, "xb_gemm: null arguments");
  XB_REQUIRE(a->M >= 0 && a->N >= 0 && a->K >= 0 && a->batch >= 0, XB_ERR_ARG, "xb_gemm: negative size");
  XB_REQUIRE(a->A && a->B && a->Y, XB_ERR_ARG, "xb_gemm: null matrix");
  XB_REQUIRE(a->ab_dtype == XB_F32 || a->ab_dtype == XB_F16 || a->ab_dtype == XB_BF16, XB_ERR_UNSUPPORTED,
             "xb_gemm: operand dtype %d", a->ab_dtype);
  XB_REQUIRE(a->y_dtype == XB_F32 || a->y_dtype == XB_F16 || a->y_dtype == XB_BF16, XB_ERR_UNSUPPORTED,
             "xb_gemm: output dtype %d", a->y_dtype);
  XB_REQUIRE(a->epilogue >= XB_EPI_NONE && a->epilogue <= XB_EPI_SIGMOID, XB_ERR_UNSUPPORTED,
             "xb_gemm: epilogue %d", a->epilogue);
  XB_REQUIRE(a->epilogue != XB_EPI_PRELU || (a->ep_a && (a->ep_count == 1 || a->ep_count == a->N)), XB_ERR_ARG,
             "xb_gemm: PRelu needs 1 or N slopes");
  XB_REQUIRE(a->epilogue != XB_EPI_DICE || (a->ep_a && a->ep_b && a->ep_c), XB_ERR_ARG,
             "xb_gemm: Dice needs gamma, mean and var");
  XB_REQUIRE(!a->bias || a->bias_kind == XB_BIAS_ROW || a->bias_kind == XB_BIAS_FULL, XB_ERR_ARG,
             "xb_gemm: bias kind %d", a->bias_kind);
  XB_REQUIRE(!a->bias || dtype_size(a->bias_dtype) != 0, XB_ERR_UNSUPPORTED, "xb_gemm: bias dtype %d", a->bias_dtype);
  XB_REQUIRE(a->bias_row_group >= 0 && (a->bias_row_group <= 1 || (a->bias && a->bias_kind == XB_BIAS_FULL)), XB_ERR_ARG,
             "xb_gemm: bias_row_group needs a full [rows, N] bias");
  const int64_t a_cols = a->trans_a ? a->M : a->K, b_cols = a->trans_b ? a->K : a->N;
  XB_REQUIRE(a->lda >= a_cols && a->ldb >= b_cols && a->ldy >= a->N, XB_ERR_ARG,
             "xb_gemm: leading dimension smaller than the row (lda=%lld ldb=%lld ldy=%lld)", (long long)a->lda,
             (long long)a->ldb, (long long)a->ldy);
  return 0;
}

extern "C" int xb_gemm_uses_tcgen05(const xb_gemm_args* a) {
  if (!a || a->engine == XB_GEMM_SIMT) return 0;
  return umma_eligible(*a) ? 1 : 0;
}

extern "C" int xb_gemm(const xb_gemm_args* a, xb_stream_t stream) {
  if (int rc = validate_gemm(a)) return rc;
  if (a->M == 0 || a->N == 0 || a->batch == 0) return 0;
  if (a->engine == XB_GEMM_TCGEN05) {
    XB_REQUIRE(umma_eligible(*a), XB_ERR_UNSUPPORTED,
               "xb_gemm: tcgen05 engine needs fp16/bf16, A [M,K] and B [N,K] row-major, 16-byte aligned, "
               "leading dimensions and batch strides multiples of 8");
    XB_REQUIRE(a->K > 0, XB_ERR_ARG, "xb_gemm: K = 0");
    return gemm_umma(*a, (cudaStream_t)stream);
  }
  // small problems are launch-bound either way; the CUDA-core engine has no TMA descriptor cost
  if (a->engine == XB_GEMM_AUTO && umma_eligible(*a) && a->K > 0 &&
      (int64_t)a->M * a->N * a->batch >= 128 * 64)
    return gemm_umma(*a, (cudaStream_t)stream);
  return gemm_simt(*a, (cudaStream_t)stream);
}
