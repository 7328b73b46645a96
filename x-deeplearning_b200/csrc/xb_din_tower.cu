// Fused DIN tower: feature assembly, the three tower layers with their activations and the final
// softmax in one persistent tcgen05 kernel; nothing between the attention output and the
// probabilities touches HBM.
//
// The first layer runs in the PrunedGemm form (blaze/blaze/operator/op/pruned_gemm_op.h:1-10:
// [A|B] x [C;D] = A x C + B x D): the columns of the layer input that are equal for every candidate
// of a request, [user | his_sum], are multiplied once per request by a small CUDA-core kernel
// (din_tower_partial_kernel, which also forms his_sum); the tower kernel multiplies the per-candidate
// columns [q | q*his_sum | att | q-his_sum] and adds the per-request row in fp32 before the activation.
//
// One CTA walks 128-candidate tiles of single requests. Per tile:
//   workers : q and att rows (prefetched into shared memory with cp.async while the previous tile
//             runs) -> A1 = [q | q*his_sum | att | q-his_sum] as fp16 pairs in tensor memory
//   MMA     : acc1[128 x n1p] = A1 * W1c^T          (A from tensor memory, weights from shared memory)
//   workers : acc1 + partial[request] -> Dice -> A2 in tensor memory (one extra column of ones carries b2)
//   MMA     : acc2[128 x n2p] = A2 * W2^T
//   workers : acc2 -> Dice -> third layer (n3 <= 8 dot products per row, fp32) -> softmax -> HBM
// Eight worker warps in two warpgroups split the columns of every phase; a ninth warp issues the MMAs.
// Dice runs on packed fp16 pairs with one SFU instruction per pair, as in the attention unit:
//   Dice(x) = x * (C + D*tanh(A*x + B)), A = rstd/2, B = -mean*rstd/2, C = (1+gamma)/2, D = (1-gamma)/2.
#include <algorithm>
#include <cstring>

#include "xb_common.cuh"
#include "xb_umma.cuh"

namespace xb {
namespace {

constexpr int TW_THREADS = 288;          // 8 worker warps + 1 MMA-issuing warp
constexpr int TW_WORKERS = 256;
constexpr int TW_MMA_WARP = 8;
constexpr int TW_MAX_N3 = 8;

struct TowerGeom {
  int dp, nch, k1, n1p, k2, n2p;
  int c_acc2, c_a1, c_a2, cols;          // tensor-memory columns: [acc1 | acc2 | A1 | A2]
  // packed image
  int o_w1, o_w2, o_c1, o_c2, o_w3, o_b3, image_bytes;
  // the rest of shared memory
  int o_q, o_att, o_part, o_hs, o_lg, total;
};

__host__ __device__ inline TowerGeom tower_geom(int d, int n1, int n2, int n3) {
  TowerGeom g;
  g.dp = (d + 7) / 8 * 8;
  g.nch = g.dp / 8;
  g.k1 = (4 * g.dp + 15) / 16 * 16;
  g.n1p = (n1 + 15) / 16 * 16;
  g.k2 = g.n1p + 16;                               // column n1p of A2 is constant 1 (bias of layer 2)
  g.n2p = (n2 + 15) / 16 * 16;
  g.c_acc2 = g.n1p;
  g.c_a1 = g.n1p + g.n2p;
  g.c_a2 = g.c_a1 + g.k1 / 2;
  g.cols = g.c_a2 + g.k2 / 2;
  int off = 0;
  g.o_w1 = off; off += g.n1p * g.k1 * 2;
  g.o_w2 = off; off += g.n2p * g.k2 * 2;
  g.o_c1 = off; off += (g.n1p / 2) * 16;
  g.o_c2 = off; off += (g.n2p / 2) * 16;
  g.o_w3 = off; off += g.n2p * TW_MAX_N3 * 4;      // [n2p][8] fp32, zero padded
  g.o_b3 = off; off += TW_MAX_N3 * 4;
  g.image_bytes = off;
  g.o_q = off; off += 2 * 128 * g.dp * 2;          // two tiles of q rows (pitch dp halves)
  g.o_att = off; off += 2 * 128 * g.dp * 2;
  g.o_part = off; off += 2 * g.n1p * 4;            // per-request partial product of layer 1, fp32
  g.o_hs = off; off += 2 * g.dp * 4;               // his_sum of the request, fp32
  g.o_lg = off; off += 128 * TW_MAX_N3 * 4;        // third-layer partial sums of the second warpgroup
  g.total = off;
  (void)n3;
  return g;
}

struct TowerParams {
  const __half* user; int64_t ldu;
  const __half* q; int64_t ldq;
  const __half* k; int64_t ldk;
  const __half* att; int64_t ldatt;
  float* prob;
  float* hs;            // [requests, d]
  float* partial;       // [requests, n1]
  int requests, n_cand, T, d, du, n1, n2, n3, softmax, tiles_per_req;
  const __half* W1; const float* b1; const float *g1, *m1, *v1;
  const __half* W2; const float* b2; const float *g2, *m2, *v2;
  const __half* W3; const float* b3;
  const uint8_t* packed;
  uint32_t idesc1, idesc2;
};

__device__ __forceinline__ uint32_t h2u(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u2h(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

using umma::cp_async16;
using umma::cp_async4;
using umma::cp_async8;
using umma::cp_async_commit;
using umma::cp_async_wait_all;

// ---- once per model: weight operands, activation constants ---------------------------------------
__global__ void tower_pack_kernel(const __grid_constant__ TowerParams p, uint8_t* dst) {
  const TowerGeom G = tower_geom(p.d, p.n1, p.n2, p.n3);
  const int d = p.d, dp = G.dp, du = p.du;
  const __half zero = __float2half(0.f);
  __half* w1 = reinterpret_cast<__half*>(dst + G.o_w1);
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < G.n1p * G.k1; idx += gridDim.x * blockDim.x) {
    const int n = idx / G.k1, kk = idx - n * G.k1;
    __half v = zero;
    if (n < p.n1 && kk < 4 * dp) {
      const int seg = kk / dp, i = kk - seg * dp;
      // layer-1 rows of the per-candidate columns: q, q*his_sum, att, q-his_sum
      const int row0 = seg == 0 ? du : du + (seg + 1) * d;
      if (i < d) v = p.W1[(int64_t)(row0 + i) * p.n1 + n];
    }
    w1[(kk >> 3) * (G.n1p * 8) + n * 8 + (kk & 7)] = v;
  }
  __half* w2 = reinterpret_cast<__half*>(dst + G.o_w2);
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < G.n2p * G.k2; idx += gridDim.x * blockDim.x) {
    const int n = idx / G.k2, kk = idx - n * G.k2;
    __half v = zero;
    if (n < p.n2) {
      if (kk < p.n1) v = p.W2[(int64_t)kk * p.n2 + n];
      else if (kk == G.n1p) v = __float2half_rn(p.b2 ? p.b2[n] : 0.f);
    }
    w2[(kk >> 3) * (G.n2p * 8) + n * 8 + (kk & 7)] = v;
  }
  if (blockIdx.x == 0) {
    uint4* c1 = reinterpret_cast<uint4*>(dst + G.o_c1);
    uint4* c2 = reinterpret_cast<uint4*>(dst + G.o_c2);
    for (int layer = 0; layer < 2; ++layer) {
      const int n = layer ? p.n2 : p.n1, np = layer ? G.n2p : G.n1p;
      const float *gm = layer ? p.g2 : p.g1, *mu = layer ? p.m2 : p.m1, *var = layer ? p.v2 : p.v1;
      uint4* c = layer ? c2 : c1;
      for (int j = threadIdx.x; j < np / 2; j += blockDim.x) {
        float A[2] = {0, 0}, B[2] = {0, 0}, C[2] = {0, 0}, D[2] = {0, 0};
        for (int u = 0; u < 2; ++u) {
          const int col = 2 * j + u;
          if (col >= n) continue;
          const float rs = dice_rstd(var[col], 0), g = gm[col];
          A[u] = 0.5f * rs; B[u] = -0.5f * mu[col] * rs; C[u] = 0.5f * (1.f + g); D[u] = 0.5f * (1.f - g);
        }
        c[j] = make_uint4(h2u(__floats2half2_rn(A[0], A[1])), h2u(__floats2half2_rn(B[0], B[1])),
                          h2u(__floats2half2_rn(C[0], C[1])), h2u(__floats2half2_rn(D[0], D[1])));
      }
    }
    float* w3 = reinterpret_cast<float*>(dst + G.o_w3);
    for (int idx = threadIdx.x; idx < G.n2p * TW_MAX_N3; idx += blockDim.x) {
      const int c = idx / TW_MAX_N3, j = idx - c * TW_MAX_N3;
      w3[idx] = (c < p.n2 && j < p.n3) ? __half2float(p.W3[(int64_t)c * p.n3 + j]) : 0.f;
    }
    float* b3 = reinterpret_cast<float*>(dst + G.o_b3);
    for (int j = threadIdx.x; j < TW_MAX_N3; j += blockDim.x) b3[j] = (j < p.n3 && p.b3) ? p.b3[j] : 0.f;
  }
}

// ---- once per launch: his_sum and the per-request product of layer 1 -------------------------------
// partial[r][n] = b1[n] + sum_c user[r][c] * W1[c][n] + sum_e fp16(his_sum[r][e]) * W1[du+d+e][n]
// One CTA per (request, 64 output columns): 4 groups of 64 threads split the du + d weight rows, sixteen
// independent loads in flight per thread; the group sums are added in group order. his_sum: the T steps
// are split over groups of d threads and added in group order.
constexpr int PT_COLS = 64, PT_SLICES = 4;
__global__ void __launch_bounds__(PT_COLS * PT_SLICES) din_tower_partial_kernel(const __grid_constant__ TowerParams p) {
  extern __shared__ float sm[];            // [d] his_sum, [du] user row, [G][d] step sums, [PT_SLICES][PT_COLS]
  const int r = blockIdx.x, d = p.d, du = p.du;
  float* hs = sm;
  float* us = hs + d;
  float* part = us + du;
  const int G = max(1, min((int)blockDim.x / d, 8));
  float* colsum = part + 8 * d;
  if ((int)threadIdx.x < G * d) {
    const int gi = threadIdx.x / d, e = threadIdx.x - gi * d;
    float s = 0.f;
    for (int t = gi; t < p.T; t += G) s += __half2float(p.k[((int64_t)r * p.T + t) * p.ldk + e]);
    part[gi * d + e] = s;
  }
  for (int e = threadIdx.x; e < du; e += blockDim.x) us[e] = __half2float(p.user[(int64_t)r * p.ldu + e]);
  __syncthreads();
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float s = 0.f;
    for (int gi = 0; gi < G; ++gi) s += part[gi * d + e];
    // his_sum is an fp16 tensor in the model's graph: every use sees the rounded value
    s = __half2float(__float2half_rn(s));
    hs[e] = s;
    if (blockIdx.y == 0) p.hs[(int64_t)r * d + e] = s;
  }
  __syncthreads();
  // weight rows 0..du-1 meet the user row, rows du+d..du+2d-1 meet his_sum; x(c) is the matching input
  const int col = threadIdx.x % PT_COLS, slice = threadIdx.x / PT_COLS;
  const int n = blockIdx.y * PT_COLS + col;
  const int rows = du + d, per = (rows + PT_SLICES - 1) / PT_SLICES;
  const int c_begin = slice * per, c_end = min(rows, c_begin + per);
  float acc = 0.f;
  if (n < p.n1) {
    for (int c0 = c_begin; c0 < c_end; c0 += 16) {
      __half w[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int c = c0 + u;
        const int wr = c < du ? c : c + d;               // skip the q rows of W1
        w[u] = c < c_end ? p.W1[(int64_t)wr * p.n1 + n] : __float2half(0.f);
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int c = c0 + u;
        if (c < c_end) acc = fmaf(c < du ? us[c] : hs[c - du], __half2float(w[u]), acc);
      }
    }
  }
  colsum[slice * PT_COLS + col] = acc;
  __syncthreads();
  if (slice == 0 && n < p.n1) {
    float s = p.b1 ? p.b1[n] : 0.f;
    for (int g = 0; g < PT_SLICES; ++g) s += colsum[g * PT_COLS + col];
    p.partial[(int64_t)r * p.n1 + n] = s;
  }
}

// ---- the tower kernel --------------------------------------------------------------------------------
__global__ void __launch_bounds__(TW_THREADS, 1) din_tower_tc_kernel(const __grid_constant__ TowerParams p) {
  using namespace umma;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[4];
  __shared__ uint32_t tmem_base_s;
  const TowerGeom G = tower_geom(p.d, p.n1, p.n2, p.n3);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = p.d, dp = G.dp, nch = G.nch, n1p = G.n1p, n2p = G.n2p, n3 = p.n3;
  const int64_t total_tiles = (int64_t)p.requests * p.tiles_per_req;

  // weight image: asynchronous 16-byte copies, all in flight at once
  {
    for (int i = threadIdx.x; i < G.image_bytes / 16; i += TW_THREADS) cp_async16(smem + 16 * i, p.packed + 16 * i);
    cp_async_commit();
    for (int i = threadIdx.x; i < (G.total - G.image_bytes) / 16; i += TW_THREADS)
      reinterpret_cast<uint4*>(smem + G.image_bytes)[i] = make_uint4(0, 0, 0, 0);     // padding columns stay zero
    cp_async_wait_all();
  }
  uint64_t* a1_full = &bars[0];
  uint64_t* acc1_full = &bars[1];
  uint64_t* a2_full = &bars[2];
  uint64_t* acc2_full = &bars[3];
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(a1_full), 8);
    mbar_init(smem_u32(acc1_full), 1);
    mbar_init(smem_u32(a2_full), 8);
    mbar_init(smem_u32(acc2_full), 1);
    fence_barrier_init();
  }
  if (warp == TW_MMA_WARP) tmem_alloc(smem_u32(&tmem_base_s), 512);
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = tmem_base_s;

  if (warp == TW_MMA_WARP) {
    // the whole warp runs the issue loop in uniform control flow and one elected lane issues: the descriptors
    // stay in uniform registers, which the MMA instruction reads, and an MMA issues several times faster than
    // from one thread under `if (lane == 0)`
    {
      const uint64_t db1_0 = make_desc_interleaved(smem_u32(smem + G.o_w1), n1p * 16, 128);
      const uint64_t db2_0 = make_desc_interleaved(smem_u32(smem + G.o_w2), n2p * 16, 128);
      const uint64_t db1_step = (uint64_t)((2 * n1p * 16) >> 4), db2_step = (uint64_t)((2 * n2p * 16) >> 4);
      const int nks1 = G.k1 / 16, nks2 = G.k2 / 16;
      uint32_t it = 0;
      for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
        const uint32_t ph = it & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(a1_full), ph, 30))) break;
        tc_fence_after_sync();
#pragma unroll 4
        for (int ks = 0; ks < nks1; ++ks)
          mma_f16_ts_elect(tmem0, tmem0 + G.c_a1 + 8 * ks, db1_0 + (uint64_t)ks * db1_step, p.idesc1, ks > 0 ? 1u : 0u);
        mma_commit_elect(smem_u32(acc1_full));
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(a2_full), ph, 31))) break;
        tc_fence_after_sync();
#pragma unroll 4
        for (int ks = 0; ks < nks2; ++ks)
          mma_f16_ts_elect(tmem0 + G.c_acc2, tmem0 + G.c_a2 + 8 * ks, db2_0 + (uint64_t)ks * db2_step, p.idesc2,
                           ks > 0 ? 1u : 0u);
        mma_commit_elect(smem_u32(acc2_full));
      }
    }
  } else {
    // ---- workers: thread = candidate row of the tile = tensor-memory lane; warpgroup h takes half of the
    //      columns of every phase ----------------------------------------------------------------------
    const int h = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int wtid = threadIdx.x;                       // 0..255
    const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t a1t = lane_addr + G.c_a1, a2t = lane_addr + G.c_a2;
    const uint4* c1 = reinterpret_cast<const uint4*>(smem + G.o_c1);
    const uint4* c2 = reinterpret_cast<const uint4*>(smem + G.o_c2);
    const float* w3 = reinterpret_cast<const float*>(smem + G.o_w3);
    const float* b3 = reinterpret_cast<const float*>(smem + G.o_b3);
    float* lg = reinterpret_cast<float*>(smem + G.o_lg);
    const int pitch = dp * 2;                           // bytes per staged row
    const bool async8 = (d % 4 == 0) && (p.ldq % 4 == 0) && (p.ldatt % 4 == 0) &&
                        (((uintptr_t)p.q | (uintptr_t)p.att) & 7) == 0;

    // requests the rows of a tile into buffer `buf` (rows past the last candidate keep stale data: their
    // results are never stored)
    auto stage = [&](int buf, int64_t tile) {
      const int r = (int)(tile / p.tiles_per_req), n0 = (int)(tile % p.tiles_per_req) * 128;
      const int rows = min(128, p.n_cand - n0);
      uint8_t* qs = smem + G.o_q + buf * 128 * pitch;
      uint8_t* as = smem + G.o_att + buf * 128 * pitch;
      const int64_t g0 = (int64_t)r * p.n_cand + n0;
      if (async8) {
        const int ppr = d / 4;                          // 8-byte pieces per row
        for (int idx = wtid; idx < rows * ppr; idx += TW_WORKERS) {
          const int rr = idx / ppr, pc = idx - rr * ppr;
          cp_async8(qs + rr * pitch + pc * 8, p.q + (g0 + rr) * p.ldq + pc * 4);
          cp_async8(as + rr * pitch + pc * 8, p.att + (g0 + rr) * p.ldatt + pc * 4);
        }
      } else {
        for (int idx = wtid; idx < rows * d; idx += TW_WORKERS) {
          const int rr = idx / d, e = idx - rr * d;
          reinterpret_cast<__half*>(qs + rr * pitch)[e] = p.q[(g0 + rr) * p.ldq + e];
          reinterpret_cast<__half*>(as + rr * pitch)[e] = p.att[(g0 + rr) * p.ldatt + e];
        }
      }
      float* ps = reinterpret_cast<float*>(smem + G.o_part) + buf * n1p;
      float* hs = reinterpret_cast<float*>(smem + G.o_hs) + buf * dp;
      for (int n = wtid; n < p.n1; n += TW_WORKERS) cp_async4(ps + n, p.partial + (int64_t)r * p.n1 + n);
      for (int e = wtid; e < d; e += TW_WORKERS) cp_async4(hs + e, p.hs + (int64_t)r * d + e);
      cp_async_commit();
    };

    // constant columns: zero padding of A1 beyond the four segments, the ones column of A2
    if (h == 0) {
      for (int c = 4 * nch; c < G.k1 / 8; ++c) tmem_st4(a1t + 4 * c, 0u, 0u, 0u, 0u);
      tmem_st4(a2t + n1p / 2, 0x00003C00u, 0u, 0u, 0u);
      tmem_st4(a2t + n1p / 2 + 4, 0u, 0u, 0u, 0u);
      tmem_wait_st();
    }
    if ((int64_t)blockIdx.x < total_tiles) stage(0, blockIdx.x);

    uint32_t it = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t ph = it & 1u;
      const int r = (int)(tile / p.tiles_per_req), n0 = (int)(tile % p.tiles_per_req) * 128;
      cp_async_wait_all();
      asm volatile("bar.sync 1, 256;" ::: "memory");     // this tile's rows are in shared memory
      if (tile + gridDim.x < total_tiles) stage(buf ^ 1, tile + gridDim.x);

      // ---- A1 = [q | q*his_sum | att | q-his_sum]; warpgroup h takes the 16-byte chunks c = h, h+2, ...
      if (ok) {
        const uint8_t* qrow = smem + G.o_q + buf * 128 * pitch + row * pitch;
        const uint8_t* arow = smem + G.o_att + buf * 128 * pitch + row * pitch;
        const float* hs = reinterpret_cast<const float*>(smem + G.o_hs) + buf * dp;
        for (int c = h; c < nch; c += 2) {
          const uint4 qc = *reinterpret_cast<const uint4*>(qrow + c * 16);
          const uint4 ac = *reinterpret_cast<const uint4*>(arow + c * 16);
          const __half2* qh = reinterpret_cast<const __half2*>(&qc);
          uint32_t pr[4], df[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 qf = __half22float2(qh[e]);
            const float h0 = hs[c * 8 + 2 * e], h1 = hs[c * 8 + 2 * e + 1];
            pr[e] = h2u(__floats2half2_rn(qf.x * h0, qf.y * h1));
            df[e] = h2u(__floats2half2_rn(qf.x - h0, qf.y - h1));
          }
          tmem_st4(a1t + 4 * c, qc.x, qc.y, qc.z, qc.w);
          tmem_st4(a1t + 4 * (nch + c), pr[0], pr[1], pr[2], pr[3]);
          tmem_st4(a1t + 4 * (2 * nch + c), ac.x, ac.y, ac.z, ac.w);
          tmem_st4(a1t + 4 * (3 * nch + c), df[0], df[1], df[2], df[3]);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(a1_full));
      }

      // ---- layer 1 epilogue: acc1 + partial -> Dice -> A2; warpgroup h takes blocks of 16 columns ----------
      // (a wait that ran out makes every later wait give up at once; the warps keep walking the tiles
      // without touching tensor memory so that nobody is left alone at a named barrier)
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc1_full), ph, 32));
      if (ok) {
        tc_fence_after_sync();
        const float* ps = reinterpret_cast<const float*>(smem + G.o_part) + buf * n1p;
        const int nb = n1p / 16, b_begin = h ? (nb + 1) / 2 : 0, b_end = h ? nb : (nb + 1) / 2;
        uint32_t va[16], vb[16];
        auto block = [&](int b, uint32_t (&cur)[16], uint32_t (&nxt)[16]) {
          tmem_wait_ld(cur);
          if (b + 1 < b_end) tmem_ld16_nowait(lane_addr + 16 * (b + 1), nxt);
          const float4* pp = reinterpret_cast<const float4*>(ps + 16 * b);
          const uint4* cc = c1 + 8 * b;
          uint32_t y[8], th[8];
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            const float4 pv = pp[e4];
            y[2 * e4] = h2u(__floats2half2_rn(__uint_as_float(cur[4 * e4]) + pv.x, __uint_as_float(cur[4 * e4 + 1]) + pv.y));
            y[2 * e4 + 1] = h2u(__floats2half2_rn(__uint_as_float(cur[4 * e4 + 2]) + pv.z, __uint_as_float(cur[4 * e4 + 3]) + pv.w));
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) th[e] = tanh_f16x2(h2u(__hfma2(u2h(y[e]), u2h(cc[e].x), u2h(cc[e].y))));
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = h2u(__hmul2(u2h(y[e]), __hfma2(u2h(th[e]), u2h(cc[e].w), u2h(cc[e].z))));
          tmem_st8(a2t + 8 * b, y);
        };
        if (b_begin < b_end) tmem_ld16_nowait(lane_addr + 16 * b_begin, va);
        for (int b = b_begin; b < b_end; b += 2) {
          block(b, va, vb);
          if (b + 1 < b_end) block(b + 1, vb, va);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(a2_full));
      }

      // ---- layer 2 epilogue: acc2 -> Dice -> layer 3 (fp32 dot products) -> softmax -> HBM ---------------------
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc2_full), ph, 33));
      float logit[TW_MAX_N3];
#pragma unroll
      for (int j = 0; j < TW_MAX_N3; ++j) logit[j] = 0.f;
      if (ok) {
        tc_fence_after_sync();
        const int nb = n2p / 16, b_begin = h ? (nb + 1) / 2 : 0, b_end = h ? nb : (nb + 1) / 2;
        uint32_t va[16], vb[16];
        auto block = [&](int b, uint32_t (&cur)[16], uint32_t (&nxt)[16]) {
          tmem_wait_ld(cur);
          if (b + 1 < b_end) tmem_ld16_nowait(lane_addr + G.c_acc2 + 16 * (b + 1), nxt);
          const uint4* cc = c2 + 8 * b;
          uint32_t y[8], th[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            y[e] = h2u(__floats2half2_rn(__uint_as_float(cur[2 * e]), __uint_as_float(cur[2 * e + 1])));
#pragma unroll
          for (int e = 0; e < 8; ++e) th[e] = tanh_f16x2(h2u(__hfma2(u2h(y[e]), u2h(cc[e].x), u2h(cc[e].y))));
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            // the layer output is an fp16 tensor in the model's graph: round, then feed layer 3 in fp32
            const float2 f = __half22float2(__hmul2(u2h(y[e]), __hfma2(u2h(th[e]), u2h(cc[e].w), u2h(cc[e].z))));
            const float* wr = w3 + (16 * b + 2 * e) * TW_MAX_N3;
#pragma unroll
            for (int j = 0; j < TW_MAX_N3; ++j)
              if (j < n3) logit[j] = fmaf(f.y, wr[TW_MAX_N3 + j], fmaf(f.x, wr[j], logit[j]));
          }
        };
        if (b_begin < b_end) tmem_ld16_nowait(lane_addr + G.c_acc2 + 16 * b_begin, va);
        for (int b = b_begin; b < b_end; b += 2) {
          block(b, va, vb);
          if (b + 1 < b_end) block(b + 1, vb, va);
        }
        tc_fence_before_sync();
      }
      if (h == 1) {
#pragma unroll
        for (int j = 0; j < TW_MAX_N3; ++j)
          if (j < n3) lg[row * TW_MAX_N3 + j] = logit[j];
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (h == 0 && ok) {
        const int n = n0 + row;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < TW_MAX_N3; ++j) {
          if (j < n3) {
            // layer-3 output rounded to the model's fp16, as the un-fused graph stores it
            logit[j] = __half2float(__float2half_rn(logit[j] + lg[row * TW_MAX_N3 + j] + b3[j]));
            mx = fmaxf(mx, logit[j]);
          }
        }
        if (p.softmax) {
          float sum = 0.f;
#pragma unroll
          for (int j = 0; j < TW_MAX_N3; ++j)
            if (j < n3) { logit[j] = __expf(logit[j] - mx); sum += logit[j]; }
          const float inv = 1.f / sum;
#pragma unroll
          for (int j = 0; j < TW_MAX_N3; ++j) logit[j] *= inv;
        }
        if (n < p.n_cand) {
          float* o = p.prob + ((int64_t)r * p.n_cand + n) * n3;
          if (n3 == 2) *reinterpret_cast<float2*>(o) = make_float2(logit[0], logit[1]);
          else {
#pragma unroll
            for (int j = 0; j < TW_MAX_N3; ++j)
              if (j < n3) o[j] = logit[j];
          }
        }
      }
    }
    cp_async_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == TW_MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem0, 512);
  }
}

bool tower_eligible(const xb_din_tower_args& a, int* why) {
  const TowerGeom g = tower_geom(a.d, a.n1, a.n2, a.n3);
  if (a.d > 64 || g.k1 > 256) { if (why) *why = 1; return false; }
  if (g.n1p > 256 || g.n2p > 128 || a.n3 < 1 || a.n3 > TW_MAX_N3) { if (why) *why = 2; return false; }
  if (g.cols > 512) { if (why) *why = 3; return false; }
  if (g.total > 220 * 1024) { if (why) *why = 4; return false; }
  return true;
}

void fill_params(TowerParams& p, const xb_din_tower_args& a) {
  memset(&p, 0, sizeof(p));
  p.user = (const __half*)a.user; p.ldu = a.ldu; p.q = (const __half*)a.q; p.ldq = a.ldq;
  p.k = (const __half*)a.k; p.ldk = a.ldk; p.att = (const __half*)a.att; p.ldatt = a.ldatt;
  p.prob = a.prob;
  p.requests = a.requests; p.n_cand = a.n_cand; p.T = a.T; p.d = a.d; p.du = a.du;
  p.n1 = a.n1; p.n2 = a.n2; p.n3 = a.n3; p.softmax = a.softmax;
  p.W1 = (const __half*)a.W1; p.b1 = a.b1; p.g1 = a.gamma1; p.m1 = a.mean1; p.v1 = a.var1;
  p.W2 = (const __half*)a.W2; p.b2 = a.b2; p.g2 = a.gamma2; p.m2 = a.mean2; p.v2 = a.var2;
  p.W3 = (const __half*)a.W3; p.b3 = a.b3;
  p.packed = (const uint8_t*)a.packed;
}

}  // namespace

int tower_status(int* out) { return umma::read_status_word(out); }
int tower_clear_status() { return umma::clear_status_word(); }
int tower_set_status_mirror(int* p) { return umma::set_status_mirror(p); }

}  // namespace xb

using namespace xb;

static int validate_tower(const xb_din_tower_args* a, const char* who) {
  XB_REQUIRE(a, XB_ERR_ARG, "%s: null arguments", who);
  XB_REQUIRE(a->d > 0 && a->du >= 0 && a->n1 > 0 && a->n2 > 0 && a->n3 > 0, XB_ERR_ARG, "%s: bad sizes", who);
  XB_REQUIRE(a->W1 && a->W2 && a->W3 && a->gamma1 && a->mean1 && a->var1 && a->gamma2 && a->mean2 && a->var2, XB_ERR_ARG,
             "%s: missing weights or Dice parameters", who);
  int why = 0;
  XB_REQUIRE(tower_eligible(*a, &why), XB_ERR_UNSUPPORTED, "%s: shape outside the fused tower kernel (reason %d)", who, why);
  return 0;
}

extern "C" size_t xb_din_tower_packed_bytes(int32_t d, int32_t n1, int32_t n2, int32_t n3) {
  if (d <= 0 || n1 <= 0 || n2 <= 0 || n3 <= 0) return 0;
  xb_din_tower_args a;
  memset(&a, 0, sizeof(a));
  a.d = d; a.n1 = n1; a.n2 = n2; a.n3 = n3;
  if (!tower_eligible(a, nullptr)) return 0;
  return (size_t)tower_geom(d, n1, n2, n3).image_bytes;
}

extern "C" size_t xb_din_tower_workspace_bytes(int32_t requests, int32_t d, int32_t n1) {
  if (requests <= 0 || d <= 0 || n1 <= 0) return 0;
  return ((size_t)requests * d * 4 + 255) / 256 * 256 + (size_t)requests * n1 * 4;
}

extern "C" int xb_din_tower_pack(const xb_din_tower_args* a, void* packed, size_t bytes, xb_stream_t stream) {
  if (int rc = validate_tower(a, "xb_din_tower_pack")) return rc;
  const size_t need = xb_din_tower_packed_bytes(a->d, a->n1, a->n2, a->n3);
  XB_REQUIRE(packed && bytes >= need && ((uintptr_t)packed & 15) == 0, XB_ERR_ARG,
             "xb_din_tower_pack: buffer of %zu bytes, need %zu, 16-byte aligned", bytes, need);
  TowerParams p;
  fill_params(p, *a);
  tower_pack_kernel<<<64, 256, 0, (cudaStream_t)stream>>>(p, (uint8_t*)packed);
  return check_launch("tower_pack_kernel");
}

extern "C" int xb_din_tower(const xb_din_tower_args* a, void* workspace, size_t workspace_bytes, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (int rc = validate_tower(a, "xb_din_tower")) return rc;
  XB_REQUIRE((a->user || a->du == 0) && a->q && a->k && a->att && a->prob && a->packed, XB_ERR_ARG,
             "xb_din_tower: null tensor");
  XB_REQUIRE(a->requests >= 0 && a->n_cand >= 0 && a->T >= 0, XB_ERR_ARG, "xb_din_tower: negative size");
  XB_REQUIRE(a->ldu >= a->du && a->ldq >= a->d && a->ldk >= a->d && a->ldatt >= a->d, XB_ERR_ARG,
             "xb_din_tower: leading dimension too small");
  XB_REQUIRE(a->du <= 4096, XB_ERR_LIMIT, "xb_din_tower: du <= 4096");
  if (a->requests == 0 || a->n_cand == 0) return 0;
  const size_t need = xb_din_tower_workspace_bytes(a->requests, a->d, a->n1);
  XB_REQUIRE(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0, XB_ERR_SCRATCH,
             "xb_din_tower: workspace of %zu bytes, need %zu, 16-byte aligned", workspace_bytes, need);
  TowerParams p;
  fill_params(p, *a);
  p.hs = (float*)workspace;
  p.partial = (float*)((char*)workspace + ((size_t)a->requests * a->d * 4 + 255) / 256 * 256);
  p.tiles_per_req = (a->n_cand + 127) / 128;
  const TowerGeom g = tower_geom(a->d, a->n1, a->n2, a->n3);
  p.idesc1 = umma::make_idesc(128, g.n1p, 0);
  p.idesc2 = umma::make_idesc(128, g.n2p, 0);
  XB_REQUIRE(a->requests <= 65535 * 32, XB_ERR_LIMIT, "xb_din_tower: too many requests per call");
  din_tower_partial_kernel<<<dim3(a->requests, (a->n1 + PT_COLS - 1) / PT_COLS), PT_COLS * PT_SLICES,
                             sizeof(float) * (9 * a->d + a->du + PT_COLS * PT_SLICES + 2), stream>>>(p);
  if (int rc = check_launch("din_tower_partial_kernel")) return rc;
  static PerDeviceOnce attr_set;
  XB_SET_MAX_SMEM_ONCE(attr_set, 220 * 1024, (const void*)din_tower_tc_kernel);
  const int64_t tiles = (int64_t)a->requests * p.tiles_per_req;
  const int grid = (int)std::min<int64_t>(tiles, sm_count());
  din_tower_tc_kernel<<<grid, TW_THREADS, g.total, stream>>>(p);
  return check_launch("din_tower_tc_kernel");
}
