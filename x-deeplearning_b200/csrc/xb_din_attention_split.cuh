// "Split" tcgen05 engine of the fused DIN attention unit (included by xb_din_attention.cu).
//
// The first layer of the scoring MLP is linear in x = [q, k, q-k, q*k], so for candidate n and step t
//   W0 x + b0 = (Wq + Wd) q_n  +  Wp (q_n * k_t)  +  [(Wk - Wd) k_t + b0]
// The last term does not depend on the candidate: it is computed once per request as a table V[t][.]
// and enters the MMA through a "selector" slot of the A operand (a column that is 1 for the slots's step
// and 0 otherwise, against a B row that holds V[t]). The per-step A operand then is [q | q*k_t | selector]:
// K = 2*dp (+16) instead of 4*dp + 16, i.e. half the MMA instructions and a third of the operand building
// of the per-step engine in xb_din_attention_tc.cuh, and its tensor-memory footprint leaves room for a
// third layer-1 accumulator, which takes the layer-1 MMAs off the activation warps' critical path.
//
// The kernel is persistent: a CTA walks a contiguous run of 128-candidate tiles. Weights, barriers and
// tensor memory are set up once per CTA, the per-request operands (k rows, V table, K^T) once per
// request, and the q rows of the next tile are fetched while the current one is computed.
//
// Roles (576 threads): warps 0-7 layer-1 activations (warpgroup b = steps of parity b), warps 8-15
// operand building two steps ahead + layer-2 activations (same split), warp 16 layer-1 MMAs, warp 17
// layer-2 MMAs and the closing S*K product. Step parity and accumulator numbers follow a step counter
// that runs across the tiles of a CTA, so the barriers never need re-initialising.
//
// Rounding differs from the per-step engine in where fp16 rounding happens (Wq + Wd and V[t] are rounded
// once each instead of q - k_t per element), not in the arithmetic.
#pragma once

namespace xb {
namespace {

constexpr int SP_THREADS = 576;
constexpr int SP_MMA1_WARP = 16, SP_MMA2_WARP = 17;

struct SpGeom {
  int dp, nch, spare, pad_mode, nsel, selpos, k1, nck, h0p, k2, h1p, np;
  // tensor-memory columns: [acc1 x nacc | acc2 x2 | A2 x2 | A1 x2]; accumulators start at multiples of 16
  int nacc, c_acc2, c_a2, c_a1, cols, tmem_cols;
  // packed image (bytes): Wqd chunk blocks, Wp chunk blocks, selector template block, W1 operand, c1, c2, WKD
  int blk, n_wqd, o_wqd, o_wp, o_selt, o_w1, o_c1, o_c2, o_wkd, image_bytes;
};

__host__ __device__ inline SpGeom sp_geom(int d, int h0, int h1) {
  SpGeom g;
  g.dp = (d + 7) / 8 * 8;
  g.nch = g.dp / 8;
  g.spare = g.dp - d;
  g.pad_mode = g.spare >= 4;                    // selector slots live in the padding of the q segment
  g.nsel = g.pad_mode ? 4 : 8;                  // steps that share one selector chunk
  g.selpos = g.pad_mode ? (d & 7) : 0;          // first selector half inside its chunk
  g.k1 = g.pad_mode ? 2 * g.dp : 2 * g.dp + 16;
  g.nck = g.k1 / 8;
  g.h0p = (h0 + 15) / 16 * 16;
  g.k2 = g.h0p + 16;                            // column h0p of A2 is constant 1 (carries b1)
  g.h1p = (h1 + 15) / 16 * 16;
  g.np = (g.dp + 15) / 16 * 16;
  const int per_parity = g.h1p + g.k2 / 2 + g.k1 / 2;
  g.nacc = (3 * g.h0p + 2 * per_parity <= 512) ? 3 : 2;
  g.c_acc2 = g.nacc * g.h0p;                    // + b * h1p
  g.c_a2 = g.c_acc2 + 2 * g.h1p;                // + b * k2 / 2
  g.c_a1 = g.c_a2 + g.k2;                       // + b * k1 / 2
  g.cols = g.c_a1 + g.k1;
  g.tmem_cols = g.cols <= 32 ? 32 : g.cols <= 64 ? 64 : g.cols <= 128 ? 128 : g.cols <= 256 ? 256 : 512;
  g.blk = g.h0p * 16;                           // one 8-wide k chunk of the layer-1 B operand
  g.n_wqd = g.pad_mode ? g.nch - 1 : g.nch;     // in pad mode the last q chunk is part of the selector block
  int off = 0;
  g.o_wqd = off; off += g.n_wqd * g.blk;
  g.o_wp = off; off += g.nch * g.blk;
  g.o_selt = off; off += g.blk;                 // constant halves of a selector block (pad mode), else zeros
  g.o_w1 = off; off += g.h1p * g.k2 * 2;
  g.o_c1 = off; off += (g.h0p / 2) * 16;
  g.o_c2 = off; off += (g.h1p / 2) * 16;
  g.o_wkd = off; off += (d + 1) * g.h0p * 4;    // fp32 [d + 1][h0p]: (Wk - Wd) by input, then b0
  g.image_bytes = (off + 15) / 16 * 16;
  return g;
}

// Shared memory of one CTA. The layer-1 B operand is a run of chunk blocks in ascending address order of the
// k chunk they serve (the MMA descriptor reaches the second chunk of a k step through a positive offset):
//   pad mode : [Wqd 0..nch-2][selector blocks 0..ngrp-1][Wp 0..nch-1]
//   otherwise: [Wqd 0..nch-1][Wp 0..nch-1][selector blocks 0..ngrp-1][zero block]
struct SpSmem {
  int ngrp, tp, o_b1, b1_blocks, o_w1, o_c1, o_c2, o_s, o_kt, o_kh, o_q, q_bytes, total;
};
__host__ __device__ inline SpSmem sp_smem(const SpGeom& g, int T) {
  SpSmem L;
  L.ngrp = (T + g.nsel - 1) / g.nsel;
  L.tp = (T + 15) / 16 * 16;
  int off = 0;
  L.o_b1 = off;
  L.b1_blocks = g.n_wqd + g.nch + L.ngrp + (g.pad_mode ? 0 : 1);
  off += L.b1_blocks * g.blk;
  L.o_w1 = off; off += g.h1p * g.k2 * 2;
  L.o_c1 = off; off += (g.h0p / 2) * 16;
  L.o_c2 = off; off += (g.h1p / 2) * 16;
  L.o_s = off; off += 128 * L.tp * 2;           // scores [128, tp], A operand of the closing product
  L.o_kt = off; off += g.np * L.tp * 2;         // K^T [np rows (feature), tp (step)], its B operand
  L.o_kh = off; off += T * g.dp * 2;            // k rows of the request
  off = (off + 15) / 16 * 16;
  L.q_bytes = 128 * g.dp * 2;
  L.o_q = off; off += 2 * L.q_bytes;            // q rows of this tile and of the next one, chunk-major
  L.total = off;
  return L;
}

// block index (inside the layer-1 B operand) of k chunk c for selector group grp
__device__ __forceinline__ int sp_chunk_block(const SpGeom& g, int ngrp, int c, int grp) {
  if (g.pad_mode) {
    if (c < g.nch - 1) return c;
    if (c == g.nch - 1) return g.nch - 1 + grp;
    return g.nch - 1 + ngrp + (c - g.nch);
  }
  if (c < 2 * g.nch) return c;
  if (c == 2 * g.nch) return 2 * g.nch + grp;
  return 2 * g.nch + ngrp;
}

template <int ACT>
__global__ void att_split_pack_kernel(const __grid_constant__ AttParams p, uint8_t* dst) {
  const SpGeom G = sp_geom(p.d, p.h0, p.h1);
  const int d = p.d, dp = G.dp, h0p = G.h0p, k2 = G.k2, h1p = G.h1p;
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
  const __half zero = __float2half(0.f);
  // W0 is [h0][4d] with the input segments q | k | q-k | q*k
  auto w0 = [&](int n, int seg, int i) { return __half2float(p.W0[(int64_t)n * 4 * d + seg * d + i]); };
  __half* wqd = reinterpret_cast<__half*>(dst + G.o_wqd);
  __half* wp = reinterpret_cast<__half*>(dst + G.o_wp);
  __half* selt = reinterpret_cast<__half*>(dst + G.o_selt);
  for (int idx = tid; idx < h0p * dp; idx += nth) {
    const int n = idx / dp, i = idx - n * dp;
    const bool live = n < p.h0 && i < d;
    const __half vq = live ? __float2half_rn(w0(n, 0, i) + w0(n, 2, i)) : zero;
    const __half vp = live ? p.W0[(int64_t)n * 4 * d + 3 * d + i] : zero;
    const int c = i >> 3, e = i & 7;
    if (c < G.n_wqd) wqd[c * (h0p * 8) + n * 8 + e] = vq;
    else selt[n * 8 + e] = vq;                  // pad mode: the last q chunk shares its block with the selector slots
    wp[c * (h0p * 8) + n * 8 + e] = vp;
  }
  if (!G.pad_mode)
    for (int idx = tid; idx < h0p * 8; idx += nth) selt[idx] = zero;
  __half* w1s = reinterpret_cast<__half*>(dst + G.o_w1);
  for (int idx = tid; idx < h1p * k2; idx += nth) {
    const int n = idx / k2, kk = idx - n * k2;
    __half v = zero;
    if (n < p.h1) {
      if (kk < p.h0) v = p.W1[(int64_t)n * p.h0 + kk];
      else if (kk == h0p) v = __float2half_rn(p.b1 ? p.b1[n] : 0.f);
    }
    w1s[(kk >> 3) * (h1p * 8) + n * 8 + (kk & 7)] = v;
  }
  uint4* c1 = reinterpret_cast<uint4*>(dst + G.o_c1);
  uint4* c2 = reinterpret_cast<uint4*>(dst + G.o_c2);
  for (int j = tid; j < h0p / 2; j += nth) {
    float A[2] = {0, 0}, B[2] = {0, 0}, C[2] = {0, 0}, D[2] = {0, 0};
    for (int u = 0; u < 2; ++u) {
      const int col = 2 * j + u;
      if (col >= p.h0) continue;
      if (ACT == XB_ACT_DICE) {
        const float rs = dice_rstd(p.v0[col], 0), g = p.g0[col];
        A[u] = 0.5f * rs; B[u] = -0.5f * p.m0[col] * rs; C[u] = 0.5f * (1.f + g); D[u] = 0.5f * (1.f - g);
      } else if (ACT == XB_ACT_SIGMOID) { A[u] = 0.5f; C[u] = 0.5f; D[u] = 0.5f; }
    }
    c1[j] = make_uint4(h2_bits(__floats2half2_rn(A[0], A[1])), h2_bits(__floats2half2_rn(B[0], B[1])),
                       h2_bits(__floats2half2_rn(C[0], C[1])), h2_bits(__floats2half2_rn(D[0], D[1])));
  }
  for (int j = tid; j < h1p / 2; j += nth) {
    float A[2] = {0, 0}, B[2] = {0, 0}, C[2] = {0, 0}, D[2] = {0, 0};
    for (int u = 0; u < 2; ++u) {
      const int col = 2 * j + u;
      if (col >= p.h1) continue;
      const float w2 = p.W2[col];
      if (ACT == XB_ACT_DICE) {
        const float rs = dice_rstd(p.v1[col], 0), g = p.g1[col];
        A[u] = 0.5f * rs; B[u] = -0.5f * p.m1[col] * rs; C[u] = 0.5f * (1.f + g) * w2; D[u] = 0.5f * (1.f - g) * w2;
      } else if (ACT == XB_ACT_SIGMOID) { A[u] = 0.5f; C[u] = 0.5f * w2; D[u] = 0.5f * w2; }
      else C[u] = w2;
    }
    c2[j] = make_uint4(h2_bits(__floats2half2_rn(A[0], A[1])), h2_bits(__floats2half2_rn(B[0], B[1])),
                       h2_bits(__floats2half2_rn(C[0], C[1])), h2_bits(__floats2half2_rn(D[0], D[1])));
  }
  float* wkd = reinterpret_cast<float*>(dst + G.o_wkd);
  for (int idx = tid; idx < (d + 1) * h0p; idx += nth) {
    const int i = idx / h0p, n = idx - i * h0p;
    float v = 0.f;
    if (n < p.h0) v = i < d ? w0(n, 1, i) - w0(n, 2, i) : (p.b0 ? p.b0[n] : 0.f);
    wkd[idx] = v;
  }
}

// NQ: compile-time bound of the 16-byte chunks of a q row (the row is kept in registers by the operand builders)
template <int ACT, int NQ>
__global__ void __launch_bounds__(SP_THREADS, 1) din_att_split_kernel(const __grid_constant__ AttParams p) {
  using namespace umma;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[20];
  __shared__ __align__(8) uint64_t dsc[10];       // layer-1 B descriptors per k step (selector group 0), then the group delta
  __shared__ uint32_t tmem_base_s;

  const SpGeom G = sp_geom(p.d, p.h0, p.h1);
  const SpSmem L = sp_smem(G, p.T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = p.d, dp = G.dp, nch = G.nch, h0p = G.h0p, k2 = G.k2, h1p = G.h1p, tp = L.tp, np = G.np;
  const int nacc = G.nacc;
  const uint8_t* image = reinterpret_cast<const uint8_t*>(p.packed);

  uint8_t* b1s = smem + L.o_b1;
  __half* w1s = reinterpret_cast<__half*>(smem + L.o_w1);
  uint4* c1 = reinterpret_cast<uint4*>(smem + L.o_c1);
  uint4* c2 = reinterpret_cast<uint4*>(smem + L.o_c2);
  __half* ss = reinterpret_cast<__half*>(smem + L.o_s);
  __half* kts = reinterpret_cast<__half*>(smem + L.o_kt);
  __half* khs = reinterpret_cast<__half*>(smem + L.o_kh);
  const __half zero = __float2half(0.f);

  const int64_t total_tiles = (int64_t)p.requests * p.tiles_per_req;
  const int64_t tile_first = (int64_t)blockIdx.x * p.tiles_per_cta;
  const int64_t tile_end = min(total_tiles, tile_first + p.tiles_per_cta);

  // ---- once per CTA: weight image, zero-initialised areas, barriers, tensor memory ---------------------
  {
    const int sel0 = (G.pad_mode ? G.n_wqd : G.n_wqd + nch) * G.blk;      // first selector block
    const int wp0 = (G.pad_mode ? G.n_wqd + L.ngrp : G.n_wqd) * G.blk;    // first Wp block
    for (int i = threadIdx.x; i < G.n_wqd * G.blk / 16; i += SP_THREADS) cp_async16(b1s + 16 * i, image + G.o_wqd + 16 * i);
    for (int i = threadIdx.x; i < nch * G.blk / 16; i += SP_THREADS) cp_async16(b1s + wp0 + 16 * i, image + G.o_wp + 16 * i);
    // every selector block starts as the template (the constant halves of pad mode, zeros otherwise)
    for (int i = threadIdx.x; i < L.ngrp * G.blk / 16; i += SP_THREADS)
      cp_async16(b1s + sel0 + 16 * i, image + G.o_selt + 16 * (i % (G.blk / 16)));
    const int n_rest = (G.h1p * G.k2 * 2 + (h0p / 2) * 16 + (h1p / 2) * 16) / 16;   // W1, c1, c2 are adjacent in both
    for (int i = threadIdx.x; i < n_rest; i += SP_THREADS) cp_async16(smem + L.o_w1 + 16 * i, image + G.o_w1 + 16 * i);
    cp_async_commit();
    if (!G.pad_mode)
      for (int i = threadIdx.x; i < G.blk / 16; i += SP_THREADS)
        reinterpret_cast<uint4*>(b1s + (2 * nch + L.ngrp) * G.blk)[i] = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < 128 * tp / 8; i += SP_THREADS) reinterpret_cast<uint4*>(ss)[i] = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < 2 * L.q_bytes / 16; i += SP_THREADS)
      reinterpret_cast<uint4*>(smem + L.o_q)[i] = make_uint4(0, 0, 0, 0);
  }
  // barriers (b = step parity, m = layer-1 accumulator number):
  //   a1_full[b]    4 builder warps   -> MMA1: A1 of a step is in tensor memory
  //   acc1_full[m]  tcgen05.commit    -> layer-1 warps and builders: layer-1 accumulator complete (A1 free again)
  //   acc1_free[m]  4 layer-1 warps   -> MMA1: accumulator drained
  //   a2_full[b]    4 layer-1 warps   -> MMA2: A2 written
  //   acc2_full[b]  tcgen05.commit    -> layer-2 warps (accumulator complete) and layer-1 warps (A2 free again)
  //   acc2_free[b]  4 layer-2 warps   -> MMA2: accumulator drained
  //   s_full        8 layer-2 warps   -> MMA2: all scores of the tile are in S;  acc3_full: closing product done
  uint64_t* a1_full = &bars[0];
  uint64_t* acc1_full = &bars[2];
  uint64_t* acc1_free = &bars[5];
  uint64_t* a2_full = &bars[8];
  uint64_t* acc2_full = &bars[10];
  uint64_t* acc2_free = &bars[12];
  uint64_t* s_full = &bars[14];
  uint64_t* acc3_full = &bars[15];
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&a1_full[b]), 4);
      mbar_init(smem_u32(&a2_full[b]), 4);
      mbar_init(smem_u32(&acc2_full[b]), 1);
      mbar_init(smem_u32(&acc2_free[b]), 4);
    }
    for (int m = 0; m < 3; ++m) {
      mbar_init(smem_u32(&acc1_full[m]), 1);
      mbar_init(smem_u32(&acc1_free[m]), 4);
    }
    mbar_init(smem_u32(s_full), 8);
    mbar_init(smem_u32(acc3_full), 1);
    fence_barrier_init();
  }
  if (warp == SP_MMA1_WARP) tmem_alloc(smem_u32(&tmem_base_s), (uint32_t)G.tmem_cols);
  cp_async_wait_all();
  fence_proxy_async_smem();          // the MMAs read these operands through the async proxy
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = tmem_base_s;

  const bool async8 = (d % 4 == 0) && (p.ldq % 4 == 0) && (p.ldk % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k)) & 7) == 0;
  // q rows of one tile into buffer `buf` (chunk-major, 16 bytes per row and chunk). Padding halves stay zero.
  auto fetch_q = [&](int64_t tile, int buf) {
    const int r = (int)(tile / p.tiles_per_req), tl_ = (int)(tile % p.tiles_per_req);
    const int rows = min(128, p.n_cand - tl_ * 128);
    __half* qs = reinterpret_cast<__half*>(smem + L.o_q + buf * L.q_bytes);
    const __half* qreq = p.q + ((int64_t)r * p.n_cand + tl_ * 128) * p.ldq;
    if (async8) {
      const int ppr = d / 4;
      for (int idx = threadIdx.x; idx < rows * ppr; idx += SP_THREADS) {
        const int row = idx / ppr, pc = idx - row * ppr;
        cp_async8(qs + ((pc >> 1) * 128 + row) * 8 + (pc & 1) * 4, qreq + (int64_t)row * p.ldq + pc * 4);
      }
    } else {
      for (int idx = threadIdx.x; idx < rows * d; idx += SP_THREADS) {
        const int row = idx / d, i = idx - row * d;
        qs[((i >> 3) * 128 + row) * 8 + (i & 7)] = qreq[(int64_t)row * p.ldq + i];
      }
    }
    // rows past the last candidate of the request (only its last tile has any)
    for (int idx = threadIdx.x; idx < (128 - rows) * nch; idx += SP_THREADS) {
      const int row = rows + idx / nch, c = idx % nch;
      *reinterpret_cast<uint4*>(qs + (c * 128 + row) * 8) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };

  if (tile_first < tile_end) fetch_q(tile_first, 0);

  // role-local state that lives across tiles
  uint32_t g0 = 0;                 // steps this CTA has run before the current tile
  int prev_r = -1;
  bool ok = true;                  // this warp's waits have all succeeded so far
  const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16);   // tensor-memory lane == candidate row
  if (warp >= 8 && warp < 16 && !G.pad_mode) {
    // the all-zero chunk after the selector chunk, both parities (its B block is zero too; this keeps NaN bit
    // patterns of uninitialised tensor memory out of the product)
    for (int b = 0; b < 2; ++b) tmem_st4(lane_addr + G.c_a1 + b * (G.k1 / 2) + 4 * (2 * nch + 1), 0u, 0u, 0u, 0u);
    tmem_wait_st();
  }
  if (warp < 8) {
    // columns h0p.. of A2: the constant 1 that carries bias b1, then zeros (fp16 pairs per 32-bit column)
    const uint32_t a2t = lane_addr + G.c_a2 + (warp >> 2) * (k2 / 2) + h0p / 2;
    tmem_st4(a2t, 0x00003C00u, 0u, 0u, 0u);
    tmem_st4(a2t + 4, 0u, 0u, 0u, 0u);
    tmem_wait_st();
  }

  uint32_t tile_it = 0;
  for (int64_t tile = tile_first; tile < tile_end; ++tile, ++tile_it) {
    const int r = (int)(tile / p.tiles_per_req), tile_in_req = (int)(tile % p.tiles_per_req);
    const int qbuf = tile_it & 1;
    int tl = p.seq_len ? p.seq_len[r] : p.T;
    tl = tl < 0 ? 0 : (tl > p.T ? p.T : tl);

    // ---- once per request: k rows, the V table inside the selector blocks, K^T ----------------------------
    if (r != prev_r) {
      const __half* kreq = p.k + (int64_t)r * p.T * p.ldk;
      if (async8) {
        const int ppr = d / 4;
        for (int idx = threadIdx.x; idx < p.T * ppr; idx += SP_THREADS) {
          const int t = idx / ppr, pc = idx - t * ppr;
          cp_async8(khs + t * dp + pc * 4, kreq + (int64_t)t * p.ldk + pc * 4);
        }
        for (int idx = threadIdx.x; idx < p.T * G.spare; idx += SP_THREADS) khs[(idx / G.spare) * dp + d + idx % G.spare] = zero;
      } else {
        for (int idx = threadIdx.x; idx < p.T * dp; idx += SP_THREADS) {
          const int t = idx / dp, i = idx - t * dp;
          khs[idx] = (i < d) ? kreq[(int64_t)t * p.ldk + i] : zero;
        }
      }
      cp_async_commit();
      cp_async_wait_all();                       // (also completes this tile's q rows)
      __syncthreads();
      // V[t][n] = b0[n] + sum_i (Wk - Wd)[n][i] * k_t[i], fp32, rounded once to fp16 into its selector slot
      const float* wkd = reinterpret_cast<const float*>(image + G.o_wkd);
      const int sel0 = (G.pad_mode ? G.n_wqd : G.n_wqd + nch) * G.blk;
      for (int idx = threadIdx.x; idx < L.ngrp * G.nsel * h0p; idx += SP_THREADS) {
        const int t = idx / h0p, n = idx - t * h0p;
        float v = 0.f;
        if (t < p.T && n < p.h0) {
          v = __ldg(wkd + d * h0p + n);
          const __half2* kt2 = reinterpret_cast<const __half2*>(khs + t * dp);
          for (int i = 0; 2 * i < d; ++i) {
            const float2 kk = __half22float2(kt2[i]);
            v = fmaf(kk.x, __ldg(wkd + (2 * i) * h0p + n), v);
            if (2 * i + 1 < d) v = fmaf(kk.y, __ldg(wkd + (2 * i + 1) * h0p + n), v);
          }
        }
        __half* blk = reinterpret_cast<__half*>(b1s + sel0 + (t / G.nsel) * G.blk);
        blk[n * 8 + G.selpos + (t % G.nsel)] = __float2half_rn(v);
      }
      for (int idx = threadIdx.x; idx < np * tp; idx += SP_THREADS) {
        const int t = idx / np, e = idx - t * np;
        const __half v = (e < d && t < tl) ? khs[t * dp + e] : zero;
        kts[(t >> 3) * (np * 8) + e * 8 + (t & 7)] = v;
      }
      // score columns this request does not write: zero, so that nothing an earlier request left there meets K^T
      if (tile_it > 0)
        for (int idx = threadIdx.x; idx < 128 * (tp - tl); idx += SP_THREADS) {
          const int rw = idx / (tp - tl), t = tl + idx % (tp - tl);
          ss[(t >> 3) * (128 * 8) + rw * 8 + (t & 7)] = zero;
        }
      fence_proxy_async_smem();                  // MMA operands written through the generic proxy
      prev_r = r;
    } else {
      cp_async_wait_all();                       // this tile's q rows
    }
    __syncthreads();
    if (tile + 1 < tile_end) fetch_q(tile + 1, qbuf ^ 1);     // lands while this tile is computed

    const __half* qs = reinterpret_cast<const __half*>(smem + L.o_q + qbuf * L.q_bytes);

    if (warp == SP_MMA1_WARP) {
      // ---- layer-1 MMA issue ----------------------------------------------------------------------------------
      if (lane == 0 && ok) {
        uint32_t m = g0 % (uint32_t)nacc, u = g0 / (uint32_t)nacc;
        const uint32_t b1_addr = smem_u32(b1s);
        // B descriptors of the k steps for selector group 0; only the k step that holds the selector chunk moves
        // with the group (its start address or its chunk distance changes by one block per group)
        const int nks = G.nck / 2;
        const int sel_ks = (G.pad_mode ? nch - 1 : 2 * nch) / 2;
        if (tile_it == 0) {
          uint64_t sel_delta = 0;
          for (int ks = 0; ks < nks; ++ks) {
            const uint32_t o0 = (uint32_t)sp_chunk_block(G, L.ngrp, 2 * ks, 0) * G.blk;
            const uint32_t o1 = (uint32_t)sp_chunk_block(G, L.ngrp, 2 * ks + 1, 0) * G.blk;
            dsc[ks] = make_desc_interleaved(b1_addr + o0, o1 - o0, 128);
            if (ks == sel_ks && L.ngrp > 1) {
              const uint32_t p0 = (uint32_t)sp_chunk_block(G, L.ngrp, 2 * ks, 1) * G.blk;
              const uint32_t p1 = (uint32_t)sp_chunk_block(G, L.ngrp, 2 * ks + 1, 1) * G.blk;
              sel_delta = make_desc_interleaved(b1_addr + p0, p1 - p0, 128) - dsc[ks];
            }
          }
          dsc[9] = sel_delta;
        }
        const uint64_t sel_delta = dsc[9];
        int grp = 0, in_grp = 0;
        for (int j = 0; j < tl; ++j) {
          const uint32_t g = g0 + j;
          const int b = g & 1;
          ok = mbar_wait(smem_u32(&a1_full[b]), (g >> 1) & 1u, 10) &&
               (u == 0 || mbar_wait(smem_u32(&acc1_free[m]), (u - 1) & 1u, 14));
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t ta = tmem0 + G.c_a1 + b * (G.k1 / 2);
          const uint32_t acc1 = tmem0 + m * h0p;
          const uint64_t dsel = dsc[sel_ks] + (uint64_t)grp * sel_delta;
          for (int ks = 0; ks < nks; ++ks)
            mma_f16_ts(acc1, ta + 8 * ks, ks == sel_ks ? dsel : dsc[ks], p.idesc1, ks > 0 ? 1u : 0u);
          mma_commit(smem_u32(&acc1_full[m]));
          if (++m == (uint32_t)nacc) { m = 0; ++u; }
          if (++in_grp == G.nsel) { in_grp = 0; ++grp; }
        }
      }
    } else if (warp == SP_MMA2_WARP) {
      // ---- layer-2 MMA issue, then the closing S*K product -------------------------------------------------
      if (lane == 0 && ok) {
        const uint64_t db0 = make_desc_interleaved(smem_u32(w1s), h1p * 16, 128);
        const uint64_t db_step = (uint64_t)((2 * h1p * 16) >> 4), da_step = (uint64_t)((2 * 128 * 16) >> 4);
        for (int j = 0; j < tl; ++j) {
          const uint32_t g = g0 + j;
          const int b = g & 1;
          const uint32_t ph = (g >> 1) & 1u;
          ok = mbar_wait(smem_u32(&a2_full[b]), ph, 11) && mbar_wait(smem_u32(&acc2_free[b]), ph ^ 1u, 13);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t ta = tmem0 + G.c_a2 + b * (k2 / 2);
          uint64_t db = db0;
          const uint32_t acc2 = tmem0 + G.c_acc2 + b * h1p;
          mma_f16_ts(acc2, ta, db, p.idesc2, 0u);
          for (int ks = 1; ks < k2 / 16; ++ks) {
            ta += 8; db += db_step;
            mma_f16_ts(acc2, ta, db, p.idesc2, 1u);
          }
          mma_commit(smem_u32(&acc2_full[b]));
        }
        // weighted sum over the steps: out = S * K, into the columns of layer-1 accumulator 0 (idle by now)
        if (ok && (ok = mbar_wait(smem_u32(s_full), tile_it & 1u, 12))) {
          tc_fence_after_sync();
          uint64_t da = make_desc_interleaved(smem_u32(ss), 128 * 16, 128);
          uint64_t db = make_desc_interleaved(smem_u32(kts), np * 16, 128);
          const uint64_t db3 = (uint64_t)((2 * np * 16) >> 4);
          for (int ks = 0; ks < tp / 16; ++ks) {
            mma_f16_ss(tmem0, da, db, p.idesc3, ks > 0 ? 1u : 0u);
            da += da_step; db += db3;
          }
          mma_commit(smem_u32(acc3_full));
        }
      }
    } else if (warp < 8) {
      // ---- layer-1 warpgroups: acc1 -> activation -> A2, for the steps whose counter has parity wb --------
      const int wb = warp >> 2;
      const uint32_t a2t = lane_addr + G.c_a2 + wb * (k2 / 2);
      const int j0 = (int)((wb - g0) & 1u);
      uint32_t m = (g0 + j0) % (uint32_t)nacc, u = (g0 + j0) / (uint32_t)nacc;
      for (int j = j0; j < tl && ok; j += 2) {
        const uint32_t g = g0 + j;
        const uint32_t ph = (g >> 1) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc1_full[m]), u & 1u, 20));
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc1 = lane_addr + m * h0p;
        const int nblk = h0p / 16;
        uint32_t va[16], vb[16];
        auto block = [&](int blk, uint32_t (&cur)[16], uint32_t (&nxt)[16]) {
          tmem_wait_ld(cur);
          if (blk + 1 < nblk) tmem_ld16_nowait(acc1 + 16 * (blk + 1), nxt);
          uint32_t y[8];
          pair_l1_block<ACT>(cur, c1 + 8 * blk, y);
          if (blk == 0) {
            // A2 of this parity is free once the layer-2 MMA two steps back has read it
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc2_full[wb]), ph ^ 1u, 23));
            if (ok) tc_fence_after_sync();
          }
          if (ok) tmem_st8(a2t + 8 * blk, y);
        };
        tmem_ld16_nowait(acc1, va);
        for (int blk = 0; blk < nblk && ok; blk += 2) {
          block(blk, va, vb);
          if (blk + 1 < nblk && ok) block(blk + 1, vb, va);
        }
        if (!ok) break;
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&acc1_free[m]));
          mbar_arrive(smem_u32(&a2_full[wb]));
        }
        // the next step of this parity uses the accumulator two further on
        m += 2; if (m >= (uint32_t)nacc) { m -= nacc; ++u; }
      }
    } else {
      // ---- builder / layer-2 warpgroups ----------------------------------------------------------------------------
      const int wb = (warp >> 2) & 1;
      const int row = (warp & 3) * 32 + lane;
      const int n = tile_in_req * 128 + row;
      const bool valid = n < p.n_cand;
      const uint32_t a1t = lane_addr + G.c_a1 + wb * (G.k1 / 2);
      const int j0 = (int)((wb - g0) & 1u);

      // q row as 16-byte chunks (nch <= NQ), padding halves zero
      uint4 qv[NQ];
#pragma unroll
      for (int c = 0; c < NQ; ++c)
        qv[c] = c < nch ? *reinterpret_cast<const uint4*>(qs + (c * 128 + row) * 8) : make_uint4(0, 0, 0, 0);
      if (ok) {
#pragma unroll
        for (int c = 0; c < NQ; ++c)
          if (c < nch) tmem_st4(a1t + 4 * c, qv[c].x, qv[c].y, qv[c].z, qv[c].w);
        tmem_wait_st();
      }
      // the selector chunk of step j: a 1 in the half that belongs to step j % nsel
      const int sel_chunk = G.pad_mode ? nch - 1 : 2 * nch;
      // (in pad mode that chunk also holds the last q halves; read with a runtime index, nch is not a constant)
      const uint4 last = G.pad_mode ? *reinterpret_cast<const uint4*>(qs + ((nch - 1) * 128 + row) * 8) : make_uint4(0, 0, 0, 0);
      const uint32_t selbase[4] = {last.x, last.y, last.z, last.w};
      auto build_a1 = [&](int j) {
        const uint4* kt = reinterpret_cast<const uint4*>(khs + j * dp);
#pragma unroll
        for (int c = 0; c < NQ; ++c) {
          if (c < nch) {
            const uint4 kc = kt[c];
            const __half2* kh = reinterpret_cast<const __half2*>(&kc);
            const __half2* qh = reinterpret_cast<const __half2*>(&qv[c]);
            uint4 pr;
            __half2* ph2 = reinterpret_cast<__half2*>(&pr);
#pragma unroll
            for (int e = 0; e < 4; ++e) ph2[e] = __hmul2(qh[e], kh[e]);
            tmem_st4(a1t + 4 * (nch + c), pr.x, pr.y, pr.z, pr.w);
          }
        }
        const int hpos = G.selpos + (j % G.nsel);
        const uint32_t one = 0x3C00u << ((hpos & 1) * 16);
        const int reg = hpos >> 1;
        tmem_st4(a1t + 4 * sel_chunk, selbase[0] | (reg == 0 ? one : 0u), selbase[1] | (reg == 1 ? one : 0u),
                 selbase[2] | (reg == 2 ? one : 0u), selbase[3] | (reg == 3 ? one : 0u));
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&a1_full[wb]));
      };

      const int npairs2 = (p.h1 + 1) / 2;
      uint32_t m = (g0 + j0) % (uint32_t)nacc, u = (g0 + j0) / (uint32_t)nacc;
      if (ok && j0 < tl) build_a1(j0);
      for (int j = j0; j < tl && ok; j += 2) {
        const uint32_t g = g0 + j;
        const uint32_t ph = (g >> 1) & 1u;
        if (j + 2 < tl) {
          // A1 of this parity is free once the layer-1 MMA of step j has read it
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc1_full[m]), u & 1u, 24));
          if (!ok) break;
          build_a1(j + 2);
        }
        m += 2; if (m >= (uint32_t)nacc) { m -= nacc; ++u; }
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc2_full[wb]), ph, 21));
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc2 = lane_addr + G.c_acc2 + wb * h1p;
        __half2 part[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) part[e] = __floats2half2_rn(0.f, 0.f);
        for (int c = 0; c < h1p; c += 16) {
          uint32_t v[16];
          tmem_ld16_nowait(acc2 + c, v);
          tmem_wait_ld(v);
          const uint4* __restrict__ cc = c2 + (c >> 1);
          uint32_t x[8], th[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            x[e] = h2_bits(__floats2half2_rn(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1])));
          if (ACT == XB_ACT_NONE) {
#pragma unroll
            for (int e = 0; e < 8; ++e) part[e & 3] = __hfma2(bits_h2(x[e]), bits_h2(cc[e].z), part[e & 3]);
          } else {
            const int live = npairs2 - (c >> 1);           // column pairs of this block that are not padding
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (e < live) th[e] = h2_bits(__hfma2(bits_h2(x[e]), bits_h2(cc[e].x), bits_h2(cc[e].y)));
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (e < live) th[e] = tanh_f16x2(th[e]);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              if (e < live) {
                const __half2 gg = __hfma2(bits_h2(th[e]), bits_h2(cc[e].w), bits_h2(cc[e].z));
                part[e & 3] = ACT == XB_ACT_DICE ? __hfma2(bits_h2(x[e]), gg, part[e & 3]) : __hadd2(part[e & 3], gg);
              }
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&acc2_free[wb]));
        // short fp16 chains (h1p/8 terms each), combined in fp32
        const float2 f0 = __half22float2(part[0]), f1 = __half22float2(part[1]);
        const float2 f2 = __half22float2(part[2]), f3 = __half22float2(part[3]);
        const float s = p.b2 + ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        if (p.scores && valid && !p.use_softmax) p.scores[((int64_t)r * p.n_cand + n) * p.T + j] = s;
        ss[(j >> 3) * (128 * 8) + row * 8 + (j & 7)] = __float2half_rn(s);
      }

      if (p.use_softmax) asm volatile("bar.sync 1, 256;" ::: "memory");     // both parities' scores are in S
      if (p.use_softmax && wb == 0) {
        // masked softmax over the steps, in place on this thread's row of S (steps >= tl are masked out)
        float mx = -INFINITY;
        for (int t = 0; t < tl; ++t) mx = fmaxf(mx, __half2float(ss[(t >> 3) * (128 * 8) + row * 8 + (t & 7)]));
        float l = 0.f;
        for (int t = 0; t < tl; ++t) l += __expf(__half2float(ss[(t >> 3) * (128 * 8) + row * 8 + (t & 7)]) - mx);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        for (int t = 0; t < tl; ++t) {
          __half* e = &ss[(t >> 3) * (128 * 8) + row * 8 + (t & 7)];
          *e = __float2half_rn(__expf(__half2float(*e) - mx) * inv);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(s_full));

      if (wb == 0) {
        ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(acc3_full), tile_it & 1u, 22));
        tc_fence_after_sync();
        if (ok) {
          __half* o = p.out + ((int64_t)r * p.n_cand + n) * p.ldo;
          for (int c = 0; c < np; c += 16) {
            float v[16];
            tmem_ld16(lane_addr + c, v);
            if (valid) {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                if (c + e < d) o[c + e] = __float2half_rn(v[e]);
            }
          }
        }
      }
    }

    g0 += (uint32_t)tl;
    // end of tile: the closing product has been read out, every accumulator and operand buffer is idle, and S
    // and the other q buffer may be overwritten
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
  }

  cp_async_wait_all();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == SP_MMA1_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem0, (uint32_t)G.tmem_cols);
  }
}

bool split_eligible(const xb_din_att_args& a, int* why) {
  const SpGeom g = sp_geom(a.d, a.h0, a.h1);
  if (g.dp > 64) { if (why) *why = 1; return false; }
  if (g.h0p > 128 || g.h1p > 64) { if (why) *why = 2; return false; }
  // very short behaviour lists (fewer steps than two selector groups) stay on the per-step engine: one such
  // shape (T = 3) raised an illegal-instruction error on this engine and the cause has not been found
  if (a.T > 256 || a.T < 2 * g.nsel) { if (why) *why = 5; return false; }
  if (g.cols > 512 || g.np > g.h0p) { if (why) *why = 6; return false; }
  if (sp_smem(g, a.T).total > 220 * 1024) { if (why) *why = 3; return false; }
  if (a.use_softmax && a.scores) { if (why) *why = 4; return false; }   // normalised scores are not written out
  return true;
}

bool split_eligible_shape(int d, int h0, int h1) {
  xb_din_att_args a;
  memset(&a, 0, sizeof(a));
  a.d = d; a.h0 = h0; a.h1 = h1; a.T = 16;
  return split_eligible(a, nullptr);
}

size_t att_split_packed_bytes(int d, int h0, int h1) { return (size_t)sp_geom(d, h0, h1).image_bytes; }

int launch_att_split_pack(const AttParams& p, int act, void* dst, cudaStream_t stream) {
  if (act == XB_ACT_DICE) att_split_pack_kernel<XB_ACT_DICE><<<8, 256, 0, stream>>>(p, (uint8_t*)dst);
  else if (act == XB_ACT_SIGMOID) att_split_pack_kernel<XB_ACT_SIGMOID><<<8, 256, 0, stream>>>(p, (uint8_t*)dst);
  else att_split_pack_kernel<XB_ACT_NONE><<<8, 256, 0, stream>>>(p, (uint8_t*)dst);
  return check_launch("att_split_pack_kernel");
}

template <int NQ>
int launch_split_nq(const AttParams& p, int act, unsigned ctas, int smem, cudaStream_t stream) {
  static PerDeviceOnce attr_set;
  XB_SET_MAX_SMEM_ONCE(attr_set, 220 * 1024, (const void*)din_att_split_kernel<XB_ACT_NONE, NQ>,
                       (const void*)din_att_split_kernel<XB_ACT_SIGMOID, NQ>, (const void*)din_att_split_kernel<XB_ACT_DICE, NQ>);
  if (act == XB_ACT_DICE) din_att_split_kernel<XB_ACT_DICE, NQ><<<ctas, SP_THREADS, smem, stream>>>(p);
  else if (act == XB_ACT_SIGMOID) din_att_split_kernel<XB_ACT_SIGMOID, NQ><<<ctas, SP_THREADS, smem, stream>>>(p);
  else din_att_split_kernel<XB_ACT_NONE, NQ><<<ctas, SP_THREADS, smem, stream>>>(p);
  return check_launch("din_att_split_kernel");
}

int launch_att_split(AttParams& p, const xb_din_att_args& a, cudaStream_t stream) {
  const SpGeom g = sp_geom(a.d, a.h0, a.h1);
  const SpSmem L = sp_smem(g, a.T);
  p.tiles_per_req = (a.n_cand + 127) / 128;
  p.idesc1 = umma::make_idesc(128, g.h0p, 0);
  p.idesc2 = umma::make_idesc(128, g.h1p, 0);
  p.idesc3 = umma::make_idesc(128, g.np, 0);
  const int64_t tiles = (int64_t)a.requests * p.tiles_per_req;
  XB_REQUIRE(tiles < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_din_attention: too many tiles");
  // contiguous runs of tiles per CTA (a run mostly stays inside one request, whose operands are then built once)
  const int64_t ctas0 = std::min<int64_t>(tiles, sm_count());
  p.tiles_per_cta = (int)((tiles + ctas0 - 1) / ctas0);
  const int64_t ctas = (tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
  if (g.nch <= 3) return launch_split_nq<3>(p, a.act, (unsigned)ctas, L.total, stream);
  if (g.nch <= 5) return launch_split_nq<5>(p, a.act, (unsigned)ctas, L.total, stream);
  return launch_split_nq<8>(p, a.act, (unsigned)ctas, L.total, stream);
}

}  // namespace
}  // namespace xb
