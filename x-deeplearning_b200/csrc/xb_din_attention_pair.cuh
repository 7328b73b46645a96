// Step-pair tcgen05 engine of the fused DIN attention unit (included by xb_din_attention.cu).
//
// Layer 1 of the unit, x = [q, k_t, q-k_t, q*k_t] times W0 = [Wq; Wk; Wd; Wp], is regrouped as
//     x W0 = q (Wq + Wd + diag(k_t) Wp) + [b0 + k_t (Wk - Wd)]
// so that the operand which changes with the step is the small weight matrix
//     B_t[n][i] = (Wq + Wd)[i][n] + k_t[i] Wp[i][n]   (i < d),     B_t[n][d] = b0[n] + k_t (Wk - Wd)[.][n]
// and the candidate rows q (with a constant-1 column at index d) are a fixed A operand for the whole
// tile. Two steps then share one MMA: their B_t are stacked along N (N = 2*h0p), so a pair of steps
// costs kq/16 instructions instead of 2*k1/16, and nothing has to be built per candidate row.
// Layer 2, the activations and the closing S*K product are those of the per-step engine
// (xb_din_attention_tc.cuh): A2 lives in tensor memory, Dice / sigmoid on fp16 pairs.
//
//   builders : B of the pair P+1 = [B_2P+2 ; B_2P+3] into shared memory (half a pair per warpgroup)
//   MMA      : acc1[pair buffer][128 x 2*h0p] = q * B^T                 (A and B from shared memory)
//   workers  : columns [b*h0p, (b+1)*h0p) of acc1 -> activation -> A2[b] (tensor memory), b = step parity
//   MMA      : acc2[b][128 x h1p] = A2[b] * W1^T
//   workers  : acc2[b] -> activation, dot with W2 -> score -> column of S
// The regrouping changes where fp16 rounding happens (Wq + Wd and B_t are rounded once each instead of
// q - k_t and q * k_t), not the arithmetic.
#pragma once

namespace xb {
namespace {

constexpr int PAIR_THREADS = 640;        // 4 worker warpgroups, 2 MMA-issuing warps, 2 B-building warps
constexpr int MMA1_WARP = 16, MMA2_WARP = 17;
constexpr int BUILD_WARP0 = 18;

struct PairGeom {
  int dp, nb, kq, ones, h0p, n2, k2, h1p, tp, np;
  int c_acc2, c_a2, cols;                       // tensor memory: [acc1 x2 | acc2 x2 | A2 x2]
  // packed image: W1 operand, c1, c2, WQ, WP (fp16 [h0p][kq]), WKD (fp32 [d][h0p], b0 in row d)
  int o_w1, o_c1, o_c2, o_wq, o_wp, o_wkd, image_bytes;
  int o_s, o_kt, o_kh, o_q, o_kw, o_b, total;
};

__host__ __device__ inline PairGeom pair_geom(int d, int h0, int h1, int T) {
  PairGeom g;
  g.dp = (d + 7) / 8 * 8;
  g.nb = (d + 1 + 7) / 8;                       // 16-byte chunks of a B row that change with the step
  g.kq = (8 * g.nb + 15) / 16 * 16;
  g.ones = d;                                   // column of q that is constant 1
  g.h0p = (h0 + 15) / 16 * 16;
  g.n2 = 2 * g.h0p;
  g.k2 = g.h0p + 16;                            // column h0p of A2 is constant 1
  g.h1p = (h1 + 15) / 16 * 16;
  g.tp = (T + 15) / 16 * 16;
  g.np = (g.dp + 15) / 16 * 16;
  g.c_acc2 = 2 * g.n2;
  g.c_a2 = g.c_acc2 + 2 * g.h1p;
  g.cols = g.c_a2 + g.k2;                       // two A2 buffers of k2/2 columns each
  int off = 0;
  g.o_w1 = off; off += g.h1p * g.k2 * 2;
  g.o_c1 = off; off += (g.h0p / 2) * 16;
  g.o_c2 = off; off += (g.h1p / 2) * 16;
  g.o_wq = off; off += g.h0p * g.kq * 2;
  g.o_wp = off; off += g.h0p * g.kq * 2;
  g.o_wkd = off; off += (d + 1) * g.h0p * 4;
  off = (off + 15) / 16 * 16;
  g.image_bytes = off;
  g.o_s = off; off += 128 * g.tp * 2;
  g.o_kt = off; off += g.np * g.tp * 2;
  g.o_kh = off; off += T * g.dp * 2;
  off = (off + 15) / 16 * 16;
  g.o_q = off; off += 128 * g.kq * 2;
  g.o_kw = off; off += ((T * g.h0p * 2 + 15) / 16) * 16;     // KW[t][n], fp16
  g.o_b = off; off += 2 * g.n2 * g.kq * 2;                     // two pair operands
  g.total = off;
  return g;
}

bool pair_eligible(const xb_din_att_args& a, int* why) {
  const PairGeom g = pair_geom(a.d, a.h0, a.h1, a.T);
  if (a.d > 63 || g.kq > 64) { if (why) *why = 11; return false; }
  if (g.n2 > 256 || g.h1p > 64) { if (why) *why = 12; return false; }
  if (g.cols > TMEM_COLS || g.np > g.n2) { if (why) *why = 13; return false; }
  if (g.tp > 256) { if (why) *why = 15; return false; }
  if (g.total > 220 * 1024) { if (why) *why = 14; return false; }
  if (a.use_softmax && a.scores) { if (why) *why = 4; return false; }
  if (a.w.packed == nullptr) { if (why) *why = 16; return false; }     // this engine only runs from a packed image
  return true;
}

// whether xb_din_attention_pack appends this engine's image (a property of the weights' shape alone)
bool pair_image_wanted(int d, int h0, int h1) {
  const PairGeom g = pair_geom(d, h0, h1, 16);
  return d <= 63 && g.kq <= 64 && g.n2 <= 256 && g.h1p <= 64 && g.cols <= TMEM_COLS && g.np <= g.n2;
}

template <int ACT>
__global__ void att_pair_pack_kernel(const __grid_constant__ AttParams p, uint8_t* dst) {
  const PairGeom G = pair_geom(p.d, p.h0, p.h1, p.T);
  const int d = p.d, h0p = G.h0p, h1p = G.h1p, k2 = G.k2, kq = G.kq;
  const __half zero = __float2half(0.f);
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
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
  // W0 arrives K-major [h0][4d]: segments q, k, q-k, q*k
  __half* wq = reinterpret_cast<__half*>(dst + G.o_wq);
  __half* wp = reinterpret_cast<__half*>(dst + G.o_wp);
  for (int idx = tid; idx < h0p * kq; idx += nth) {
    const int n = idx / kq, i = idx - n * kq;
    float a = 0.f, b = 0.f;
    if (n < p.h0 && i < d) {
      const __half* row = p.W0 + (int64_t)n * 4 * d;
      a = __half2float(row[i]) + __half2float(row[2 * d + i]);
      b = __half2float(row[3 * d + i]);
    }
    wq[idx] = __float2half_rn(a);
    wp[idx] = __float2half_rn(b);
  }
  float* wkd = reinterpret_cast<float*>(dst + G.o_wkd);
  for (int idx = tid; idx < (d + 1) * h0p; idx += nth) {
    const int i = idx / h0p, n = idx - i * h0p;
    float v = 0.f;
    if (n < p.h0) {
      if (i < d) {
        const __half* row = p.W0 + (int64_t)n * 4 * d;
        v = __half2float(row[d + i]) - __half2float(row[2 * d + i]);
      } else {
        v = p.b0 ? p.b0[n] : 0.f;
      }
    }
    wkd[idx] = v;
  }
  if (blockIdx.x == 0) {
    uint4* c1 = reinterpret_cast<uint4*>(dst + G.o_c1);
    uint4* c2 = reinterpret_cast<uint4*>(dst + G.o_c2);
    for (int j = threadIdx.x; j < h0p / 2; j += blockDim.x) {
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
    for (int j = threadIdx.x; j < h1p / 2; j += blockDim.x) {
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
  }
}

template <int ACT>
__global__ void __launch_bounds__(PAIR_THREADS, 1) din_att_pair_kernel(const __grid_constant__ AttParams p) {
  using namespace umma;
  using umma::tanh_f16x2;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[14];
  __shared__ uint32_t tmem_base_s;

  const PairGeom G = pair_geom(p.d, p.h0, p.h1, p.T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x / p.tiles_per_req, tile = blockIdx.x % p.tiles_per_req;
  const int d = p.d, dp = G.dp, nb = G.nb, kq = G.kq, h0p = G.h0p, n2 = G.n2, k2 = G.k2, h1p = G.h1p, tp = G.tp, np = G.np;
  int tl = p.seq_len ? p.seq_len[r] : p.T;
  tl = tl < 0 ? 0 : (tl > p.T ? p.T : tl);
  const int n_pairs = (tl + 1) >> 1;

  __half* w1s = reinterpret_cast<__half*>(smem + G.o_w1);
  uint4* c1 = reinterpret_cast<uint4*>(smem + G.o_c1);
  uint4* c2 = reinterpret_cast<uint4*>(smem + G.o_c2);
  const __half* wqs = reinterpret_cast<const __half*>(smem + G.o_wq);
  const __half* wps = reinterpret_cast<const __half*>(smem + G.o_wp);
  const float* wkd = reinterpret_cast<const float*>(smem + G.o_wkd);
  __half* ss = reinterpret_cast<__half*>(smem + G.o_s);
  __half* kts = reinterpret_cast<__half*>(smem + G.o_kt);
  __half* khs = reinterpret_cast<__half*>(smem + G.o_kh);
  __half* qs = reinterpret_cast<__half*>(smem + G.o_q);
  __half* kws = reinterpret_cast<__half*>(smem + G.o_kw);
  uint8_t* bop = smem + G.o_b;
  const __half zero = __float2half(0.f), one = __float2half(1.f);

  // ---- prologue ------------------------------------------------------------------------------------
  const bool async8 = (d % 4 == 0) && (p.ldq % 4 == 0) && (p.ldk % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k)) & 7) == 0;
  {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.packed);
    for (int i = threadIdx.x; i < G.image_bytes / 16; i += PAIR_THREADS) cp_async16(smem + 16 * i, src + 16 * i);
  }
  if (async8) {
    const int ppr = d / 4;                                   // 8-byte pieces per row
    const __half* kreq = p.k + (int64_t)r * p.T * p.ldk;
    for (int idx = threadIdx.x; idx < p.T * ppr; idx += PAIR_THREADS) {
      const int t = idx / ppr, pc = idx - t * ppr;
      cp_async8(khs + t * dp + pc * 4, kreq + (int64_t)t * p.ldk + pc * 4);
    }
    const int rows = min(128, p.n_cand - tile * 128);
    const __half* qreq = p.q + ((int64_t)r * p.n_cand + tile * 128) * p.ldq;
    for (int idx = threadIdx.x; idx < rows * ppr; idx += PAIR_THREADS) {
      const int row = idx / ppr, pc = idx - row * ppr;
      cp_async8(qs + ((pc >> 1) * 128 + row) * 8 + (pc & 1) * 4, qreq + (int64_t)row * p.ldq + pc * 4);
    }
  }
  cp_async_commit();
  // what no copy writes: padding columns, rows past the last candidate, the constant-1 column, S, B padding
  for (int idx = threadIdx.x; idx < 128 * kq; idx += PAIR_THREADS) {
    const int row = idx / kq, i = idx - row * kq;
    const bool have = i < d && tile * 128 + row < p.n_cand;
    __half* dst = &qs[(i >> 3) * (128 * 8) + row * 8 + (i & 7)];
    if (!async8) *dst = have ? p.q[((int64_t)r * p.n_cand + tile * 128 + row) * p.ldq + i] : (i == G.ones ? one : zero);
    else if (!have) *dst = (i == G.ones) ? one : zero;
  }
  for (int idx = threadIdx.x; idx < p.T * dp; idx += PAIR_THREADS) {
    const int t = idx / dp, i = idx - t * dp;
    if (!async8) khs[idx] = (i < d) ? p.k[((int64_t)r * p.T + t) * p.ldk + i] : zero;
    else if (i >= d) khs[idx] = zero;
  }
  for (int idx = threadIdx.x; idx < 128 * tp / 8; idx += PAIR_THREADS)
    reinterpret_cast<uint4*>(ss)[idx] = make_uint4(0, 0, 0, 0);
  for (int idx = threadIdx.x; idx < 2 * n2 * kq * 2 / 16; idx += PAIR_THREADS)
    reinterpret_cast<uint4*>(bop)[idx] = make_uint4(0, 0, 0, 0);
  cp_async_wait_all();
  __syncthreads();
  // K^T operand of the closing product and the per-step constant row KW[t][n] = b0[n] + k_t (Wk - Wd)[.][n]
  for (int idx = threadIdx.x; idx < np * tp; idx += PAIR_THREADS) {
    const int t = idx / np, e = idx - t * np;
    const __half v = (e < d && t < tl) ? khs[t * dp + e] : zero;
    kts[(t >> 3) * (np * 8) + e * 8 + (t & 7)] = v;
  }
  for (int idx = threadIdx.x; idx < tl * h0p; idx += PAIR_THREADS) {
    const int t = idx / h0p, n = idx - t * h0p;
    float acc = wkd[d * h0p + n];
    const __half* kt = khs + t * dp;
    for (int i = 0; i < d; ++i) acc = fmaf(__half2float(kt[i]), wkd[i * h0p + n], acc);
    kws[idx] = __float2half_rn(acc);
  }

  // barriers; pb = pair & 1, b = step & 1
  //   b_full[pb]    2 builder warps -> layer-1 MMA warp: B of a pair is in shared memory
  //   acc1_full[pb] tcgen05.commit  -> layer-1 warpgroups (accumulator complete), builders (B consumed)
  //   acc1_free[pb] 8 layer-1 warps -> layer-1 MMA warp: accumulator is in registers
  //   a2_full[b]    4 layer-1 warps -> layer-2 MMA warp
  //   acc2_full[b]  tcgen05.commit  -> layer-2 warpgroup (accumulator complete), layer-1 warpgroup (A2 consumed)
  //   acc2_free[b]  4 layer-2 warps -> layer-2 MMA warp
  //   s_full, acc3_full: the closing S*K product
  uint64_t* b_full = &bars[0];
  uint64_t* acc1_full = &bars[2];
  uint64_t* acc1_free = &bars[4];
  uint64_t* a2_full = &bars[6];
  uint64_t* acc2_full = &bars[8];
  uint64_t* acc2_free = &bars[10];
  uint64_t* s_full = &bars[12];
  uint64_t* acc3_full = &bars[13];
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&b_full[b]), 2);
      mbar_init(smem_u32(&acc1_full[b]), 1);
      mbar_init(smem_u32(&acc1_free[b]), 8);
      mbar_init(smem_u32(&a2_full[b]), 4);
      mbar_init(smem_u32(&acc2_full[b]), 1);
      mbar_init(smem_u32(&acc2_free[b]), 4);
    }
    mbar_init(smem_u32(s_full), 8);
    mbar_init(smem_u32(acc3_full), 1);
    fence_barrier_init();
  }
  if (warp == MMA1_WARP) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = tmem_base_s;

  if (warp == MMA1_WARP) {
    // ---- layer-1 MMA issue: one product per pair of steps, N = 2*h0p ---------------------------------------
    if (lane == 0) {
      const int nks = kq / 16;
      const uint64_t da0 = make_desc_interleaved(smem_u32(qs), 128 * 16, 128);
      const uint64_t da_step = (uint64_t)((2 * 128 * 16) >> 4), db_step = (uint64_t)((2 * n2 * 16) >> 4);
      for (int P = 0; P < n_pairs; ++P) {
        const int pb = P & 1;
        const uint32_t ph = (uint32_t)(P >> 1) & 1u;
        if (!(mbar_wait(smem_u32(&b_full[pb]), ph, 10) && mbar_wait(smem_u32(&acc1_free[pb]), ph ^ 1u, 14))) break;
        tc_fence_after_sync();
        uint64_t da = da0;
        uint64_t db = make_desc_interleaved(smem_u32(bop + pb * (n2 * kq * 2)), n2 * 16, 128);
        const uint32_t acc1 = tmem0 + pb * n2;
        mma_f16_ss(acc1, da, db, p.idesc1, 0u);
        for (int ks = 1; ks < nks; ++ks) {
          da += da_step; db += db_step;
          mma_f16_ss(acc1, da, db, p.idesc1, 1u);
        }
        mma_commit(smem_u32(&acc1_full[pb]));
      }
    }
  } else if (warp == MMA2_WARP) {
    // ---- layer-2 MMA issue per step, then the closing S*K product ----------------------------------------
    if (lane == 0) {
      const uint64_t db0 = make_desc_interleaved(smem_u32(w1s), h1p * 16, 128);
      const uint64_t db_step = (uint64_t)((2 * h1p * 16) >> 4), da_step = (uint64_t)((2 * 128 * 16) >> 4);
      const int nks = k2 / 16;
      bool ok = true;
      for (int j = 0; j < tl; ++j) {
        const int b = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        ok = mbar_wait(smem_u32(&a2_full[b]), ph, 11) && mbar_wait(smem_u32(&acc2_free[b]), ph ^ 1u, 13);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t ta = tmem0 + G.c_a2 + b * (k2 / 2);
        uint64_t db = db0;
        const uint32_t acc2 = tmem0 + G.c_acc2 + b * h1p;
        mma_f16_ts(acc2, ta, db, p.idesc2, 0u);
        for (int ks = 1; ks < nks; ++ks) {
          ta += 8; db += db_step;
          mma_f16_ts(acc2, ta, db, p.idesc2, 1u);
        }
        mma_commit(smem_u32(&acc2_full[b]));
      }
      // weighted sum over the steps: out = S * K; every earlier MMA has completed once all scores are written
      if (ok && mbar_wait(smem_u32(s_full), 0, 12)) {
        tc_fence_after_sync();
        uint64_t da = make_desc_interleaved(smem_u32(ss), 128 * 16, 128);
        uint64_t db = make_desc_interleaved(smem_u32(kts), np * 16, 128);
        const uint64_t db3 = (uint64_t)((2 * np * 16) >> 4);
        for (int ks = 0; ks < tp / 16; ++ks) {
          mma_f16_ss(tmem0, da, db, p.idesc3, ks > 0 ? 1u : 0u);
          da += da_step; db += db3;
        }
      }
      mma_commit(smem_u32(acc3_full));
    }
  } else if (warp >= BUILD_WARP0) {
    // ---- B builders: warp hb lays out B_t of the step of parity hb for every pair, one pair ahead of the MMA:
    //      B_t[n][8c..8c+8) = (Wq+Wd)[n] chunk + k_t chunk * Wp[n] chunk, the constant-1 column gets KW[t][n] --------
    const int hb = warp - BUILD_WARP0;
    const int oc = G.ones >> 3, oe = G.ones & 7;               // chunk and slot of the constant-1 column
    const uint32_t sh = (uint32_t)(oe & 1) * 16u, keep = ~(0xFFFFu << sh);
    const int ow = oe >> 1;
    for (int P = 0; P < n_pairs; ++P) {
      const int pb = P & 1;
      // the pair buffer is free once the MMA of pair P-2 has read it
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&acc1_full[pb]), (uint32_t)((P - 2) >> 1) & 1u, 24))) break;
      const int t = 2 * P + hb;
      if (t < tl) {
        uint8_t* dstb = bop + pb * (n2 * kq * 2) + (hb * h0p) * 16;
        const uint4* kt = reinterpret_cast<const uint4*>(khs + t * dp);
        const __half* kwt = kws + t * h0p;
        // chunk by chunk: the lanes take consecutive rows (up to 4 x 32), so the k_t chunk is one broadcast
        // read, the stores are contiguous and only the chunk with the constant-1 column pays for KW
        for (int c = 0; c < nb; ++c) {
          uint4 kc = make_uint4(0, 0, 0, 0);
          if (c * 8 < dp) kc = kt[c];
          uint4 wq[4], wp[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int nn = lane + 32 * u;
            if (nn < h0p) {
              wq[u] = *reinterpret_cast<const uint4*>(wqs + nn * kq + c * 8);
              wp[u] = *reinterpret_cast<const uint4*>(wps + nn * kq + c * 8);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int nn = lane + 32 * u;
            if (nn < h0p) {
              uint4 o;
              o.x = h2_bits(__hfma2(bits_h2(kc.x), bits_h2(wp[u].x), bits_h2(wq[u].x)));
              o.y = h2_bits(__hfma2(bits_h2(kc.y), bits_h2(wp[u].y), bits_h2(wq[u].y)));
              o.z = h2_bits(__hfma2(bits_h2(kc.z), bits_h2(wp[u].z), bits_h2(wq[u].z)));
              o.w = h2_bits(__hfma2(bits_h2(kc.w), bits_h2(wp[u].w), bits_h2(wq[u].w)));
              if (c == oc) {
                const uint32_t kwb = (uint32_t)__half_as_ushort(kwt[nn]) << sh;
                o.x = ow == 0 ? (o.x & keep) | kwb : o.x;
                o.y = ow == 1 ? (o.y & keep) | kwb : o.y;
                o.z = ow == 2 ? (o.z & keep) | kwb : o.z;
                o.w = ow == 3 ? (o.w & keep) | kwb : o.w;
              }
              *reinterpret_cast<uint4*>(dstb + c * (n2 * 16) + nn * 16) = o;
            }
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&b_full[pb]));
    }
  } else if (warp < 8) {
    // ---- layer-1 warpgroups: half b of the pair accumulator -> activation -> A2[b] -------------------------
    const int wb = warp >> 2, b = wb;
    const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16);   // TMEM lane == candidate row of the tile
    const uint32_t a2t = lane_addr + G.c_a2 + b * (k2 / 2);
    tmem_st4(a2t + h0p / 2, 0x00003C00u, 0u, 0u, 0u);        // column h0p: the constant 1 that carries b1
    tmem_st4(a2t + h0p / 2 + 4, 0u, 0u, 0u, 0u);
    tmem_wait_st();
    bool ok = true;
    for (int j = wb; j < tl; j += 2) {
      const int P = j >> 1, pb = P & 1;
      const uint32_t php = (uint32_t)(P >> 1) & 1u, phs = (uint32_t)P & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc1_full[pb]), php, 20));
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t acc1 = lane_addr + pb * n2 + b * h0p;
      // blocks of 16 columns (8 fp16 pairs); the load of the next block is in flight while this one is
      // converted, activated and stored
      const int nblk = h0p / 16;
      uint32_t va[16], vb[16];
      auto block = [&](int blk, uint32_t (&cur)[16], uint32_t (&nxt)[16]) {
        tmem_wait_ld(cur);
        if (blk + 1 < nblk) tmem_ld16_nowait(acc1 + 16 * (blk + 1), nxt);
        else {
          // the whole half is in registers: the pair accumulator goes back once both halves say so
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&acc1_free[pb]));
        }
        uint32_t y[8];
        pair_l1_block<ACT>(cur, c1 + 8 * blk, y);
        if (blk == 0) {
          // A2[b] is free once the layer-2 MMA of step j-2 has read it: waited for here, after the first block's
          // arithmetic, so that that MMA overlaps the start of this step
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc2_full[b]), phs ^ 1u, 23));
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
      if (lane == 0) mbar_arrive(smem_u32(&a2_full[b]));        // one arrival per warp
    }
    // (with an odd number of steps the last pair is drained by warpgroup 0 alone; nobody waits for that)
  } else if (warp < 16) {
    // ---- layer-2 warpgroups: acc2[b] -> activation -> score -> column of S ----------------------------------
    const int wb = (warp >> 2) & 1, b = wb;
    const int row = (warp & 3) * 32 + lane;
    const int n = tile * 128 + row;
    const bool valid = n < p.n_cand;
    const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16);
    bool ok = true;
    const int npairs2 = (p.h1 + 1) / 2;
    for (int j = wb; j < tl; j += 2) {
      const int P = j >> 1;
      const uint32_t ph = (uint32_t)P & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc2_full[b]), ph, 21));
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t acc2 = lane_addr + G.c_acc2 + b * h1p;
      __half2 part[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) part[e] = __floats2half2_rn(0.f, 0.f);
      // blocks of 16 columns; the next block's load is in flight while this one is activated
      const int nblk2 = h1p / 16;
      uint32_t va[16], vb[16];
      auto block2 = [&](int blk, uint32_t (&v)[16], uint32_t (&nxt)[16]) {
        tmem_wait_ld(v);
        if (blk + 1 < nblk2) tmem_ld16_nowait(acc2 + 16 * (blk + 1), nxt);
        else {
          tc_fence_before_sync();                  // the accumulator is in registers
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&acc2_free[b]));
        }
        const uint4* __restrict__ cc = c2 + 8 * blk;
        uint32_t x[8], th[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
          x[e] = h2_bits(__floats2half2_rn(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1])));
        if (ACT == XB_ACT_NONE) {
#pragma unroll
          for (int e = 0; e < 8; ++e) part[e & 3] = __hfma2(bits_h2(x[e]), bits_h2(cc[e].z), part[e & 3]);
        } else {
          const int live = npairs2 - 8 * blk;            // column pairs of this block that are not padding
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (e < live) th[e] = tanh_f16x2(h2_bits(__hfma2(bits_h2(x[e]), bits_h2(cc[e].x), bits_h2(cc[e].y))));
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if (e < live) {
              const __half2 g = __hfma2(bits_h2(th[e]), bits_h2(cc[e].w), bits_h2(cc[e].z));
              part[e & 3] = ACT == XB_ACT_DICE ? __hfma2(bits_h2(x[e]), g, part[e & 3]) : __hadd2(part[e & 3], g);
            }
          }
        }
      };
      tmem_ld16_nowait(acc2, va);
      for (int blk = 0; blk < nblk2; blk += 2) {
        block2(blk, va, vb);
        if (blk + 1 < nblk2) block2(blk + 1, vb, va);
      }
      const float2 f0 = __half22float2(part[0]), f1 = __half22float2(part[1]);
      const float2 f2 = __half22float2(part[2]), f3 = __half22float2(part[3]);
      const float s = p.b2 + ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
      if (p.scores && valid && !p.use_softmax) p.scores[((int64_t)r * p.n_cand + n) * p.T + j] = s;
      ss[(j >> 3) * (128 * 8) + row * 8 + (j & 7)] = __float2half_rn(s);
    }

    if (p.use_softmax) asm volatile("bar.sync 1, 256;" ::: "memory");     // both parities' scores are in S
    if (p.use_softmax && wb == 0) {
      float m = -INFINITY;
      for (int t = 0; t < tl; ++t) m = fmaxf(m, __half2float(ss[(t >> 3) * (128 * 8) + row * 8 + (t & 7)]));
      float l = 0.f;
      for (int t = 0; t < tl; ++t) l += __expf(__half2float(ss[(t >> 3) * (128 * 8) + row * 8 + (t & 7)]) - m);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      for (int t = 0; t < tl; ++t) {
        __half* e = &ss[(t >> 3) * (128 * 8) + row * 8 + (t & 7)];
        *e = __float2half_rn(__expf(__half2float(*e) - m) * inv);
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(s_full));

    if (wb == 0) ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(acc3_full), 0, 22));
    tc_fence_after_sync();
    if (ok && wb == 0) {
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

  tc_fence_before_sync();
  __syncthreads();
  if (warp == MMA1_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem0, TMEM_COLS);
  }
}

size_t att_pair_packed_bytes(int d, int h0, int h1) { return (size_t)pair_geom(d, h0, h1, 16).image_bytes; }

int launch_att_pair_pack(const AttParams& p, int act, void* dst, cudaStream_t stream) {
  if (act == XB_ACT_DICE) att_pair_pack_kernel<XB_ACT_DICE><<<8, 256, 0, stream>>>(p, (uint8_t*)dst);
  else if (act == XB_ACT_SIGMOID) att_pair_pack_kernel<XB_ACT_SIGMOID><<<8, 256, 0, stream>>>(p, (uint8_t*)dst);
  else att_pair_pack_kernel<XB_ACT_NONE><<<8, 256, 0, stream>>>(p, (uint8_t*)dst);
  return check_launch("att_pair_pack_kernel");
}

int launch_att_pair(AttParams& p, const xb_din_att_args& a, cudaStream_t stream) {
  const PairGeom g = pair_geom(a.d, a.h0, a.h1, a.T);
  p.tiles_per_req = (a.n_cand + 127) / 128;
  p.idesc1 = umma::make_idesc(128, g.n2, 0);
  p.idesc2 = umma::make_idesc(128, g.h1p, 0);
  p.idesc3 = umma::make_idesc(128, g.np, 0);
  static PerDeviceOnce attr_set;
  XB_SET_MAX_SMEM_ONCE(attr_set, 220 * 1024, (const void*)din_att_pair_kernel<XB_ACT_NONE>,
                       (const void*)din_att_pair_kernel<XB_ACT_SIGMOID>, (const void*)din_att_pair_kernel<XB_ACT_DICE>);
  const int64_t blocks = (int64_t)a.requests * p.tiles_per_req;
  XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_din_attention: too many tiles");
  if (a.act == XB_ACT_DICE) din_att_pair_kernel<XB_ACT_DICE><<<(unsigned)blocks, PAIR_THREADS, g.total, stream>>>(p);
  else if (a.act == XB_ACT_SIGMOID) din_att_pair_kernel<XB_ACT_SIGMOID><<<(unsigned)blocks, PAIR_THREADS, g.total, stream>>>(p);
  else din_att_pair_kernel<XB_ACT_NONE><<<(unsigned)blocks, PAIR_THREADS, g.total, stream>>>(p);
  return check_launch("din_att_pair_kernel");
}

}  // namespace
}  // namespace xb
