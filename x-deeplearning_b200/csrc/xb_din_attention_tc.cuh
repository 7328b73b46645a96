// tcgen05 engine of the fused DIN attention unit (included by xb_din_attention.cu).
//
// One CTA owns 128 candidates of one request and walks the behaviour steps.
// Two worker warpgroups (one candidate row per thread) take alternate steps; a
// ninth warp issues every MMA, so the tensor pipe runs one warpgroup's step
// while the other warpgroup does its activations:
//   worker: A1 = [q|k_t|q-k_t|q*k_t] (fp16, 128 x k1) into shared memory
//   MMA   : acc1[128 x h0p] = A1 * W0^T                  (TMEM accumulator)
//   worker: acc1 -> activation -> fp16 A2 in shared memory
//   MMA   : acc2[128 x h1p] = A2 * W1^T
//   worker: acc2 -> activation, dot with W2 -> score s[n,t] -> fp16 column t of S
// and, after the last step,
//   MMA   : out[128 x d] = S[128 x T] * K[T x d]          (the weighted sum is a GEMM too)
//
// Biases ride in the MMAs: A1 carries a constant-1 column (a padding column of
// the q segment when d is not a multiple of 8) whose W0 row is b0, and A2 has
// 16 extra columns, the first constant 1 with W1 row b1.
//
// Activations run on packed fp16 pairs with one SFU instruction per pair:
//   sigmoid(z) = 1/2 + 1/2 tanh(z/2), so Dice(x) = x * (C + D*tanh(A*x + B)) with
//   A = rstd/2, B = -mean*rstd/2, C = (1+gamma)/2, D = (1-gamma)/2 per column.
//
// Shared-memory operands use the un-swizzled K-major core-matrix layout: the
// 16-byte chunk c (8 consecutive k) of row r sits at c*(rows*16) + r*16, so the
// 32 rows a warp writes for one chunk are 512 contiguous bytes, the
// descriptor's leading-dimension offset is rows*16 and its stride offset 128.
#pragma once

namespace xb {
namespace {

constexpr int TC_THREADS = 288;          // 2 worker warpgroups + 1 MMA warp
constexpr int TMEM_COLS = 512;
constexpr int ACC1_COL = 0, ACC2_COL = 128, ACC3_COL = 192, WG_COL = 256;

struct TcGeom {
  int dp, nch, k1, ones1, h0p, k2, h1p, tp, np;
};

__host__ __device__ inline TcGeom tc_geom(int d, int h0, int h1, int T) {
  TcGeom g;
  g.dp = (d + 7) / 8 * 8;
  g.nch = g.dp / 8;
  g.ones1 = (d < g.dp) ? d : 4 * g.dp;               // column of A1 that is constant 1
  g.k1 = 4 * g.dp + ((d < g.dp) ? 0 : 16);
  g.h0p = (h0 + 15) / 16 * 16;
  g.k2 = g.h0p + 16;                                 // column h0p of A2 is constant 1
  g.h1p = (h1 + 15) / 16 * 16;
  g.tp = (T + 15) / 16 * 16;
  g.np = (g.dp + 15) / 16 * 16;
  return g;
}

struct TcSmemLayout {
  int w0, w1, a1, a2, s, kt, kh, c1, c2, total;
};
__host__ __device__ inline TcSmemLayout tc_layout(const TcGeom& g, int T) {
  TcSmemLayout L;
  int off = 0;
  L.w0 = off; off += g.h0p * g.k1 * 2;          // W0 operand [h0p rows, k1]
  L.w1 = off; off += g.h1p * g.k2 * 2;          // W1 operand [h1p rows, k2]
  L.a1 = off; off += 2 * 128 * g.k1 * 2;        // A1, one buffer per warpgroup
  L.a2 = off; off += 2 * 128 * g.k2 * 2;        // A2, one buffer per warpgroup
  L.s = off; off += 128 * g.tp * 2;             // scores [128, tp]
  L.kt = off; off += g.np * g.tp * 2;           // K^T operand [np rows (feature), tp (step)]
  L.kh = off; off += T * g.dp * 2;              // k rows for building A1
  off = (off + 15) / 16 * 16;
  L.c1 = off; off += (g.h0p / 2) * 16;          // per column pair: A, B, C, D as half2
  L.c2 = off; off += (g.h1p / 2) * 16;
  L.total = off;
  return L;
}

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// activation of a pair of pre-activations x (fp16 pair) with constants c = {A,B,C,D}
template <int ACT>
__device__ __forceinline__ __half2 act_pair(__half2 x, const uint4& c) {
  if (ACT == XB_ACT_NONE) return x;
  const __half2 t = __hfma2(x, bits_h2(c.x), bits_h2(c.y));
  const __half2 th = bits_h2(umma::tanh_f16x2(h2_bits(t)));
  const __half2 g = __hfma2(th, bits_h2(c.w), bits_h2(c.z));
  return ACT == XB_ACT_DICE ? __hmul2(x, g) : g;
}

// same, times the output-layer weight (folded into C and D; for ACT_NONE C holds the weight)
template <int ACT>
__device__ __forceinline__ __half2 act_pair_w(__half2 x, const uint4& c) {
  if (ACT == XB_ACT_NONE) return __hmul2(x, bits_h2(c.z));
  return act_pair<ACT>(x, c);
}

template <int ACT>
__global__ void __launch_bounds__(TC_THREADS, 1) din_att_tc_kernel(const __grid_constant__ AttParams p) {
  using namespace umma;
  extern __shared__ __align__(128) uint8_t smem[];
  // [wg][a1_full, acc1_full, a2_full, acc2_full], then s_full, acc3_full
  __shared__ __align__(8) uint64_t bars[10];
  __shared__ uint32_t tmem_base_s;

  const TcGeom G = tc_geom(p.d, p.h0, p.h1, p.T);
  const TcSmemLayout L = tc_layout(G, p.T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x / p.tiles_per_req, tile = blockIdx.x % p.tiles_per_req;
  const int d = p.d, dp = G.dp, nch = G.nch, k1 = G.k1, h0p = G.h0p, k2 = G.k2, h1p = G.h1p, tp = G.tp, np = G.np;
  int tl = p.seq_len ? p.seq_len[r] : p.T;
  tl = tl < 0 ? 0 : (tl > p.T ? p.T : tl);

  __half* w0s = reinterpret_cast<__half*>(smem + L.w0);
  __half* w1s = reinterpret_cast<__half*>(smem + L.w1);
  __half* ss = reinterpret_cast<__half*>(smem + L.s);
  __half* kts = reinterpret_cast<__half*>(smem + L.kt);
  __half* khs = reinterpret_cast<__half*>(smem + L.kh);
  uint4* c1 = reinterpret_cast<uint4*>(smem + L.c1);
  uint4* c2 = reinterpret_cast<uint4*>(smem + L.c2);
  const __half zero = __float2half(0.f), one = __float2half(1.f);

  // ---- prologue: operands that stay resident for the whole tile ----------------------------
  for (int idx = threadIdx.x; idx < h0p * k1; idx += TC_THREADS) {
    const int n = idx / k1, kk = idx - n * k1;
    __half v = zero;
    if (n < p.h0) {
      if (kk == G.ones1) v = __float2half_rn(p.b0 ? p.b0[n] : 0.f);
      else if (kk < 4 * dp) {
        const int seg = kk / dp, i = kk - seg * dp;
        if (i < d) v = p.W0[(int64_t)n * 4 * d + seg * d + i];
      }
    }
    w0s[(kk >> 3) * (h0p * 8) + n * 8 + (kk & 7)] = v;
  }
  for (int idx = threadIdx.x; idx < h1p * k2; idx += TC_THREADS) {
    const int n = idx / k2, kk = idx - n * k2;
    __half v = zero;
    if (n < p.h1) {
      if (kk < p.h0) v = p.W1[(int64_t)n * p.h0 + kk];
      else if (kk == h0p) v = __float2half_rn(p.b1 ? p.b1[n] : 0.f);
    }
    w1s[(kk >> 3) * (h1p * 8) + n * 8 + (kk & 7)] = v;
  }
  for (int idx = threadIdx.x; idx < p.T * dp; idx += TC_THREADS) {
    const int t = idx / dp, i = idx - t * dp;
    khs[idx] = (i < d) ? p.k[((int64_t)r * p.T + t) * p.ldk + i] : zero;
  }
  for (int idx = threadIdx.x; idx < np * tp; idx += TC_THREADS) {
    const int e = idx / tp, t = idx - e * tp;
    const __half v = (e < d && t < tl) ? p.k[((int64_t)r * p.T + t) * p.ldk + e] : zero;
    kts[(t >> 3) * (np * 8) + e * 8 + (t & 7)] = v;
  }
  for (int idx = threadIdx.x; idx < 128 * tp / 8; idx += TC_THREADS)
    reinterpret_cast<uint4*>(ss)[idx] = make_uint4(0, 0, 0, 0);
  for (int j = threadIdx.x; j < h0p / 2; j += TC_THREADS) {
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
  for (int j = threadIdx.x; j < h1p / 2; j += TC_THREADS) {
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
  if (threadIdx.x == 0) {
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&bars[4 * g + 0]), 128);
      mbar_init(smem_u32(&bars[4 * g + 1]), 1);
      mbar_init(smem_u32(&bars[4 * g + 2]), 128);
      mbar_init(smem_u32(&bars[4 * g + 3]), 1);
    }
    mbar_init(smem_u32(&bars[8]), 256);
    mbar_init(smem_u32(&bars[9]), 1);
    fence_barrier_init();
  }
  if (warp == 8) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
  fence_proxy_async_smem();          // operands were written through the generic proxy
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = tmem_base_s;

  if (warp == 8) {
    // ---- MMA issue --------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t w0a = smem_u32(w0s), w1a = smem_u32(w1s);
      bool ok = true;
      for (int t = 0; t <= tl && ok; ++t) {
        if (t < tl) {
          const int g = t & 1, i = t >> 1;
          ok = mbar_wait(smem_u32(&bars[4 * g + 0]), (uint32_t)i & 1u, 10);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a1 = smem_u32(smem + L.a1 + g * (128 * k1 * 2));
          const uint32_t acc1 = tmem0 + g * WG_COL + ACC1_COL;
          for (int ks = 0; ks < k1 / 16; ++ks) {
            const uint64_t da = make_desc_interleaved(a1 + ks * 2 * (128 * 16), 128 * 16, 128);
            const uint64_t db = make_desc_interleaved(w0a + ks * 2 * (h0p * 16), h0p * 16, 128);
            mma_f16_ss(acc1, da, db, p.idesc1, ks > 0 ? 1u : 0u);
          }
          mma_commit(smem_u32(&bars[4 * g + 1]));
        }
        if (t > 0) {
          const int tt = t - 1, g = tt & 1, i = tt >> 1;
          ok = mbar_wait(smem_u32(&bars[4 * g + 2]), (uint32_t)i & 1u, 11);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a2 = smem_u32(smem + L.a2 + g * (128 * k2 * 2));
          const uint32_t acc2 = tmem0 + g * WG_COL + ACC2_COL;
          for (int ks = 0; ks < k2 / 16; ++ks) {
            const uint64_t da = make_desc_interleaved(a2 + ks * 2 * (128 * 16), 128 * 16, 128);
            const uint64_t db = make_desc_interleaved(w1a + ks * 2 * (h1p * 16), h1p * 16, 128);
            mma_f16_ss(acc2, da, db, p.idesc2, ks > 0 ? 1u : 0u);
          }
          mma_commit(smem_u32(&bars[4 * g + 3]));
        }
      }
      // weighted sum over the steps: out = S * K
      if (ok && mbar_wait(smem_u32(&bars[8]), 0, 12)) {
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(ss), ka = smem_u32(kts);
        for (int ks = 0; ks < tp / 16; ++ks) {
          const uint64_t da = make_desc_interleaved(sa + ks * 2 * (128 * 16), 128 * 16, 128);
          const uint64_t db = make_desc_interleaved(ka + ks * 2 * (np * 16), np * 16, 128);
          mma_f16_ss(tmem0 + ACC3_COL, da, db, p.idesc3, ks > 0 ? 1u : 0u);
        }
      }
      mma_commit(smem_u32(&bars[9]));
    }
  } else {
    // ---- workers ----------------------------------------------------------------------------
    const int g = warp >> 2;                 // warpgroup
    const int row = (warp & 3) * 32 + lane;  // TMEM lane == candidate row of the tile
    const int n = tile * 128 + row;
    const bool valid = n < p.n_cand;
    const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16) + g * WG_COL;
    uint8_t* a1 = smem + L.a1 + g * (128 * k1 * 2);
    uint8_t* a2 = smem + L.a2 + g * (128 * k2 * 2);

    // q row as 16-byte chunks (dp <= 64 -> at most 8), with the constant-1 column when it lives here
    uint4 qv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      __half h[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int i = c * 8 + e;
        __half v = zero;
        if (c < nch) {
          if (i < d) v = valid ? p.q[((int64_t)r * p.n_cand + n) * p.ldq + i] : zero;
          else if (i == G.ones1) v = one;
        }
        h[e] = v;
      }
      qv[c] = *reinterpret_cast<uint4*>(h);
    }
    // constant parts of both operands: the q segment (and the ones columns)
#pragma unroll
    for (int c = 0; c < 8; ++c)
      if (c < nch) *reinterpret_cast<uint4*>(a1 + c * (128 * 16) + row * 16) = qv[c];
    const uint4 ones_chunk = make_uint4(0x00003C00u, 0, 0, 0);          // fp16 {1,0,0,0,0,0,0,0}
    if (G.ones1 == 4 * dp) {
      *reinterpret_cast<uint4*>(a1 + (4 * nch) * (128 * 16) + row * 16) = ones_chunk;
      *reinterpret_cast<uint4*>(a1 + (4 * nch + 1) * (128 * 16) + row * 16) = make_uint4(0, 0, 0, 0);
    }
    *reinterpret_cast<uint4*>(a2 + (h0p / 8) * (128 * 16) + row * 16) = ones_chunk;
    *reinterpret_cast<uint4*>(a2 + (h0p / 8 + 1) * (128 * 16) + row * 16) = make_uint4(0, 0, 0, 0);

    auto build_a1 = [&](int t) {
      const uint4* kt = reinterpret_cast<const uint4*>(khs + t * dp);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < nch) {
          const uint4 kc = kt[c];
          const __half2* kh = reinterpret_cast<const __half2*>(&kc);
          const __half2* qh = reinterpret_cast<const __half2*>(&qv[c]);
          uint4 df, pr;
          __half2* dh = reinterpret_cast<__half2*>(&df);
          __half2* ph = reinterpret_cast<__half2*>(&pr);
#pragma unroll
          for (int e = 0; e < 4; ++e) { dh[e] = __hsub2(qh[e], kh[e]); ph[e] = __hmul2(qh[e], kh[e]); }
          // q's padding column holding the constant 1 gives 1-0 in `df`; harmless, its W0 rows are zero
          *reinterpret_cast<uint4*>(a1 + (nch + c) * (128 * 16) + row * 16) = kc;
          *reinterpret_cast<uint4*>(a1 + (2 * nch + c) * (128 * 16) + row * 16) = df;
          *reinterpret_cast<uint4*>(a1 + (3 * nch + c) * (128 * 16) + row * 16) = pr;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&bars[4 * g + 0]));
    };

    bool ok = true;
    if (g < tl) build_a1(g);
    int i = 0;
    for (int t = g; t < tl; t += 2, ++i) {
      // layer-1 accumulator -> activation -> A2
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[4 * g + 1]), (uint32_t)i & 1u, 20));
      if (!ok) break;
      tc_fence_after_sync();
      for (int c = 0; c < h0p; c += 32) {
        uint32_t v[32];
        const bool full = h0p - c >= 32;
        if (full) { tmem_ld32_nowait(lane_addr + ACC1_COL + c, v); tmem_wait_ld(v); }
        else {
          uint32_t v16[16];
          tmem_ld16_nowait(lane_addr + ACC1_COL + c, v16);
          tmem_wait_ld(v16);
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = v16[e];
        }
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          if (full || q8 < 2) {
            uint32_t y[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int col = q8 * 8 + 2 * e;
              const __half2 x = __floats2half2_rn(__uint_as_float(v[col]), __uint_as_float(v[col + 1]));
              y[e] = h2_bits(act_pair<ACT>(x, c1[(c + col) >> 1]));
            }
            *reinterpret_cast<uint4*>(a2 + ((c >> 3) + q8) * (128 * 16) + row * 16) = make_uint4(y[0], y[1], y[2], y[3]);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars[4 * g + 2]));

      // next step's A1 while the second MMA runs
      if (t + 2 < tl) build_a1(t + 2);

      // layer-2 accumulator -> activation -> score
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[4 * g + 3]), (uint32_t)i & 1u, 21));
      if (!ok) break;
      tc_fence_after_sync();
      float s = p.b2;
      for (int c = 0; c < h1p; c += 16) {
        uint32_t v[16];
        tmem_ld16_nowait(lane_addr + ACC2_COL + c, v);
        tmem_wait_ld(v);
        float2 part = make_float2(0.f, 0.f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const __half2 x = __floats2half2_rn(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
          const float2 f = __half22float2(act_pair_w<ACT>(x, c2[(c >> 1) + e]));
          part.x += f.x; part.y += f.y;
        }
        s += part.x + part.y;
      }
      tc_fence_before_sync();
      if (p.scores && valid && !p.use_softmax) p.scores[((int64_t)r * p.n_cand + n) * p.T + t] = s;
      ss[(t >> 3) * (128 * 8) + row * 8 + (t & 7)] = __float2half_rn(s);
    }

    if (p.use_softmax) {
      // masked softmax over the steps, in place on this thread's row of S (steps >= tl are masked out)
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (g == 0) {
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
    }
    fence_proxy_async_smem();
    mbar_arrive(smem_u32(&bars[8]));

    if (g == 0) {
      ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(&bars[9]), 0, 22));
      tc_fence_after_sync();
      if (ok) {
        __half* o = p.out + ((int64_t)r * p.n_cand + n) * p.ldo;
        for (int c = 0; c < np; c += 16) {
          float v[16];
          tmem_ld16(tmem0 + ((uint32_t)((warp & 3) * 32) << 16) + ACC3_COL + c, v);
          if (valid) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (c + e < d) o[c + e] = __float2half_rn(v[e]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem0, TMEM_COLS);
  }
}

bool tc_eligible(const xb_din_att_args& a, int* why) {
  const TcGeom g = tc_geom(a.d, a.h0, a.h1, a.T);
  if (g.dp > 64 || g.k1 > 272) { if (why) *why = 1; return false; }
  if (g.h0p > 128 || g.h1p > 64) { if (why) *why = 2; return false; }
  if (g.tp > 256) { if (why) *why = 5; return false; }
  if (tc_layout(g, a.T).total > 220 * 1024) { if (why) *why = 3; return false; }
  if (a.use_softmax && a.scores) { if (why) *why = 4; return false; }   // normalised scores are not written out
  return true;
}

int launch_att_tc(AttParams& p, const xb_din_att_args& a, cudaStream_t stream) {
  const TcGeom g = tc_geom(a.d, a.h0, a.h1, a.T);
  p.tiles_per_req = (a.n_cand + 127) / 128;
  p.idesc1 = umma::make_idesc(128, g.h0p, 0);
  p.idesc2 = umma::make_idesc(128, g.h1p, 0);
  p.idesc3 = umma::make_idesc(128, g.np, 0);
  const TcSmemLayout L = tc_layout(g, p.T);
  static bool attr_set = false;
  if (!attr_set) {
    XB_CUDA(cudaFuncSetAttribute(din_att_tc_kernel<XB_ACT_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    XB_CUDA(cudaFuncSetAttribute(din_att_tc_kernel<XB_ACT_SIGMOID>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    XB_CUDA(cudaFuncSetAttribute(din_att_tc_kernel<XB_ACT_DICE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  const int64_t blocks = (int64_t)a.requests * p.tiles_per_req;
  XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_din_attention: too many tiles");
  if (a.act == XB_ACT_DICE) din_att_tc_kernel<XB_ACT_DICE><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  else if (a.act == XB_ACT_SIGMOID) din_att_tc_kernel<XB_ACT_SIGMOID><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  else din_att_tc_kernel<XB_ACT_NONE><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  return check_launch("din_att_tc_kernel");
}

}  // namespace
}  // namespace xb
