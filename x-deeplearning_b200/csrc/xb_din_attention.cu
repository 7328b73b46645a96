// Fused DIN attention unit.
//
// For every (candidate n, behaviour step t) pair of a request the unit runs a
// three-layer MLP on x = [q_n, k_t, q_n-k_t, q_n*k_t] and sums k_t weighted by
// the resulting score. Nothing but q, k and the [n_cand, d] result touches HBM.
//
// tcgen05 engine. One CTA owns 128 candidates of one request and walks the
// behaviour steps. Two worker warpgroups (one candidate row per thread) take
// alternate steps; a ninth warp issues the MMAs, so the tensor pipe works on one
// warpgroup's step while the other warpgroup runs its activations:
//   worker: build A1 = [q|k_t|q-k_t|q*k_t] (fp16, 128 x 4dp) in shared memory
//   MMA   : acc1[128 x h0] = A1 * W0^T               (tcgen05.mma, TMEM accumulator)
//   worker: acc1 -> +bias, activation -> fp16 A2 in shared memory
//   MMA   : acc2[128 x h1] = A2 * W1^T
//   worker: acc2 -> +bias, activation, dot with W2 -> score; out += score * k_t
// Shared-memory operands use the un-swizzled K-major core-matrix layout: the
// 16-byte chunk c of row r sits at c*(rows*16) + r*16, so a warp's 32 rows of one
// chunk are 512 contiguous bytes (conflict-free stores) and the descriptor's
// leading-dimension offset is rows*16, its stride offset 128.
// Each feature segment is padded from d to dp = roundup(d, 8) columns so that
// segments start on chunk boundaries; the padded weight rows are zero.
//
// CUDA-core engine: the same arithmetic in fp32 without intermediate rounding,
// one CTA per candidate; it serves shapes the tcgen05 engine does not take and
// cross-checks it in the tests.
#include <cstring>

#include "xb_common.cuh"
#include "xb_umma.cuh"

namespace xb {
namespace {

struct AttParams {
  const __half* q; int64_t ldq;
  const __half* k; int64_t ldk;
  const int32_t* seq_len;
  __half* out; int64_t ldo;
  float* scores;
  int requests, n_cand, T, d, h0, h1, act, use_softmax;
  const __half* W0; const __half* W1; const float* W2;
  const float *b0, *b1; float b2;
  const float *g0, *m0, *v0, *g1, *m1, *v1;
  // tcgen05 engine geometry
  int dp, k1, h0p, h1p, tiles_per_req;
  uint32_t idesc1, idesc2;
};

__device__ __forceinline__ float att_act(int act, float x, float g, float a, float bneg) {
  // a = rstd, bneg = -mean*rstd (Dice); g = gamma
  if (act == XB_ACT_DICE) {
    float p = 1.f / (1.f + __expf(-fmaf(x, a, bneg)));
    return x * fmaf(p, 1.f - g, g);
  }
  if (act == XB_ACT_SIGMOID) return 1.f / (1.f + __expf(-x));
  return x;
}

// --------------------------------------------------------------------------
// CUDA-core engine: one CTA per (request, candidate); thread = behaviour step.
constexpr int SIMT_THREADS = 128;

__global__ void __launch_bounds__(SIMT_THREADS) din_att_simt_kernel(const __grid_constant__ AttParams p) {
  extern __shared__ float sm[];
  const int r = blockIdx.y, n = blockIdx.x;
  const int d = p.d, h0 = p.h0, h1 = p.h1, T = p.T;
  float* qs = sm;                       // [d]
  float* y0 = qs + d;                   // [h0][SIMT_THREADS]
  float* sc = y0 + h0 * SIMT_THREADS;   // [T]
  float* red = sc + T;                  // [SIMT_THREADS]
  const __half* q = p.q + ((int64_t)r * p.n_cand + n) * p.ldq;
  const __half* kbase = p.k + (int64_t)r * T * p.ldk;
  for (int i = threadIdx.x; i < d; i += SIMT_THREADS) qs[i] = __half2float(q[i]);
  __syncthreads();
  int tl = p.seq_len ? p.seq_len[r] : T;
  tl = tl < 0 ? 0 : (tl > T ? T : tl);

  for (int t0 = 0; t0 < T; t0 += SIMT_THREADS) {
    const int t = t0 + threadIdx.x;
    if (t < tl) {
      const __half* kt = kbase + (int64_t)t * p.ldk;
      for (int j = 0; j < h0; ++j) {
        const __half* w = p.W0 + (int64_t)j * 4 * d;
        float acc = p.b0 ? p.b0[j] : 0.f;
        for (int i = 0; i < d; ++i) {
          const float qi = qs[i], ki = __half2float(kt[i]);
          acc = fmaf(qi, __half2float(w[i]), acc);
          acc = fmaf(ki, __half2float(w[d + i]), acc);
          acc = fmaf(qi - ki, __half2float(w[2 * d + i]), acc);
          acc = fmaf(qi * ki, __half2float(w[3 * d + i]), acc);
        }
        float g = 0.f, a = 1.f, bn = 0.f;
        if (p.act == XB_ACT_DICE) { g = p.g0[j]; a = dice_rstd(p.v0[j], 0); bn = -p.m0[j] * a; }
        y0[j * SIMT_THREADS + threadIdx.x] = att_act(p.act, acc, g, a, bn);
      }
      float s = p.b2;
      for (int j2 = 0; j2 < h1; ++j2) {
        const __half* w = p.W1 + (int64_t)j2 * h0;
        float acc = p.b1 ? p.b1[j2] : 0.f;
        for (int j = 0; j < h0; ++j) acc = fmaf(y0[j * SIMT_THREADS + threadIdx.x], __half2float(w[j]), acc);
        float g = 0.f, a = 1.f, bn = 0.f;
        if (p.act == XB_ACT_DICE) { g = p.g1[j2]; a = dice_rstd(p.v1[j2], 0); bn = -p.m1[j2] * a; }
        s = fmaf(att_act(p.act, acc, g, a, bn), p.W2[j2], s);
      }
      sc[t] = s;
    } else if (t < T) {
      sc[t] = p.use_softmax ? -4294967295.0f : 0.f;
    }
  }
  __syncthreads();
  if (p.use_softmax) {
    float m = -INFINITY;
    for (int t = threadIdx.x; t < T; t += SIMT_THREADS) m = fmaxf(m, sc[t]);
    red[threadIdx.x] = m;
    __syncthreads();
    for (int s = SIMT_THREADS / 2; s > 0; s >>= 1) {
      if (threadIdx.x < s) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + s]);
      __syncthreads();
    }
    m = red[0];
    __syncthreads();
    float l = 0.f;
    for (int t = threadIdx.x; t < T; t += SIMT_THREADS) { float e = __expf(sc[t] - m); sc[t] = e; l += e; }
    red[threadIdx.x] = l;
    __syncthreads();
    for (int s = SIMT_THREADS / 2; s > 0; s >>= 1) {
      if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
      __syncthreads();
    }
    l = red[0];
    for (int t = threadIdx.x; t < T; t += SIMT_THREADS) sc[t] /= l;
    __syncthreads();
  }
  if (p.scores)
    for (int t = threadIdx.x; t < T; t += SIMT_THREADS) p.scores[((int64_t)r * p.n_cand + n) * T + t] = sc[t];
  for (int e = threadIdx.x; e < d; e += SIMT_THREADS) {
    float o = 0.f;
    for (int t = 0; t < T; ++t) o = fmaf(sc[t], __half2float(kbase[(int64_t)t * p.ldk + e]), o);
    p.out[((int64_t)r * p.n_cand + n) * p.ldo + e] = __float2half_rn(o);
  }
}

// --------------------------------------------------------------------------
// tcgen05 engine
constexpr int TC_THREADS = 288;          // 2 worker warpgroups + 1 MMA warp
constexpr int TMEM_COLS = 512;
constexpr int ACC1_COL = 0, ACC2_COL = 128, WG_COL = 256;

struct TcSmemLayout {
  int w0, w1, a1, a2, kh, cst, total;
};
__host__ __device__ inline TcSmemLayout tc_layout(int dp, int k1, int h0p, int h1p, int T) {
  TcSmemLayout L;
  int off = 0;
  L.w0 = off; off += h0p * k1 * 2;             // W0 operand, [h0p rows, k1] core-matrix layout
  L.w1 = off; off += h1p * h0p * 2;            // W1 operand
  L.a1 = off; off += 2 * 128 * k1 * 2;         // A1, one buffer per warpgroup
  L.a2 = off; off += 2 * 128 * h0p * 2;        // A2, one buffer per warpgroup
  L.kh = off; off += T * dp * 2;               // k rows, fp16, padded to dp
  off = (off + 15) / 16 * 16;
  L.cst = off; off += (4 * h0p + 5 * h1p) * 4; // per-column epilogue constants
  L.total = off;
  return L;
}

__global__ void __launch_bounds__(TC_THREADS, 1) din_att_tc_kernel(const __grid_constant__ AttParams p) {
  using namespace umma;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[8];      // [wg][a1_full, acc1_full, a2_full, acc2_full]
  __shared__ uint32_t tmem_base_s;
  __shared__ float merge[128 * 66];              // warpgroup 1 -> 0: m, l, acc[dp<=64]

  const TcSmemLayout L = tc_layout(p.dp, p.k1, p.h0p, p.h1p, p.T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x / p.tiles_per_req, tile = blockIdx.x % p.tiles_per_req;
  const int dp = p.dp, k1 = p.k1, h0p = p.h0p, h1p = p.h1p, d = p.d;
  int tl = p.seq_len ? p.seq_len[r] : p.T;
  tl = tl < 0 ? 0 : (tl > p.T ? p.T : tl);

  __half* w0s = reinterpret_cast<__half*>(smem + L.w0);
  __half* w1s = reinterpret_cast<__half*>(smem + L.w1);
  __half* khs = reinterpret_cast<__half*>(smem + L.kh);
  float* cst = reinterpret_cast<float*>(smem + L.cst);
  float* c0 = cst;                 // [h0p][4]: bias, gamma, rstd, -mean*rstd
  float* c1 = cst + 4 * h0p;       // [h1p][5]: bias, gamma, rstd, -mean*rstd, W2

  // ---- prologue: operands that stay resident for the whole tile -------------
  // W0: element (n, kk) -> chunk kk/8 of row n at chunk*(h0p*16) + n*16 bytes
  for (int idx = threadIdx.x; idx < h0p * k1; idx += TC_THREADS) {
    const int n = idx / k1, kk = idx - n * k1;
    const int seg = kk / dp, i = kk - seg * dp;
    __half v = __float2half(0.f);
    if (n < p.h0 && i < d) v = p.W0[(int64_t)n * 4 * d + seg * d + i];
    w0s[(kk >> 3) * (h0p * 8) + n * 8 + (kk & 7)] = v;
  }
  for (int idx = threadIdx.x; idx < h1p * h0p; idx += TC_THREADS) {
    const int n = idx / h0p, kk = idx - n * h0p;
    __half v = __float2half(0.f);
    if (n < p.h1 && kk < p.h0) v = p.W1[(int64_t)n * p.h0 + kk];
    w1s[(kk >> 3) * (h1p * 8) + n * 8 + (kk & 7)] = v;
  }
  for (int idx = threadIdx.x; idx < p.T * dp; idx += TC_THREADS) {
    const int t = idx / dp, i = idx - t * dp;
    khs[idx] = (i < d) ? p.k[((int64_t)r * p.T + t) * p.ldk + i] : __float2half(0.f);
  }
  for (int j = threadIdx.x; j < h0p; j += TC_THREADS) {
    float b = 0.f, g = 0.f, a = 1.f, bn = 0.f;
    if (j < p.h0) {
      b = p.b0 ? p.b0[j] : 0.f;
      if (p.act == XB_ACT_DICE) { g = p.g0[j]; a = dice_rstd(p.v0[j], 0); bn = -p.m0[j] * a; }
    }
    c0[4 * j] = b; c0[4 * j + 1] = g; c0[4 * j + 2] = a; c0[4 * j + 3] = bn;
  }
  for (int j = threadIdx.x; j < h1p; j += TC_THREADS) {
    float b = 0.f, g = 0.f, a = 1.f, bn = 0.f, w2 = 0.f;
    if (j < p.h1) {
      b = p.b1 ? p.b1[j] : 0.f; w2 = p.W2[j];
      if (p.act == XB_ACT_DICE) { g = p.g1[j]; a = dice_rstd(p.v1[j], 0); bn = -p.m1[j] * a; }
    }
    c1[5 * j] = b; c1[5 * j + 1] = g; c1[5 * j + 2] = a; c1[5 * j + 3] = bn; c1[5 * j + 4] = w2;
  }
  if (threadIdx.x == 0) {
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&bars[4 * g + 0]), 128);
      mbar_init(smem_u32(&bars[4 * g + 1]), 1);
      mbar_init(smem_u32(&bars[4 * g + 2]), 128);
      mbar_init(smem_u32(&bars[4 * g + 3]), 1);
    }
    fence_barrier_init();
  }
  if (warp == 8) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
  fence_proxy_async_smem();          // W0/W1 were written through the generic proxy
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = tmem_base_s;

  if (warp == 8) {
    // ---- MMA issue ------------------------------------------------------------
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
          const uint32_t a2 = smem_u32(smem + L.a2 + g * (128 * h0p * 2));
          const uint32_t acc2 = tmem0 + g * WG_COL + ACC2_COL;
          for (int ks = 0; ks < h0p / 16; ++ks) {
            const uint64_t da = make_desc_interleaved(a2 + ks * 2 * (128 * 16), 128 * 16, 128);
            const uint64_t db = make_desc_interleaved(w1a + ks * 2 * (h1p * 16), h1p * 16, 128);
            mma_f16_ss(acc2, da, db, p.idesc2, ks > 0 ? 1u : 0u);
          }
          mma_commit(smem_u32(&bars[4 * g + 3]));
        }
      }
    }
  } else {
    // ---- workers ----------------------------------------------------------------
    const int g = warp >> 2;                 // warpgroup
    const int row = (warp & 3) * 32 + lane;  // TMEM lane == candidate row of the tile
    const int n = tile * 128 + row;
    const bool valid = n < p.n_cand;
    const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16) + g * WG_COL;
    uint8_t* a1 = smem + L.a1 + g * (128 * k1 * 2);
    uint8_t* a2 = smem + L.a2 + g * (128 * h0p * 2);
    const int nch = dp / 8;                  // chunks per segment

    // q row in registers as 16-byte chunks (dp <= 64 -> at most 8 chunks)
    uint4 qv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      __half h[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int i = c * 8 + e;
        h[e] = (valid && c < nch && i < d) ? p.q[((int64_t)r * p.n_cand + n) * p.ldq + i] : __float2half(0.f);
      }
      qv[c] = *reinterpret_cast<uint4*>(h);
    }
    // the q segment never changes: write it once
#pragma unroll
    for (int c = 0; c < 8; ++c)
      if (c < nch) *reinterpret_cast<uint4*>(a1 + c * (128 * 16) + row * 16) = qv[c];

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
          *reinterpret_cast<uint4*>(a1 + (nch + c) * (128 * 16) + row * 16) = kc;
          *reinterpret_cast<uint4*>(a1 + (2 * nch + c) * (128 * 16) + row * 16) = df;
          *reinterpret_cast<uint4*>(a1 + (3 * nch + c) * (128 * 16) + row * 16) = pr;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&bars[4 * g + 0]));
    };

    float acc[64];
#pragma unroll
    for (int e = 0; e < 64; ++e) acc[e] = 0.f;
    float mrun = -INFINITY, lrun = 0.f;
    bool ok = true;

    if (g < tl) build_a1(g);
    int i = 0;
    for (int t = g; t < tl; t += 2, ++i) {
      // layer-1 accumulator -> activation -> A2
      ok = ok && mbar_wait(smem_u32(&bars[4 * g + 1]), (uint32_t)i & 1u, 20);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      for (int c = 0; c < h0p; c += 16) {
        float v[16];
        tmem_ld16(lane_addr + ACC1_COL + c, v);
        uint32_t packed[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const float4 k0 = *reinterpret_cast<const float4*>(c0 + 4 * (c + e));
          const float4 k1v = *reinterpret_cast<const float4*>(c0 + 4 * (c + e + 1));
          const float y0 = att_act(p.act, v[e] + k0.x, k0.y, k0.z, k0.w);
          const float y1 = att_act(p.act, v[e + 1] + k1v.x, k1v.y, k1v.z, k1v.w);
          __half2 h = __floats2half2_rn(y0, y1);
          packed[e >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(a2 + (c / 8) * (128 * 16) + row * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(a2 + (c / 8 + 1) * (128 * 16) + row * 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars[4 * g + 2]));

      // next step's A1 while the second MMA runs
      if (t + 2 < tl) build_a1(t + 2);

      // layer-2 accumulator -> activation -> score
      ok = ok && mbar_wait(smem_u32(&bars[4 * g + 3]), (uint32_t)i & 1u, 21);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      float s = p.b2;
      for (int c = 0; c < h1p; c += 16) {
        float v[16];
        tmem_ld16(lane_addr + ACC2_COL + c, v);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float* kc = c1 + 5 * (c + e);
          s = fmaf(att_act(p.act, v[e] + kc[0], kc[1], kc[2], kc[3]), kc[4], s);
        }
      }
      tc_fence_before_sync();
      if (p.scores && valid && !p.use_softmax) p.scores[((int64_t)r * p.n_cand + n) * p.T + t] = s;
      float wgt = s;
      if (p.use_softmax) {
        const float mnew = fmaxf(mrun, s);
        const float corr = __expf(mrun - mnew);     // exp(-inf) = 0 on the first step
        wgt = __expf(s - mnew);
        lrun = lrun * corr + wgt;
#pragma unroll
        for (int e = 0; e < 64; ++e) acc[e] *= corr;
        mrun = mnew;
      }
      const __half2* kt2 = reinterpret_cast<const __half2*>(khs + t * dp);
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        if (2 * e < dp) {
          const float2 kf = __half22float2(kt2[e]);
          acc[2 * e] = fmaf(wgt, kf.x, acc[2 * e]);
          acc[2 * e + 1] = fmaf(wgt, kf.y, acc[2 * e + 1]);
        }
      }
    }

    // ---- combine the two warpgroups and store -------------------------------------
    if (g == 1) {
      merge[row * 66] = mrun; merge[row * 66 + 1] = lrun;
#pragma unroll
      for (int e = 0; e < 64; ++e) if (e < dp) merge[row * 66 + 2 + e] = acc[e];
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight worker warps only
    if (g == 0 && valid) {
      const float m1 = merge[row * 66], l1 = merge[row * 66 + 1];
      float f0 = 1.f, f1 = 1.f, inv = 1.f;
      if (p.use_softmax) {
        const float m = fmaxf(mrun, m1);
        f0 = (mrun == -INFINITY) ? 0.f : __expf(mrun - m);
        f1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - m);
        const float l = lrun * f0 + l1 * f1;
        inv = l > 0.f ? 1.f / l : 0.f;
      }
      __half* o = p.out + ((int64_t)r * p.n_cand + n) * p.ldo;
#pragma unroll
      for (int e = 0; e < 64; ++e)
        if (e < d) o[e] = __float2half_rn((acc[e] * f0 + merge[row * 66 + 2 + e] * f1) * inv);
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
  const int dp = (a.d + 7) / 8 * 8, h0p = (a.h0 + 15) / 16 * 16, h1p = (a.h1 + 15) / 16 * 16;
  if (dp > 64 || 4 * dp > 256) { if (why) *why = 1; return false; }
  if (h0p > 128 || h1p > 128) { if (why) *why = 2; return false; }
  const TcSmemLayout L = tc_layout(dp, 4 * dp, h0p, h1p, a.T);
  if (L.total > 190 * 1024) { if (why) *why = 3; return false; }
  if (a.use_softmax && a.scores) { if (why) *why = 4; return false; }   // normalised scores need a second pass
  return true;
}

}  // namespace

int att_status(int* out) { return umma::read_status_word(out); }
int att_clear_status() { return umma::clear_status_word(); }

}  // namespace xb

using namespace xb;

extern "C" int xb_din_attention(const xb_din_att_args* a, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(a, XB_ERR_ARG, "xb_din_attention: null arguments");
  XB_REQUIRE(a->q && a->k && a->out, XB_ERR_ARG, "xb_din_attention: null tensor");
  XB_REQUIRE(a->requests >= 0 && a->n_cand >= 0 && a->T > 0 && a->d > 0 && a->h0 > 0 && a->h1 > 0, XB_ERR_ARG,
             "xb_din_attention: bad sizes");
  XB_REQUIRE(a->ldq >= a->d && a->ldk >= a->d && a->ldo >= a->d, XB_ERR_ARG, "xb_din_attention: leading dimension < d");
  XB_REQUIRE(a->w.W0 && a->w.W1 && a->w.W2, XB_ERR_ARG, "xb_din_attention: missing weights");
  XB_REQUIRE(a->act >= XB_ACT_NONE && a->act <= XB_ACT_DICE, XB_ERR_UNSUPPORTED, "xb_din_attention: act %d", a->act);
  XB_REQUIRE(a->act != XB_ACT_DICE || (a->w.gamma0 && a->w.mean0 && a->w.var0 && a->w.gamma1 && a->w.mean1 && a->w.var1),
             XB_ERR_ARG, "xb_din_attention: Dice needs gamma/mean/var for both layers");
  XB_REQUIRE(a->T <= 4096 && a->d <= 256 && a->h0 <= 256, XB_ERR_LIMIT, "xb_din_attention: T<=4096, d<=256, h0<=256");
  if (a->requests == 0 || a->n_cand == 0) return 0;

  AttParams p;
  memset(&p, 0, sizeof(p));
  p.q = (const __half*)a->q; p.ldq = a->ldq; p.k = (const __half*)a->k; p.ldk = a->ldk;
  p.seq_len = a->seq_len; p.out = (__half*)a->out; p.ldo = a->ldo; p.scores = a->scores;
  p.requests = a->requests; p.n_cand = a->n_cand; p.T = a->T; p.d = a->d; p.h0 = a->h0; p.h1 = a->h1;
  p.act = a->act; p.use_softmax = a->use_softmax;
  p.W0 = (const __half*)a->w.W0; p.W1 = (const __half*)a->w.W1; p.W2 = a->w.W2;
  p.b0 = a->w.b0; p.b1 = a->w.b1; p.b2 = a->w.b2;
  p.g0 = a->w.gamma0; p.m0 = a->w.mean0; p.v0 = a->w.var0;
  p.g1 = a->w.gamma1; p.m1 = a->w.mean1; p.v1 = a->w.var1;

  int why = 0;
  const bool tc = a->engine != XB_GEMM_SIMT && tc_eligible(*a, &why);
  XB_REQUIRE(tc || a->engine != XB_GEMM_TCGEN05, XB_ERR_UNSUPPORTED,
             "xb_din_attention: shape outside the tcgen05 engine (reason %d)", why);
  if (tc) {
    p.dp = (a->d + 7) / 8 * 8; p.k1 = 4 * p.dp;
    p.h0p = (a->h0 + 15) / 16 * 16; p.h1p = (a->h1 + 15) / 16 * 16;
    p.tiles_per_req = (a->n_cand + 127) / 128;
    p.idesc1 = umma::make_idesc(128, p.h0p, 0);
    p.idesc2 = umma::make_idesc(128, p.h1p, 0);
    const TcSmemLayout L = tc_layout(p.dp, p.k1, p.h0p, p.h1p, p.T);
    static bool attr_set = false;
    if (!attr_set) {
      XB_CUDA(cudaFuncSetAttribute(din_att_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 190 * 1024));
      attr_set = true;
    }
    const int64_t blocks = (int64_t)a->requests * p.tiles_per_req;
    XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_din_attention: too many tiles");
    din_att_tc_kernel<<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
    return check_launch("din_att_tc_kernel");
  }
  const size_t smem = sizeof(float) * ((size_t)a->d + (size_t)a->h0 * SIMT_THREADS + a->T + SIMT_THREADS);
  XB_REQUIRE(smem <= 200 * 1024, XB_ERR_LIMIT, "xb_din_attention: shape too large for the CUDA-core engine");
  XB_REQUIRE(a->requests <= 65535, XB_ERR_LIMIT, "xb_din_attention: more than 65535 requests per call");
  static bool simt_attr = false;
  if (!simt_attr) {
    XB_CUDA(cudaFuncSetAttribute(din_att_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    simt_attr = true;
  }
  dim3 grid(a->n_cand, a->requests);
  din_att_simt_kernel<<<grid, SIMT_THREADS, smem, stream>>>(p);
  return check_launch("din_att_simt_kernel");
}
