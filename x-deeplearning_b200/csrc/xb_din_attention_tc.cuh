// tcgen05 engine of the fused DIN attention unit (included by xb_din_attention.cu).
//
// One CTA owns 128 candidates of one request and walks the behaviour steps.
// Worker warpgroups (one candidate row per thread) split the work by phase and
// step: layer-1 warpgroup w (one per acc1 buffer: three, or two when tensor
// memory is short) runs the layer-1 activations of the steps j with j % na1 == w,
// layer-2 warpgroup b (b = 0, 1) the layer-2 activations of the steps of parity b,
// two builder warps write A1 of every step up to na1 steps ahead; two more warps
// issue the MMAs, one per layer (the closing product goes with layer 2).
// The layer-1 accumulator, its operand A1 and the layer-2 operand are three deep
// when tensor memory has room (two otherwise), acc2 is double-buffered by step parity,
// and the activation math of up to five steps is in flight on each scheduler,
// so in steady state the tensor pipe, the SFU and the FP16 pipe overlap: the
// layer-1 MMA of a later step runs while the layer-1 warps still work on this one.
//   worker: A1 = [q|k_t|q*k_t] (fp16, 128 x k1) into shared memory; the q - k_t
//           segment of the reference's input is folded into the weights:
//           q Wq + k Wk + (q-k) Wd + (q*k) Wp = q (Wq+Wd) + k (Wk-Wd) + (q*k) Wp
//   MMA   : acc1[128 x h0p] = A1 * W0'^T                 (both operands from shared memory)
//   worker: acc1 -> activation -> fp16 A2 in tensor memory
//   MMA   : acc2[128 x h1p] = A2 * W1^T
//   worker: acc2 -> activation, dot with W2 -> score s[n,t] -> fp16 column t of S
// and, after the last step,
//   MMA   : out[128 x d] = S[128 x T] * K[T x d]          (the weighted sum is a GEMM too)
//
// Biases ride in the MMAs: A1 carries a constant-1 column (a padding column of
// the q segment when d is not a multiple of 8) whose W0 row is b0, and the last
// k step of layer 2 reads 16 columns shared by all A2 buffers, the first
// constant 1 with W1 row b1.
//
// Activations run on packed fp16 pairs with one SFU instruction per pair:
//   sigmoid(z) = 1/2 + 1/2 tanh(z/2), so Dice(x) = x * (C + D*tanh(A*x + B)) with
//   A = rstd/2, B = -mean*rstd/2, C = (1+gamma)/2, D = (1-gamma)/2 per column.
//
// The layer-2 operand never touches shared memory: a thread owns one candidate row = one
// tensor-memory lane and stores its fp16 pairs into that lane's columns (two
// consecutive k per 32-bit column). Shared-memory operands (A1, weights, S, K^T) use
// the un-swizzled K-major core-matrix layout: the 16-byte chunk c (8 consecutive k)
// of row r sits at c*(rows*16) + r*16, the descriptor's leading-dimension offset
// is rows*16 and its stride offset 128.
#pragma once

namespace xb {
namespace {

#ifdef XB_ATT_TRACE
// debug builds only: cycle stamps of CTA 0, [slot][step][event]
__device__ long long g_att_trace[7 * 128 * 4];
#define ATT_TR(slot, j, ev) do { if (blockIdx.x == 0 && (j) < 128) g_att_trace[((slot) * 128 + (j)) * 4 + (ev)] = clock64(); } while (0)
#define ATT_TR_VAL(slot, j, ev, val) do { if (blockIdx.x == 0 && (j) < 128) g_att_trace[((slot) * 128 + (j)) * 4 + (ev)] = (val); } while (0)
#define ATT_CLK() clock64()
#else
#define ATT_TR(slot, j, ev) do { } while (0)
#define ATT_TR_VAL(slot, j, ev, val) do { } while (0)
#define ATT_CLK() 0ll
#endif

constexpr int TC_BUILD_WARPS = 2;                          // 2 (two rows per thread) or 4 (one)
constexpr int TC_BROWS = 4 / TC_BUILD_WARPS;
// warps 0-11 layer 1, 12-19 layer 2, then the A1 builder warps, then one MMA-issuing warp per layer
constexpr int TC_L2_WARP0 = 12, TC_BUILD_WARP0 = 20, MMA1_TC_WARP = 20 + TC_BUILD_WARPS, MMA2_TC_WARP = 21 + TC_BUILD_WARPS;
constexpr int TC_THREADS = 32 * (22 + TC_BUILD_WARPS);
constexpr int TMEM_COLS = 512;

// Tensor-memory columns: [acc1 x na1 | acc2 x2 | A2 x na2 | ones | acc3]; when there is no room for the closing
// product's accumulator it reuses the acc1 buffers, which are idle by then.
struct TcGeom {
  int dp, nch, k1, ones1, h0p, k2, h1p, tp, np;
  int c_acc2, c_a2, c_ones, c_acc3, na1, na2, cols;
};

__host__ __device__ constexpr TcGeom tc_geom(int d, int h0, int h1, int T) {
  TcGeom g{};
  g.dp = (d + 7) / 8 * 8;
  g.nch = g.dp / 8;
  g.ones1 = (d < g.dp) ? d : 3 * g.dp;               // column of A1 that is constant 1
  g.k1 = (3 * g.dp + ((d < g.dp) ? 0 : 8) + 15) / 16 * 16;
  g.h0p = (h0 + 15) / 16 * 16;
  g.k2 = g.h0p + 16;                                 // column h0p of A2 is constant 1
  g.h1p = (h1 + 15) / 16 * 16;
  g.tp = (T + 15) / 16 * 16;
  g.np = (g.dp + 15) / 16 * 16;
  // deepest buffering that fits: (acc1, A2) = (3, 3), (3, 2), (2, 2); never more A2 buffers than accumulators
  g.na1 = 2; g.na2 = 2;
  for (int c = 0; c < 2; ++c) {
    const int n2 = c == 0 ? 3 : 2;
    if (3 * g.h0p + 2 * g.h1p + n2 * (g.h0p / 2) + 8 <= TMEM_COLS) { g.na1 = 3; g.na2 = n2; break; }
  }
  g.c_acc2 = g.na1 * g.h0p;
  g.c_a2 = g.c_acc2 + 2 * g.h1p;
  g.c_ones = g.c_a2 + g.na2 * (g.h0p / 2);
  g.cols = g.c_ones + 8;
  g.c_acc3 = (g.cols + g.np <= TMEM_COLS) ? g.cols : 0;
  return g;
}

struct TcSmemLayout {
  int w0, w1, a1, s, kt, kh, q, c1, c2, total;
};
__host__ __device__ inline TcSmemLayout tc_layout(const TcGeom& g, int T) {
  TcSmemLayout L;
  int off = 0;
  L.w0 = off; off += g.h0p * g.k1 * 2;          // W0 operand [h0p rows, k1]
  L.w1 = off; off += g.h1p * g.k2 * 2;          // W1 operand [h1p rows, k2]
  L.a1 = off; off += g.na1 * 128 * g.k1 * 2;    // A1 operand [128 rows, k1], one per acc1 buffer
  L.s = off; off += 128 * g.tp * 2;             // scores [128, tp]
  L.kt = off; off += g.np * g.tp * 2;           // K^T operand [np rows (feature), tp (step)]
  L.kh = off; off += T * g.dp * 2;              // k rows for building A1
  off = (off + 15) / 16 * 16;
  L.q = off; off += 128 * g.dp * 2;             // q rows of the tile, chunk-major
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

// Builds the weight operands the way the MMAs read them from shared memory: W0 [h0p rows, k1]
// and W1 [h1p rows, k2] in core-matrix layout with the bias rows, and the per-column-pair
// activation constants. `w0s..c2` may point to shared or global memory.
template <int ACT>
__device__ __forceinline__ void pack_weights(const AttParams& p, const TcGeom& G, __half* w0s, __half* w1s, uint4* c1,
                                             uint4* c2, int tid, int nthreads) {
  const int d = p.d, dp = G.dp, k1 = G.k1, h0p = G.h0p, k2 = G.k2, h1p = G.h1p;
  const __half zero = __float2half(0.f);
  for (int idx = tid; idx < h0p * k1; idx += nthreads) {
    const int n = idx / k1, kk = idx - n * k1;
    __half v = zero;
    if (n < p.h0) {
      if (kk == G.ones1) v = __float2half_rn(p.b0 ? p.b0[n] : 0.f);
      else if (kk < 3 * dp) {
        // segments [q | k | q*k] with the weights of the q - k segment folded into the first two
        const int seg = kk / dp, i = kk - seg * dp;
        if (i < d) {
          const __half* w = p.W0 + (int64_t)n * 4 * d + i;
          const float wd = __half2float(w[2 * d]);
          v = seg == 0 ? __float2half_rn(__half2float(w[0]) + wd)
                       : (seg == 1 ? __float2half_rn(__half2float(w[d]) - wd) : w[3 * d]);
        }
      }
    }
    w0s[(kk >> 3) * (h0p * 8) + n * 8 + (kk & 7)] = v;
  }
  for (int idx = tid; idx < h1p * k2; idx += nthreads) {
    const int n = idx / k2, kk = idx - n * k2;
    __half v = zero;
    if (n < p.h1) {
      if (kk < p.h0) v = p.W1[(int64_t)n * p.h0 + kk];
      else if (kk == h0p) v = __float2half_rn(p.b1 ? p.b1[n] : 0.f);
    }
    w1s[(kk >> 3) * (h1p * 8) + n * 8 + (kk & 7)] = v;
  }
  for (int j = tid; j < h0p / 2; j += nthreads) {
    float A[2] = {0, 0}, B[2] = {0, 0}, C[2] = {0, 0}, D[2] = {0, 0};
    for (int u = 0; u < 2; ++u) {
      const int col = 2 * j + u;
      if (col >= p.h0) continue;
      if (ACT == XB_ACT_DICE) {
        const float rs = dice_rstd(p.v0[col], 0), g = p.g0[col];
        A[u] = 0.5f * rs; B[u] = -0.5f * p.m0[col] * rs; C[u] = 0.5f * (1.f + g); D[u] = 0.5f * (1.f - g);
      } else if (ACT == XB_ACT_SIGMOID) { A[u] = 0.5f; C[u] = 0.5f; D[u] = 0.5f; }
    }
    // layer 1 keeps {A, B} and {C, D} apart (two column pairs per 16 bytes each): the activation runs in two
    // stages, the first needs A and B, the second C and D
    uint32_t* ab = reinterpret_cast<uint32_t*>(c1) + 2 * j;
    uint32_t* cd = reinterpret_cast<uint32_t*>(c1 + h0p / 4) + 2 * j;
    ab[0] = h2_bits(__floats2half2_rn(A[0], A[1])); ab[1] = h2_bits(__floats2half2_rn(B[0], B[1]));
    cd[0] = h2_bits(__floats2half2_rn(C[0], C[1])); cd[1] = h2_bits(__floats2half2_rn(D[0], D[1]));
  }
  for (int j = tid; j < h1p / 2; j += nthreads) {
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

// 16 accumulator columns of layer 1 (fp32, already in registers) -> activation -> 8 fp16 pairs of A2
template <int ACT>
__device__ __forceinline__ void pair_l1_block(const uint32_t (&cur)[16], const uint4* __restrict__ cc, uint32_t (&y)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e)
    y[e] = h2_bits(__floats2half2_rn(__uint_as_float(cur[2 * e]), __uint_as_float(cur[2 * e + 1])));
  if (ACT != XB_ACT_NONE) {
    uint32_t th[8];
#pragma unroll
    for (int e = 0; e < 8; ++e)
      th[e] = umma::tanh_f16x2(h2_bits(__hfma2(bits_h2(y[e]), bits_h2(cc[e].x), bits_h2(cc[e].y))));
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const __half2 g = __hfma2(bits_h2(th[e]), bits_h2(cc[e].w), bits_h2(cc[e].z));
      y[e] = h2_bits(ACT == XB_ACT_DICE ? __hmul2(bits_h2(y[e]), g) : g);
    }
  }
}

template <int ACT>
__global__ void att_pack_kernel(const __grid_constant__ AttParams p, uint8_t* dst) {
  const TcGeom G = tc_geom(p.d, p.h0, p.h1, p.T);
  const int w0_bytes = G.h0p * G.k1 * 2, w1_bytes = G.h1p * G.k2 * 2;
  pack_weights<ACT>(p, G, reinterpret_cast<__half*>(dst), reinterpret_cast<__half*>(dst + w0_bytes),
                    reinterpret_cast<uint4*>(dst + w0_bytes + w1_bytes),
                    reinterpret_cast<uint4*>(dst + w0_bytes + w1_bytes) + G.h0p / 2, threadIdx.x, blockDim.x);
}

// D0 / H0 / H1: the shape as compile-time constants (0 = read it from the arguments). With the shape known the
// block loops of both activation phases and the MMA chains unroll completely and every tensor-memory column,
// shared-memory offset and padding test folds into the instruction stream (issue slots are the second scarcest
// resource of this kernel after the SFU).
template <int ACT, int D0, int H0, int H1>
__global__ void __launch_bounds__(TC_THREADS, 1) din_att_tc_kernel(const __grid_constant__ AttParams p) {
  using namespace umma;
  using umma::tanh_f16x2;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[21];
  __shared__ uint32_t tmem_base_s;

  const int d_ = D0 ? D0 : p.d, h0_ = H0 ? H0 : p.h0, h1_ = H1 ? H1 : p.h1;
  const TcGeom G = tc_geom(d_, h0_, h1_, p.T);
  const TcSmemLayout L = tc_layout(G, p.T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x / p.tiles_per_req, tile = blockIdx.x % p.tiles_per_req;
  const int d = d_, dp = G.dp, nch = G.nch, k1 = G.k1, h0p = G.h0p, k2 = G.k2, h1p = G.h1p, tp = G.tp, np = G.np;
  int tl = p.seq_len ? p.seq_len[r] : p.T;
  tl = tl < 0 ? 0 : (tl > p.T ? p.T : tl);

  if (threadIdx.x == 0) ATT_TR(6, 120, 0);
  __half* w0s = reinterpret_cast<__half*>(smem + L.w0);
  __half* w1s = reinterpret_cast<__half*>(smem + L.w1);
  uint8_t* a1s = smem + L.a1;
  __half* ss = reinterpret_cast<__half*>(smem + L.s);
  __half* kts = reinterpret_cast<__half*>(smem + L.kt);
  __half* khs = reinterpret_cast<__half*>(smem + L.kh);
  __half* qs = reinterpret_cast<__half*>(smem + L.q);
  uint4* c1 = reinterpret_cast<uint4*>(smem + L.c1);
  uint4* c2 = reinterpret_cast<uint4*>(smem + L.c2);
  const __half zero = __float2half(0.f), one = __float2half(1.f);

  // ---- prologue: operands that stay resident for the whole tile ----------------------------
  // Everything that comes from global memory is requested with asynchronous copies first (weight image,
  // k rows of the request, q rows of the tile), so the latencies overlap instead of adding up.
  const bool async8 = (d % 4 == 0) && (p.ldq % 4 == 0) && (p.ldk % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k)) & 7) == 0;
  if (p.packed) {
    // weight operands were laid out once by xb_din_attention_pack: W0, W1, c1, c2 are adjacent
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.packed);
    const int n01 = (h0p * k1 * 2 + h1p * k2 * 2) / 16;
    for (int i = threadIdx.x; i < n01; i += TC_THREADS) cp_async16(smem + L.w0 + 16 * i, src + 16 * i);
    for (int i = threadIdx.x; i < h0p / 2 + h1p / 2; i += TC_THREADS) cp_async16(c1 + i, src + 16 * (n01 + i));
  } else {
    pack_weights<ACT>(p, G, w0s, w1s, c1, c2, threadIdx.x, TC_THREADS);
  }
  if (async8) {
    const int ppr = d / 4;                                   // 8-byte pieces per row
    const __half* kreq = p.k + (int64_t)r * p.T * p.ldk;
    for (int idx = threadIdx.x; idx < p.T * ppr; idx += TC_THREADS) {
      const int t = idx / ppr, pc = idx - t * ppr;
      cp_async8(khs + t * dp + pc * 4, kreq + (int64_t)t * p.ldk + pc * 4);
    }
    const int rows = min(128, p.n_cand - tile * 128);
    const __half* qreq = p.q + ((int64_t)r * p.n_cand + tile * 128) * p.ldq;
    for (int idx = threadIdx.x; idx < rows * ppr; idx += TC_THREADS) {
      const int row = idx / ppr, pc = idx - row * ppr;
      cp_async8(qs + ((pc >> 1) * 128 + row) * 8 + (pc & 1) * 4, qreq + (int64_t)row * p.ldq + pc * 4);
    }
  }
  cp_async_commit();
  // what no copy writes: padding columns, rows past the last candidate, the constant-1 column, S
  if (async8) {
    const int rows = min(128, p.n_cand - tile * 128), npad = dp - d;
    for (int idx = threadIdx.x; idx < 128 * npad; idx += TC_THREADS) {         // padding columns of every q row
      const int row = idx / npad, i = d + idx - row * npad;
      qs[(i >> 3) * (128 * 8) + row * 8 + (i & 7)] = (i == G.ones1) ? one : zero;
    }
    for (int idx = threadIdx.x; idx < (128 - rows) * d; idx += TC_THREADS) {   // rows past the last candidate
      const int row = rows + idx / d, i = idx % d;
      qs[(i >> 3) * (128 * 8) + row * 8 + (i & 7)] = zero;
    }
    for (int idx = threadIdx.x; idx < p.T * npad; idx += TC_THREADS) {         // padding columns of the k rows
      const int t = idx / npad;
      khs[t * dp + d + idx - t * npad] = zero;
    }
  } else {
    for (int idx = threadIdx.x; idx < 128 * dp; idx += TC_THREADS) {
      const int row = idx / dp, i = idx - row * dp;
      const bool have = i < d && tile * 128 + row < p.n_cand;
      qs[(i >> 3) * (128 * 8) + row * 8 + (i & 7)] =
          have ? p.q[((int64_t)r * p.n_cand + tile * 128 + row) * p.ldq + i] : (i == G.ones1 ? one : zero);
    }
    for (int idx = threadIdx.x; idx < p.T * dp; idx += TC_THREADS) {
      const int t = idx / dp, i = idx - t * dp;
      khs[idx] = (i < d) ? p.k[((int64_t)r * p.T + t) * p.ldk + i] : zero;
    }
  }
  for (int idx = threadIdx.x; idx < 128 * tp / 8; idx += TC_THREADS)
    reinterpret_cast<uint4*>(ss)[idx] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) ATT_TR(6, 120, 3);
  cp_async_wait_all();
  __syncthreads();
  if (threadIdx.x == 0) ATT_TR(6, 120, 1);
  // K^T operand of the closing product, from the k rows now in shared memory
  for (int idx = threadIdx.x; idx < np * tp; idx += TC_THREADS) {
    const int t = idx / np, e = idx - t * np;
    const __half v = (e < d && t < tl) ? khs[t * dp + e] : zero;
    kts[(t >> 3) * (np * 8) + e * 8 + (t & 7)] = v;
  }
  // barriers (b = step & 1, i = step % na1, a = step % na2):
  //   a1_full[i]   2 builder warps       -> layer-1 MMA warp: A1 of a step is in shared memory
  //   acc1_full[i] tcgen05.commit        -> layer-1 warpgroup i: layer-1 accumulator complete; builder: A1 read
  //   acc1_free[i] 128 layer-1 threads   -> layer-1 MMA warp: the accumulator's last block is in registers
  //   a2_full[i]   4 layer-1 warps       -> layer-2 MMA warp: A2 written
  //   a2_free[a]   tcgen05.commit        -> layer-1 warpgroups: the layer-2 MMA has read A2 buffer a
  //   acc2_full[b] tcgen05.commit        -> layer-2 warpgroup b: layer-2 accumulator complete
  //   acc2_free[b] 4 layer-2 warps       -> layer-2 MMA warp: acc2[b] drained
  //   s_full, acc3_full: the closing S*K product
  // A barrier never runs two phases ahead of a waiter: whatever completes its next phase needs something that
  // waiter produces after its wait (the drained accumulator, the next A1, the next A2).
  uint64_t* a1_full = &bars[0];
  uint64_t* acc1_full = &bars[3];
  uint64_t* acc1_free = &bars[6];
  uint64_t* a2_full = &bars[9];
  uint64_t* a2_free = &bars[12];
  uint64_t* acc2_full = &bars[15];
  uint64_t* acc2_free = &bars[17];
  uint64_t* s_full = &bars[19];
  uint64_t* acc3_full = &bars[20];
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc2_full[b]), 1);
      mbar_init(smem_u32(&acc2_free[b]), 4);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(smem_u32(&a1_full[i]), TC_BUILD_WARPS);
      mbar_init(smem_u32(&acc1_full[i]), 1);
      mbar_init(smem_u32(&acc1_free[i]), 128);
      mbar_init(smem_u32(&a2_full[i]), 4);
      mbar_init(smem_u32(&a2_free[i]), 1);
    }
    mbar_init(smem_u32(s_full), 8);
    mbar_init(smem_u32(acc3_full), 1);
    fence_barrier_init();
  }
  if (warp == MMA1_TC_WARP) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
  fence_proxy_async_smem();          // operands were written through the generic proxy
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = tmem_base_s;
  if (threadIdx.x == 0) ATT_TR(6, 120, 2);

  if (warp == MMA1_TC_WARP) {
    // ---- layer-1 MMA issue -----------------------------------------------------------------------------
    // Both MMA warps run their loops in uniform control flow and one elected lane issues: that keeps the
    // descriptors in uniform registers, and with the chains unrolled over descriptors computed once an MMA
    // issues in about 36 cycles instead of 100. Step j + na1 reuses the accumulator of step j: it is issued as
    // soon as the layer-1 warps have that accumulator's last block in registers.
    constexpr int NK1 = D0 ? tc_geom(D0, H0, H1, 16).k1 / 16 : 13;       // k steps of layer 1 (d <= 64)
    const int nks1 = D0 ? NK1 : k1 / 16;
    const int na1 = G.na1;
    uint64_t db1[NK1];
    {
      const uint64_t db1_0 = make_desc_interleaved(smem_u32(w0s), h0p * 16, 128);
#pragma unroll
      for (int ks = 0; ks < NK1; ++ks) db1[ks] = db1_0 + (uint64_t)(ks * ((2 * h0p * 16) >> 4));
    }
    const uint64_t da_step = (uint64_t)((2 * 128 * 16) >> 4);
    const uint64_t da1_0 = make_desc_interleaved(smem_u32(a1s), 128 * 16, 128);
    const uint64_t da1_buf = (uint64_t)((128 * k1 * 2) >> 4);
    int i1 = 0;                                               // acc1 and A1 buffer of the step being issued
    uint32_t ph1 = 0;                                         // (j / na1) & 1
    for (int j = 0; j < tl; ++j) {
      bool ok = true;
      if (j >= na1) ok = mbar_wait(smem_u32(&acc1_free[i1]), ph1 ^ 1u, 11);   // drained by the step that used it before
      ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(&a1_full[i1]), ph1, 10));
      if (!ok) break;
      tc_fence_after_sync();
      const uint64_t da = da1_0 + (uint64_t)i1 * da1_buf;
      const uint32_t acc1 = tmem0 + i1 * h0p;
#pragma unroll
      for (int ks = 0; ks < NK1; ++ks)
        if (ks < nks1) mma_f16_ss_elect(acc1, da + (uint64_t)ks * da_step, db1[ks], p.idesc1, ks > 0 ? 1u : 0u);
      mma_commit_elect(smem_u32(&acc1_full[i1]));
      if (lane == 0) ATT_TR(5, j, 2);
      if (++i1 == na1) { i1 = 0; ph1 ^= 1u; }
    }
  } else if (warp == MMA2_TC_WARP) {
    // ---- layer-2 MMA issue, then the closing S*K product -----------------------------------------------
    constexpr int NK2 = H0 ? tc_geom(D0, H0, H1, 16).h0p / 16 + 1 : 9;   // the last k step is the bias chunk
    const int nks2 = H0 ? NK2 : h0p / 16 + 1;
    uint64_t db2[NK2];
    {
      const uint64_t db2_0 = make_desc_interleaved(smem_u32(w1s), h1p * 16, 128);
#pragma unroll
      for (int ks = 0; ks < NK2; ++ks) db2[ks] = db2_0 + (uint64_t)(ks * ((2 * h1p * 16) >> 4));
    }
    bool ok = true;
    int a2i = 0, w1 = 0;                                      // j % na2, j % na1
    uint32_t ph1 = 0;                                         // (j / na1) & 1
    for (int j = 0; j < tl; ++j) {
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      // the layer-1 warps have written A2 of step j; acc2 of this parity was drained (step j-2)
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&a2_full[w1]), ph1, 12) &&
                                       mbar_wait(smem_u32(&acc2_free[j & 1]), ph ^ 1u, 13));
      if (!ok) break;
      if (lane == 0) ATT_TR(5, j, 0);
      tc_fence_after_sync();
      const uint32_t acc2 = tmem0 + G.c_acc2 + (j & 1) * h1p;
      const uint32_t ta = tmem0 + G.c_a2 + a2i * (h0p / 2);
#pragma unroll
      for (int ks = 0; ks < NK2; ++ks)
        if (ks < nks2)
          mma_f16_ts_elect(acc2, ks == nks2 - 1 ? tmem0 + G.c_ones : ta + 8 * ks, db2[ks], p.idesc2, ks > 0 ? 1u : 0u);
      mma_commit_elect(smem_u32(&acc2_full[j & 1]));
      mma_commit_elect(smem_u32(&a2_free[a2i]));
      if (lane == 0) ATT_TR(5, j, 1);
      a2i = a2i + 1 == G.na2 ? 0 : a2i + 1;
      if (++w1 == G.na1) { w1 = 0; ph1 ^= 1u; }
    }
    // weighted sum over the steps: out = S * K
    if (ok && __all_sync(0xffffffffu, mbar_wait(smem_u32(s_full), 0, 14))) {
      tc_fence_after_sync();
      const uint64_t da_step = (uint64_t)((2 * 128 * 16) >> 4);
      uint64_t da = make_desc_interleaved(smem_u32(ss), 128 * 16, 128);
      uint64_t db = make_desc_interleaved(smem_u32(kts), np * 16, 128);
      const uint64_t db3 = (uint64_t)((2 * np * 16) >> 4);
      for (int ks = 0; ks < tp / 16; ++ks) {
        mma_f16_ss_elect(tmem0 + G.c_acc3, da, db, p.idesc3, ks > 0 ? 1u : 0u);
        da += da_step; db += db3;
      }
    }
    mma_commit_elect(smem_u32(acc3_full));
  } else if (warp < TC_L2_WARP0) {
    // ---- layer-1 warpgroups: acc1 -> activation -> A2; warpgroup wb owns acc1 buffer wb and takes the steps
    //      j with j % na1 == wb (with two buffers the third warpgroup has nothing to do) -----------------------
    const int wb = warp >> 2;
    const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16);   // TMEM lane == candidate row of the tile
    if (wb == 0) {
      // the 16 columns every A2 buffer ends with: the constant 1 that carries bias b1, then zeros (fp16 pairs
      // per 32-bit column); complete before this warpgroup's first arrival on a2_full, which precedes every
      // layer-2 MMA
      tmem_st4(lane_addr + G.c_ones, 0x00003C00u, 0u, 0u, 0u);
      tmem_st4(lane_addr + G.c_ones + 4, 0u, 0u, 0u, 0u);
      tmem_wait_st();
    }
    bool ok = true;
    const int i1 = wb;
    const uint32_t acc1 = lane_addr + i1 * h0p;
    uint32_t ph1 = 0;                                         // (j / na1) & 1
    for (int j = wb < G.na1 ? wb : tl; j < tl; j += G.na1, ph1 ^= 1u) {
      const int a2i = j % G.na2;
      const uint32_t a2t = lane_addr + G.c_a2 + a2i * (h0p / 2);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc1_full[i1]), ph1, 20));
      if (!ok) break;
      tc_fence_after_sync();
      if (lane == 0 && (warp & 3) == 0) ATT_TR(wb, j, 0);
      // Blocks of 16 columns (8 fp16 pairs), as a two-stage software pipeline: stage one of block b+1 (convert,
      // tanh argument, SFU) is issued before stage two of block b (scale, multiply, store), so the SFU latency of
      // one block hides behind the arithmetic of the other instead of being exposed at every block boundary (the
      // tensor-memory instructions are ordered among themselves, which would otherwise serialise the blocks).
      constexpr int NBLK = H0 ? tc_geom(D0, H0, H1, 16).h0p / 16 : 8;
      const int nblk = H0 ? NBLK : h0p / 16;
      const uint4* __restrict__ cab = c1;                   // {A, B} of two column pairs per entry
      const uint4* __restrict__ ccd = c1 + h0p / 4;         // {C, D}
      uint32_t v[2][16], x[2][8], th[2][8];
      auto stage1 = [&](int blk, int s) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          x[s][e] = h2_bits(__floats2half2_rn(__uint_as_float(v[s][2 * e]), __uint_as_float(v[s][2 * e + 1])));
        if (ACT != XB_ACT_NONE) {
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const uint4 k = cab[4 * blk + e / 2];
            th[s][e] = umma::tanh_f16x2(h2_bits(__hfma2(bits_h2(x[s][e]), bits_h2(k.x), bits_h2(k.y))));
            th[s][e + 1] = umma::tanh_f16x2(h2_bits(__hfma2(bits_h2(x[s][e + 1]), bits_h2(k.z), bits_h2(k.w))));
          }
        }
      };
      auto stage2 = [&](int blk, int s) {
        uint32_t y[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          if (ACT == XB_ACT_NONE) { y[e] = x[s][e]; y[e + 1] = x[s][e + 1]; continue; }
          const uint4 k = ccd[4 * blk + e / 2];
          const __half2 g0 = __hfma2(bits_h2(th[s][e]), bits_h2(k.y), bits_h2(k.x));
          const __half2 g1 = __hfma2(bits_h2(th[s][e + 1]), bits_h2(k.w), bits_h2(k.z));
          y[e] = h2_bits(ACT == XB_ACT_DICE ? __hmul2(bits_h2(x[s][e]), g0) : g0);
          y[e + 1] = h2_bits(ACT == XB_ACT_DICE ? __hmul2(bits_h2(x[s][e + 1]), g1) : g1);
        }
        if (blk == 0) {
          // Before the first store: the layer-2 MMA that read this A2 buffer last (step j - na2) has completed.
          // Its commit also tells that its warp has seen a2_full of every step up to j - na2, which includes
          // this warpgroup's previous step (na2 <= na1), so the arrival that follows cannot run a2_full two
          // phases ahead of that warp.
          if (j >= G.na2) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&a2_free[a2i]), (uint32_t)((j - G.na2) / G.na2) & 1u, 23));
          }
          if (ok) tc_fence_after_sync();
        }
        if (ok) tmem_st8(a2t + 8 * blk, y);
      };
      // the accumulator's last block is in registers: every thread arrives, tied to a register of that block so
      // that the arrive is issued before the block's arithmetic, not after it
      auto release_acc1 = [&](uint32_t& dep) {
        tc_fence_before_sync();
        mbar_arrive_before(smem_u32(&acc1_free[i1]), dep);
      };
      tmem_ld16_nowait(acc1, v[0]);
      tmem_wait_ld(v[0]);
      if (nblk > 1) tmem_ld16_nowait(acc1 + 16, v[1]);
      else release_acc1(v[0][0]);
      stage1(0, 0);
#pragma unroll
      for (int blk = 0; blk < NBLK; ++blk) {
        if (blk < nblk && ok) {
          const int s = blk & 1;
          if (blk + 1 < nblk) {
            tmem_wait_ld(v[s ^ 1]);
            // v[s] was consumed by stage one of this block: its registers take the block after the next
            if (blk + 2 < nblk) tmem_ld16_nowait(acc1 + 16 * (blk + 2), v[s]);
            else release_acc1(v[s ^ 1][0]);
            stage1(blk + 1, s ^ 1);
          }
          stage2(blk, s);
        }
      }
      if (!ok) break;
      [[maybe_unused]] const long long tr1 = ATT_CLK();
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&a2_full[i1]));       // one arrival per warp
      if (lane == 0 && (warp & 3) == 0) {
        ATT_TR(wb, j, 1);
        ATT_TR_VAL(wb, j, 3, ATT_CLK() - tr1);
      }
    }
  } else if (warp >= TC_BUILD_WARP0) {
    // ---- builder warps: A1 of step t (buffer t % na1) as soon as the layer-1 MMA of step t - na1 has read it; a
    //      thread owns rows `row` and `row + 64` and loads each chunk of k_t once for both -----------------------
    const int row = (warp - TC_BUILD_WARP0) * 32 + lane;
    // q rows as 16-byte chunks (dp <= 64 -> at most 8), with the constant-1 column when it lives here
    uint4 qv[TC_BROWS][8];
#pragma unroll
    for (int h = 0; h < TC_BROWS; ++h)
#pragma unroll
      for (int c = 0; c < 8; ++c)
        qv[h][c] = c < nch ? *reinterpret_cast<const uint4*>(qs + (c * 128 + row + 64 * h) * 8) : make_uint4(0, 0, 0, 0);
    // constant part of both A1 buffers: the q segment and the chunks past the three segments (the constant 1
    // when q has no padding column for it, zeros otherwise); chunk c of row r is 16 bytes at c * (128 * 16) + r * 16
    for (int b = 0; b < G.na1; ++b) {
#pragma unroll
      for (int h = 0; h < TC_BROWS; ++h) {
        uint8_t* a1b = a1s + b * (128 * k1 * 2) + (row + 64 * h) * 16;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (c < nch) *reinterpret_cast<uint4*>(a1b + c * (128 * 16)) = qv[h][c];
        for (int c = 3 * nch; c < k1 / 8; ++c)
          *reinterpret_cast<uint4*>(a1b + c * (128 * 16)) =
              make_uint4((c == 3 * nch && G.ones1 == 3 * dp) ? 0x00003C00u : 0u, 0u, 0u, 0u);
      }
    }
    int bi = 0;                                               // t % na1: A1 buffer, and acc1 buffer of the MMA that reads it
    uint32_t bph = 0;                                         // (t / na1) & 1
    for (int t = 0; t < tl; ++t) {
      // the layer-1 MMA of step t - na1 read this buffer last
      if (t >= G.na1 && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&acc1_full[bi]), bph ^ 1u, 24))) break;
      if (lane == 0 && warp == TC_BUILD_WARP0) ATT_TR(6, t, 0);
      uint8_t* a1b = a1s + bi * (128 * k1 * 2) + row * 16;
      const uint4* kt = reinterpret_cast<const uint4*>(khs + t * dp);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < nch) {
          const uint4 kc = kt[c];
          const __half2* kh = reinterpret_cast<const __half2*>(&kc);
#pragma unroll
          for (int h = 0; h < TC_BROWS; ++h) {
            const __half2* qh = reinterpret_cast<const __half2*>(&qv[h][c]);
            uint4 pr;
            __half2* ph2 = reinterpret_cast<__half2*>(&pr);
#pragma unroll
            for (int e = 0; e < 4; ++e) ph2[e] = __hmul2(qh[e], kh[e]);
            // q's padding column holding the constant 1 gives 1*0 in `pr`; its W0 rows are zero anyway
            *reinterpret_cast<uint4*>(a1b + h * (64 * 16) + (nch + c) * (128 * 16)) = kc;
            *reinterpret_cast<uint4*>(a1b + h * (64 * 16) + (2 * nch + c) * (128 * 16)) = pr;
          }
        }
      }
      fence_proxy_async_smem();                               // the MMA reads A1 through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&a1_full[bi]));
      if (lane == 0 && warp == TC_BUILD_WARP0) ATT_TR(6, t, 1);
      if (++bi == G.na1) { bi = 0; bph ^= 1u; }
    }
  } else {
    // ---- layer-2 warpgroups: acc2 -> score -> S, steps of parity wb ------------------------------------
    const int wb = (warp >> 2) & 1;
    const int row = (warp & 3) * 32 + lane;
    const int n = tile * 128 + row;
    const bool valid = n < p.n_cand;
    const uint32_t lane_addr = tmem0 + ((uint32_t)((warp & 3) * 32) << 16);

    bool ok = true;
    const int npairs2 = (h1_ + 1) / 2;
    for (int j = wb; j < tl; j += 2) {
      const int b = wb;
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc2_full[b]), ph, 21));
      if (!ok) break;
      tc_fence_after_sync();
      if (lane == 0 && (warp & 3) == 0) ATT_TR(3 + wb, j, 2);
      const uint32_t acc2 = lane_addr + G.c_acc2 + b * h1p;
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
              const __half2 g = __hfma2(bits_h2(th[e]), bits_h2(cc[e].w), bits_h2(cc[e].z));
              part[e & 3] = ACT == XB_ACT_DICE ? __hfma2(bits_h2(x[e]), g, part[e & 3]) : __hadd2(part[e & 3], g);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc2_free[b]));
      if (lane == 0 && (warp & 3) == 0) ATT_TR(3 + wb, j, 3);
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

    if (lane == 0 && warp == 16) ATT_TR(6, 121, 0);
    if (wb == 0) ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(acc3_full), 0, 22));
    tc_fence_after_sync();
    if (lane == 0 && warp == 16) ATT_TR(6, 121, 1);
    if (ok && wb == 0) {
      __half* o = p.out + ((int64_t)r * p.n_cand + n) * p.ldo;
      // 8-byte stores when every row starts on an 8-byte boundary and d is a multiple of 4
      const bool vec = (d % 4 == 0) && (p.ldo % 4 == 0) && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0;
      for (int c = 0; c < np; c += 16) {
        float v[16];
        tmem_ld16(lane_addr + G.c_acc3 + c, v);
        if (valid) {
          if (vec) {
#pragma unroll
            for (int e = 0; e < 16; e += 4)
              if (c + e < d) {
                const __half2 lo = __floats2half2_rn(v[e], v[e + 1]), hi = __floats2half2_rn(v[e + 2], v[e + 3]);
                *reinterpret_cast<uint2*>(o + c + e) = make_uint2(h2_bits(lo), h2_bits(hi));
              }
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (c + e < d) o[c + e] = __float2half_rn(v[e]);
          }
        }
      }
    }
  }

  if (lane == 0 && warp == 16) ATT_TR(6, 121, 2);
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) ATT_TR(6, 121, 3);
  if (warp == MMA1_TC_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem0, TMEM_COLS);
  }
}

bool tc_eligible(const xb_din_att_args& a, int* why) {
  const TcGeom g = tc_geom(a.d, a.h0, a.h1, a.T);
  if (g.dp > 64) { if (why) *why = 1; return false; }
  if (g.h0p > 128 || g.h1p > 64) { if (why) *why = 2; return false; }
  if (g.tp > 256) { if (why) *why = 5; return false; }
  if (g.cols > TMEM_COLS || (g.c_acc3 == 0 && g.np > g.na1 * g.h0p)) { if (why) *why = 6; return false; }
  if (tc_layout(g, a.T).total > 220 * 1024) { if (why) *why = 3; return false; }
  if (a.use_softmax && a.scores) { if (why) *why = 4; return false; }   // normalised scores are not written out
  return true;
}

// the part of tc_eligible that depends on the weights' shape only
bool tc_eligible_shape(int d, int h0, int h1) {
  xb_din_att_args a;
  memset(&a, 0, sizeof(a));
  a.d = d; a.h0 = h0; a.h1 = h1; a.T = 16;
  return tc_eligible(a, nullptr);
}

size_t att_packed_bytes(int d, int h0, int h1) {
  const TcGeom g = tc_geom(d, h0, h1, 16);
  return (size_t)g.h0p * g.k1 * 2 + (size_t)g.h1p * g.k2 * 2 + (size_t)(g.h0p / 2 + g.h1p / 2) * 16;
}

int launch_att_pack(const AttParams& p, int act, void* dst, cudaStream_t stream) {
  if (act == XB_ACT_DICE) att_pack_kernel<XB_ACT_DICE><<<1, 256, 0, stream>>>(p, (uint8_t*)dst);
  else if (act == XB_ACT_SIGMOID) att_pack_kernel<XB_ACT_SIGMOID><<<1, 256, 0, stream>>>(p, (uint8_t*)dst);
  else att_pack_kernel<XB_ACT_NONE><<<1, 256, 0, stream>>>(p, (uint8_t*)dst);
  return check_launch("att_pack_kernel");
}

int launch_att_tc(AttParams& p, const xb_din_att_args& a, cudaStream_t stream) {
  const TcGeom g = tc_geom(a.d, a.h0, a.h1, a.T);
  p.tiles_per_req = (a.n_cand + 127) / 128;
  p.idesc1 = umma::make_idesc(128, g.h0p, 0);
  p.idesc2 = umma::make_idesc(128, g.h1p, 0);
  p.idesc3 = umma::make_idesc(128, g.np, 0);
  const TcSmemLayout L = tc_layout(g, p.T);
  static PerDeviceOnce attr_set;
  XB_SET_MAX_SMEM_ONCE(attr_set, 220 * 1024, (const void*)din_att_tc_kernel<XB_ACT_NONE, 0, 0, 0>,
                       (const void*)din_att_tc_kernel<XB_ACT_SIGMOID, 0, 0, 0>, (const void*)din_att_tc_kernel<XB_ACT_DICE, 0, 0, 0>,
                       (const void*)din_att_tc_kernel<XB_ACT_SIGMOID, 36, 80, 40>, (const void*)din_att_tc_kernel<XB_ACT_DICE, 36, 80, 40>);
  const int64_t blocks = (int64_t)a.requests * p.tiles_per_req;
  XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_din_attention: too many tiles");
  // the shape of the DIN / DIEN attention unit (d = 36, MLP 144-80-40-1) has instantiations of its own
  const bool din_shape = a.d == 36 && a.h0 == 80 && a.h1 == 40;
  if (din_shape && a.act == XB_ACT_DICE) din_att_tc_kernel<XB_ACT_DICE, 36, 80, 40><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  else if (din_shape && a.act == XB_ACT_SIGMOID) din_att_tc_kernel<XB_ACT_SIGMOID, 36, 80, 40><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  else if (a.act == XB_ACT_DICE) din_att_tc_kernel<XB_ACT_DICE, 0, 0, 0><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  else if (a.act == XB_ACT_SIGMOID) din_att_tc_kernel<XB_ACT_SIGMOID, 0, 0, 0><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  else din_att_tc_kernel<XB_ACT_NONE, 0, 0, 0><<<(unsigned)blocks, TC_THREADS, L.total, stream>>>(p);
  return check_launch("din_att_tc_kernel");
}

}  // namespace
}  // namespace xb
