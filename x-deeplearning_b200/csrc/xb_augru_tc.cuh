// Attention-gated GRU (AUGRU) of the DIEN-style model on the tensor cores (included by xb_rnn.cu).
//
// Every candidate of a request walks the SAME input sequence x[r] (the interest-extractor states) with its own
// attention scores, so for candidate n and step t
//   [r|u] = sigmoid(h Wg_h + (x_t Wg_x + bg)),  c = tanh((r*h) Wc_h + (x_t Wc_x + bc)),
//   u' = (1 - a[n,t]) u,  h' = u' h + (1 - u') c
// where the bracketed terms depend on the request and the step only. One CTA owns 128 candidates of one request
// and walks the T steps on chip: the two per-candidate products are tcgen05 MMAs (A = h, then r*h, as fp16 in
// tensor memory; the recurrent weights stay in shared memory), and the request-side terms enter the same MMAs
// through a selector slot of the A operand (a 1 in the slot of the current step against B rows that hold the
// precomputed x_t terms), exactly as the split attention engine feeds its per-step bias. The state h stays in
// fp32 registers; it is rounded to fp16 only as an MMA operand. Only the final state is written (the model reads
// nothing else), the input sequence is read once per CTA instead of once per candidate.
//
// Cell semantics: VecAttGRUCell.call, xdl-algorithm-solution/DIEN/script/utils.py:178-207 (the reference ships no
// inference operator for it). Shapes: H padded to Hp = 8*ceil(H/8) must leave 4 or more spare slots (H = 36 does).
#pragma once

namespace xb {
namespace {

constexpr int AU_THREADS = 160;           // 4 worker warps (one candidate row per thread) + 1 MMA-issuing warp
constexpr int AU_MMA_WARP = 4;

struct AuGeom {
  int hp, nch, selpos, k, n1, n2, ngrp;   // k: MMA K (h, selector slots, zero chunk); n1 = pad16(2H), n2 = pad16(H)
  int blk1, blk2;                         // bytes of one 8-wide k chunk of B1 / B2
  int c_acc2, c_a1, c_a2, cols, tmem_cols;
  int o_b1, o_b2, o_att, o_x, total;      // shared memory
};

__host__ __device__ inline AuGeom au_geom(int H, int T) {
  AuGeom g;
  g.hp = (H + 7) / 8 * 8;
  g.nch = g.hp / 8;
  g.selpos = H & 7;
  g.k = (g.hp + 15) / 16 * 16;                 // the chunk after the last h chunk, if any, is all zero
  g.n1 = (2 * H + 15) / 16 * 16;
  g.n2 = (H + 15) / 16 * 16;
  g.ngrp = (T + 3) / 4;
  g.blk1 = g.n1 * 16;
  g.blk2 = g.n2 * 16;
  g.c_acc2 = g.n1;
  g.c_a1 = g.n1 + g.n2;
  g.c_a2 = g.c_a1 + g.k / 2;
  g.cols = g.c_a2 + g.k / 2;
  g.tmem_cols = g.cols <= 32 ? 32 : g.cols <= 64 ? 64 : g.cols <= 128 ? 128 : g.cols <= 256 ? 256 : 512;
  // B operands: [weight chunks 0..nch-2][selector blocks 0..ngrp-1][zero block], ascending in k
  int off = 0;
  g.o_b1 = off; off += (g.nch - 1 + g.ngrp + 1) * g.blk1;
  g.o_b2 = off; off += (g.nch - 1 + g.ngrp + 1) * g.blk2;
  g.o_att = off; off += 128 * ((T + 7) / 8 * 8) * 2;     // attention scores of the tile, [128][Tp] fp16
  g.o_x = off; off += T * g.hp * 2;                      // input sequence of the request, fp16
  g.total = (off + 15) / 16 * 16;
  return g;
}

struct AuParams {
  const __half* x; const __half* att; __half* y;
  const __half *Wg, *bg, *Wc, *bc;
  int requests, n_cand, T, H, tiles_per_req;
  uint32_t idesc1, idesc2;
};

// byte offset of k chunk c (for selector group grp) inside a B operand whose chunk blocks are `blk` bytes
__device__ __forceinline__ int au_chunk_off(const AuGeom& g, int blk, int c, int grp) {
  if (c < g.nch - 1) return c * blk;
  if (c == g.nch - 1) return (g.nch - 1 + grp) * blk;
  return (g.nch - 1 + g.ngrp) * blk;
}

// HP2: compile-time bound of the fp16 pairs of a state row (the state lives in registers)
template <int HP2>
__global__ void __launch_bounds__(AU_THREADS, 2) augru_tc_kernel(const __grid_constant__ AuParams p) {
  using namespace umma;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[4];
  __shared__ uint32_t tmem_base_s;
  const AuGeom G = au_geom(p.H, p.T);
  const int H = p.H, T = p.T, hp = G.hp, nch = G.nch, tpp = (T + 7) / 8 * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x / p.tiles_per_req, tile = blockIdx.x % p.tiles_per_req;
  const int rows = min(128, p.n_cand - tile * 128);
  uint8_t* b1s = smem + G.o_b1;
  uint8_t* b2s = smem + G.o_b2;
  __half* atts = reinterpret_cast<__half*>(smem + G.o_att);
  __half* xs = reinterpret_cast<__half*>(smem + G.o_x);
  const __half zero = __float2half(0.f);

  // ---- prologue -------------------------------------------------------------------------------------------
  // attention scores of the tile and the request's input sequence: asynchronous copies where alignment allows
  const __half* att_tile = p.att + ((int64_t)r * p.n_cand + tile * 128) * T;
  const bool a8 = (T % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.att) & 7) == 0);
  if (a8) {
    for (int idx = threadIdx.x; idx < rows * (T / 4); idx += AU_THREADS) {
      const int row = idx / (T / 4), pc = idx - row * (T / 4);
      cp_async8(atts + row * tpp + pc * 4, att_tile + (int64_t)row * T + pc * 4);
    }
  } else {
    for (int idx = threadIdx.x; idx < rows * T; idx += AU_THREADS) atts[(idx / T) * tpp + idx % T] = att_tile[idx];
  }
  const __half* xr = p.x + (int64_t)r * T * H;
  for (int idx = threadIdx.x; idx < T * hp; idx += AU_THREADS) {
    const int t = idx / hp, i = idx - t * hp;
    xs[idx] = i < H ? xr[t * H + i] : zero;
  }
  cp_async_commit();
  // recurrent weights as MMA B operands (row n = output column, k = index into h): chunk-major 8 x 16-byte blocks;
  // the last h chunk shares its block with the selector slots and is replicated into every selector block
  for (int idx = threadIdx.x; idx < G.n1 * hp; idx += AU_THREADS) {
    const int n = idx / hp, i = idx - n * hp;
    const __half v = (n < 2 * H && i < H) ? p.Wg[(int64_t)(H + i) * 2 * H + n] : zero;
    const int c = i >> 3, e = i & 7;
    if (c < nch - 1) reinterpret_cast<__half*>(b1s + c * G.blk1)[n * 8 + e] = v;
    else for (int g = 0; g < G.ngrp; ++g) reinterpret_cast<__half*>(b1s + (nch - 1 + g) * G.blk1)[n * 8 + e] = v;
  }
  for (int idx = threadIdx.x; idx < G.n2 * hp; idx += AU_THREADS) {
    const int n = idx / hp, i = idx - n * hp;
    const __half v = (n < H && i < H) ? p.Wc[(int64_t)(H + i) * H + n] : zero;
    const int c = i >> 3, e = i & 7;
    if (c < nch - 1) reinterpret_cast<__half*>(b2s + c * G.blk2)[n * 8 + e] = v;
    else for (int g = 0; g < G.ngrp; ++g) reinterpret_cast<__half*>(b2s + (nch - 1 + g) * G.blk2)[n * 8 + e] = v;
  }
  for (int i = threadIdx.x; i < G.blk1 / 16; i += AU_THREADS)
    reinterpret_cast<uint4*>(b1s + (nch - 1 + G.ngrp) * G.blk1)[i] = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < G.blk2 / 16; i += AU_THREADS)
    reinterpret_cast<uint4*>(b2s + (nch - 1 + G.ngrp) * G.blk2)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();                       // xs and the weight blocks are in place
  // request-side terms into the selector slots: slot t % 4 of selector block t / 4 holds, for output column n,
  //   B1: x_t Wg_x[:, n] + bg[n]      B2: x_t Wc_x[:, n] + bc[n]     (fp32 sums, rounded once)
  for (int idx = threadIdx.x; idx < G.ngrp * 4 * (G.n1 + G.n2); idx += AU_THREADS) {
    const int t = idx / (G.n1 + G.n2), nn = idx - t * (G.n1 + G.n2);
    const bool first = nn < G.n1;
    const int n = first ? nn : nn - G.n1;
    const int width = first ? 2 * H : H;
    float v = 0.f;
    if (t < T && n < width) {
      const __half* W = first ? p.Wg : p.Wc;
      v = __half2float(first ? p.bg[n] : p.bc[n]);
      for (int i = 0; i < H; ++i) v = fmaf(__half2float(xs[t * hp + i]), __half2float(__ldg(W + (int64_t)i * width + n)), v);
    }
    uint8_t* blk = first ? b1s + (nch - 1 + t / 4) * G.blk1 : b2s + (nch - 1 + t / 4) * G.blk2;
    reinterpret_cast<__half*>(blk)[n * 8 + G.selpos + (t & 3)] = __float2half_rn(v);
  }
  // barriers: a1_full (4 worker warps: h operand of a step written), acc1_full (gate product done),
  //           a2_full (4 worker warps: r*h written), acc2_full (candidate product done)
  uint64_t* a1_full = &bars[0];
  uint64_t* acc1_full = &bars[1];
  uint64_t* a2_full = &bars[2];
  uint64_t* acc2_full = &bars[3];
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(a1_full), 4);
    mbar_init(smem_u32(acc1_full), 1);
    mbar_init(smem_u32(a2_full), 4);
    mbar_init(smem_u32(acc2_full), 1);
    fence_barrier_init();
  }
  if (warp == AU_MMA_WARP) tmem_alloc(smem_u32(&tmem_base_s), (uint32_t)G.tmem_cols);
  cp_async_wait_all();
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = tmem_base_s;

  if (warp == AU_MMA_WARP) {
    // whole warp in uniform control flow, one elected lane issues: the descriptors stay in uniform registers
    {
      const int nks = G.k / 16, sel_ks = (nch - 1) / 2;            // nks <= 4 (H <= 64)
      const uint32_t b1a = smem_u32(b1s), b2a = smem_u32(b2s);
      // descriptors for selector group 0; only the k step with the selector chunk moves with the group
      uint64_t d1[4], d2[4], delta1 = 0, delta2 = 0;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        d1[ks] = d2[ks] = 0;
        if (ks < nks) {
          const uint32_t o0 = au_chunk_off(G, G.blk1, 2 * ks, 0), o1 = au_chunk_off(G, G.blk1, 2 * ks + 1, 0);
          const uint32_t q0 = au_chunk_off(G, G.blk2, 2 * ks, 0), q1 = au_chunk_off(G, G.blk2, 2 * ks + 1, 0);
          d1[ks] = make_desc_interleaved(b1a + o0, o1 - o0, 128);
          d2[ks] = make_desc_interleaved(b2a + q0, q1 - q0, 128);
          if (ks == sel_ks && G.ngrp > 1) {
            const uint32_t r0 = au_chunk_off(G, G.blk1, 2 * ks, 1), r1 = au_chunk_off(G, G.blk1, 2 * ks + 1, 1);
            const uint32_t s0 = au_chunk_off(G, G.blk2, 2 * ks, 1), s1 = au_chunk_off(G, G.blk2, 2 * ks + 1, 1);
            delta1 = make_desc_interleaved(b1a + r0, r1 - r0, 128) - d1[ks];
            delta2 = make_desc_interleaved(b2a + s0, s1 - s0, 128) - d2[ks];
          }
        }
      }
      for (int t = 0; t < T; ++t) {
        const uint32_t ph = (uint32_t)t & 1u;
        const uint64_t grp = (uint64_t)(t >> 2);
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(a1_full), ph, 30))) break;
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          if (ks < nks)
            mma_f16_ts_elect(tmem0, tmem0 + G.c_a1 + 8 * ks, d1[ks] + (ks == sel_ks ? grp * delta1 : 0ull), p.idesc1, ks > 0 ? 1u : 0u);
        mma_commit_elect(smem_u32(acc1_full));
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(a2_full), ph, 31))) break;
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          if (ks < nks)
            mma_f16_ts_elect(tmem0 + G.c_acc2, tmem0 + G.c_a2 + 8 * ks, d2[ks] + (ks == sel_ks ? grp * delta2 : 0ull), p.idesc2,
                             ks > 0 ? 1u : 0u);
        mma_commit_elect(smem_u32(acc2_full));
      }
    }
  } else {
    const int row = warp * 32 + lane;
    const bool valid = row < rows;
    const uint32_t lane_addr = tmem0 + ((uint32_t)(warp * 32) << 16);
    const uint32_t a1t = lane_addr + G.c_a1, a2t = lane_addr + G.c_a2;
    float h[2 * HP2];
#pragma unroll
    for (int i = 0; i < 2 * HP2; ++i) h[i] = 0.f;
    // an A operand row: chunks of 8 halves = 4 tensor-memory columns; chunk nch-1 carries the selector slots,
    // the chunk after it (if k > hp) stays zero
    auto store_operand = [&](uint32_t at, const uint32_t* pk /* hp/2 packed pairs */, int t) {
      const int hpos = G.selpos + (t & 3);
#pragma unroll
      for (int c = 0; c < HP2 / 4; ++c) {
        if (c < nch) {
          uint32_t w0 = pk[4 * c], w1 = pk[4 * c + 1], w2 = pk[4 * c + 2], w3 = pk[4 * c + 3];
          if (c == nch - 1) {
            const uint32_t one = 0x3C00u << ((hpos & 1) * 16);
            const int reg = hpos >> 1;
            w0 |= reg == 0 ? one : 0u; w1 |= reg == 1 ? one : 0u; w2 |= reg == 2 ? one : 0u; w3 |= reg == 3 ? one : 0u;
          }
          tmem_st4(at + 4 * c, w0, w1, w2, w3);
        }
      }
    };
    uint32_t pk[HP2];
#pragma unroll
    for (int i = 0; i < HP2; ++i) pk[i] = 0u;
    if (G.k > hp) {
      tmem_st4(a1t + 4 * nch, 0u, 0u, 0u, 0u);
      tmem_st4(a2t + 4 * nch, 0u, 0u, 0u, 0u);
    }
    store_operand(a1t, pk, 0);             // h_0 = 0 with the selector of step 0
    tmem_wait_st();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(a1_full));
    bool ok = true;
    const int npair = (H + 1) / 2;
    for (int t = 0; t < T && ok; ++t) {
      const uint32_t ph = (uint32_t)t & 1u;
      // ---- gates: [r|u] = sigmoid(acc1); r*h becomes the A operand of the candidate product
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc1_full), ph, 32));
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t upk[HP2];                   // update gate as fp16 pairs
#pragma unroll
      for (int blk = 0; blk < (4 * HP2 + 15) / 16; ++blk) {
        if (blk * 16 < 2 * H) {
          uint32_t v[16];
          tmem_ld16_nowait(lane_addr + 16 * blk, v);
          tmem_wait_ld(v);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = blk * 16 + 2 * e;            // columns col, col + 1 of [r | u]
            if (col < 2 * H) {
              // sigmoid(z) = 1/2 + 1/2 tanh(z/2), two columns per SFU instruction
              const __half2 z = __floats2half2_rn(0.5f * __uint_as_float(v[2 * e]), 0.5f * __uint_as_float(v[2 * e + 1]));
              const __half2 th = bits_h2(tanh_f16x2(h2_bits(z)));
              const __half2 sg = __hfma2(th, __floats2half2_rn(0.5f, 0.5f), __floats2half2_rn(0.5f, 0.5f));
              if (col < H) {
                // reset gate: r * h (H is even in every supported shape, so a pair never straddles r | u)
                const float2 rf = __half22float2(sg);
                pk[col >> 1] = h2_bits(__floats2half2_rn(rf.x * h[col], col + 1 < H ? rf.y * h[col + 1] : 0.f));
              } else {
                upk[(col - H) >> 1] = h2_bits(sg);
              }
            }
          }
        }
      }
      store_operand(a2t, pk, t);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(a2_full));
      // ---- candidate and blend
      const float a = __half2float(atts[row * tpp + t]);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc2_full), ph, 33));
      if (!ok) break;
      tc_fence_after_sync();
#pragma unroll
      for (int blk = 0; blk < (2 * HP2 + 15) / 16; ++blk) {
        if (blk * 16 < H) {
          uint32_t v[16];
          tmem_ld16_nowait(lane_addr + G.c_acc2 + 16 * blk, v);
          tmem_wait_ld(v);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = blk * 16 + 2 * e;
            if (col < H) {
              const __half2 z = __floats2half2_rn(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
              const float2 c = __half22float2(bits_h2(tanh_f16x2(h2_bits(z))));
              const float2 u = __half22float2(bits_h2(upk[col >> 1]));
              const float u0 = (1.f - a) * u.x, u1 = (1.f - a) * u.y;
              h[col] = u0 * h[col] + (1.f - u0) * c.x;
              if (col + 1 < H) h[col + 1] = u1 * h[col + 1] + (1.f - u1) * c.y;
              pk[col >> 1] = h2_bits(__floats2half2_rn(h[col], col + 1 < H ? h[col + 1] : 0.f));
            }
          }
        }
      }
      if (t + 1 < T) {
        store_operand(a1t, pk, t + 1);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(a1_full));
      }
    }
    if (ok && valid) {
      __half* o = p.y + ((int64_t)r * p.n_cand + tile * 128 + row) * H;
#pragma unroll
      for (int i = 0; i < HP2; ++i)
        if (i < npair) *reinterpret_cast<uint32_t*>(o + 2 * i) = pk[i];      // H is even: whole pairs, 4-byte aligned
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == AU_MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem0, (uint32_t)G.tmem_cols);
  }
}

bool augru_tc_eligible(int H, int T) {
  if (H < 4 || H > 64 || (H & 1)) return false;
  const AuGeom g = au_geom(H, T);
  if (g.hp - H < 4) return false;                     // selector slots live in the padding of the last h chunk
  if (g.cols > 512 || g.n1 > 256) return false;
  return g.total <= 200 * 1024 && T >= 1;
}

int launch_augru_tc(const AuParams& p0, cudaStream_t stream) {
  AuParams p = p0;
  const AuGeom g = au_geom(p.H, p.T);
  p.tiles_per_req = (p.n_cand + 127) / 128;
  p.idesc1 = umma::make_idesc(128, g.n1, 0);
  p.idesc2 = umma::make_idesc(128, g.n2, 0);
  const int64_t blocks = (int64_t)p.requests * p.tiles_per_req;
  XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_augru_shared: too many tiles");
  static PerDeviceOnce attr;
  XB_SET_MAX_SMEM_ONCE(attr, 200 * 1024, (const void*)augru_tc_kernel<20>, (const void*)augru_tc_kernel<32>);
  if (g.hp <= 40) augru_tc_kernel<20><<<(unsigned)blocks, AU_THREADS, g.total, stream>>>(p);
  else augru_tc_kernel<32><<<(unsigned)blocks, AU_THREADS, g.total, stream>>>(p);
  return check_launch("augru_tc_kernel");
}

}  // namespace
}  // namespace xb
