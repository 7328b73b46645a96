// Fused DIN attention unit.
//
// For every (candidate n, behaviour step t) pair of a request the unit runs a
// three-layer MLP on x = [q_n, k_t, q_n-k_t, q_n*k_t] and sums k_t weighted by
// the resulting score. Nothing but q, k and the [n_cand, d] result touches HBM.
//
// Two engines: the tcgen05 engine (xb_din_attention_tc.cuh) and, in this file, a
// CUDA-core engine that does the same arithmetic in fp32 without intermediate
// rounding, one CTA per candidate; it serves shapes the tcgen05 engine does not
// take and cross-checks it in the tests.
#include <algorithm>
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
  // tcgen05 engine
  int tiles_per_req, tiles_per_cta;
  uint32_t idesc1, idesc2, idesc3;
  const void* packed;      // weight operands laid out by xb_din_attention_pack, or null
};

__device__ __forceinline__ float att_act(int act, float x, float g, float a, float bneg) {
  // a = rstd, bneg = -mean*rstd (Dice); g = gamma
  if (act == XB_ACT_DICE) {
    float p = __fdividef(1.f, 1.f + __expf(-fmaf(x, a, bneg)));
    return x * fmaf(p, 1.f - g, g);
  }
  if (act == XB_ACT_SIGMOID) return __fdividef(1.f, 1.f + __expf(-x));
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

}  // namespace
}  // namespace xb

#include "xb_din_attention_tc.cuh"
#include "xb_din_attention_pair.cuh"
#include "xb_din_attention_split.cuh"

namespace xb {

int att_status(int* out) { return umma::read_status_word(out); }
int att_clear_status() { return umma::clear_status_word(); }
int att_set_status_mirror(int* p) { return umma::set_status_mirror(p); }

}  // namespace xb

using namespace xb;

// The packed image: per-step engine's operands, then the step-pair engine's, then the split engine's.
static size_t split_image_offset(int d, int h0, int h1) {
  size_t n = 0;
  if (tc_eligible_shape(d, h0, h1)) n += (att_packed_bytes(d, h0, h1) + 15) / 16 * 16;
  if (pair_image_wanted(d, h0, h1)) n += (att_pair_packed_bytes(d, h0, h1) + 15) / 16 * 16;
  return n;
}

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
  p.packed = a->w.packed;

  int why = 0;
  // The packed image holds the per-step engine's operands first and, when the shape allows, the step-pair
  // engine's after them. The step-pair engine runs on request only: it halves the tensor-pipe time but both
  // engines end up bound by the activation math, and it rounds in different places.
  if (a->engine == XB_ATT_ENGINE_PAIR) {
    XB_REQUIRE(a->w.packed && pair_image_wanted(a->d, a->h0, a->h1) && pair_eligible(*a, &why), XB_ERR_UNSUPPORTED,
               "xb_din_attention: shape outside the step-pair engine (reason %d; it needs packed weights)", why);
    const size_t first = tc_eligible_shape(a->d, a->h0, a->h1) ? att_packed_bytes(a->d, a->h0, a->h1) : 0;
    p.packed = (const char*)a->w.packed + (first + 15) / 16 * 16;
    return launch_att_pair(p, *a, stream);
  }
  // The split engine (the request-side term of layer 1 looked up through a selector column, persistent CTAs)
  // runs on request only: it issues fewer MMAs but measures slower than the per-step engine.
  if (a->engine == XB_ATT_ENGINE_SPLIT && a->w.packed && split_eligible(*a, &why)) {
    p.packed = (const char*)a->w.packed + split_image_offset(a->d, a->h0, a->h1);
    return launch_att_split(p, *a, stream);
  }
  XB_REQUIRE(a->engine != XB_ATT_ENGINE_SPLIT, XB_ERR_UNSUPPORTED,
             "xb_din_attention: shape outside the split engine (reason %d; it needs packed weights)", why);
  const bool tc = a->engine != XB_GEMM_SIMT && tc_eligible(*a, &why);
  XB_REQUIRE(tc || a->engine != XB_GEMM_TCGEN05, XB_ERR_UNSUPPORTED,
             "xb_din_attention: shape outside the tcgen05 engine (reason %d)", why);
  if (tc) return launch_att_tc(p, *a, stream);
  const size_t smem = sizeof(float) * ((size_t)a->d + (size_t)a->h0 * SIMT_THREADS + a->T + SIMT_THREADS);
  XB_REQUIRE(smem <= 200 * 1024, XB_ERR_LIMIT, "xb_din_attention: shape too large for the CUDA-core engine");
  XB_REQUIRE(a->requests <= 65535, XB_ERR_LIMIT, "xb_din_attention: more than 65535 requests per call");
  static PerDeviceOnce simt_attr;
  XB_SET_MAX_SMEM_ONCE(simt_attr, 200 * 1024, (const void*)din_att_simt_kernel);
  dim3 grid(a->n_cand, a->requests);
  din_att_simt_kernel<<<grid, SIMT_THREADS, smem, stream>>>(p);
  return check_launch("din_att_simt_kernel");
}

#ifdef XB_ATT_TRACE
extern "C" int xb_debug_att_trace(long long* host) {
  return cudaMemcpyFromSymbol(host, xb::g_att_trace, sizeof(long long) * 7 * 128 * 4) == cudaSuccess ? 0 : 1;
}
#endif

extern "C" size_t xb_din_attention_packed_bytes(int32_t d, int32_t h0, int32_t h1) {
  if (d <= 0 || h0 <= 0 || h1 <= 0) return 0;
  size_t n = 0;
  if (tc_eligible_shape(d, h0, h1)) n += (att_packed_bytes(d, h0, h1) + 15) / 16 * 16;
  if (pair_image_wanted(d, h0, h1)) n += (att_pair_packed_bytes(d, h0, h1) + 15) / 16 * 16;
  if (split_eligible_shape(d, h0, h1)) n += att_split_packed_bytes(d, h0, h1);
  return n;
}

extern "C" int xb_din_attention_pack(const xb_din_att_args* a, void* packed, size_t bytes, xb_stream_t stream) {
  XB_REQUIRE(a && packed, XB_ERR_ARG, "xb_din_attention_pack: null argument");
  XB_REQUIRE(a->w.W0 && a->w.W1 && a->w.W2, XB_ERR_ARG, "xb_din_attention_pack: missing weights");
  XB_REQUIRE(a->act != XB_ACT_DICE || (a->w.gamma0 && a->w.mean0 && a->w.var0 && a->w.gamma1 && a->w.mean1 && a->w.var1),
             XB_ERR_ARG, "xb_din_attention_pack: Dice needs gamma/mean/var for both layers");
  const size_t need = xb_din_attention_packed_bytes(a->d, a->h0, a->h1);
  XB_REQUIRE(need != 0, XB_ERR_UNSUPPORTED, "xb_din_attention_pack: shape outside the tcgen05 engine");
  XB_REQUIRE(bytes >= need && ((uintptr_t)packed & 15) == 0, XB_ERR_ARG, "xb_din_attention_pack: buffer of %zu bytes, need %zu, 16-byte aligned", bytes, need);
  AttParams p;
  memset(&p, 0, sizeof(p));
  p.T = 16; p.d = a->d; p.h0 = a->h0; p.h1 = a->h1; p.act = a->act;
  p.W0 = (const __half*)a->w.W0; p.W1 = (const __half*)a->w.W1; p.W2 = a->w.W2;
  p.b0 = a->w.b0; p.b1 = a->w.b1; p.b2 = a->w.b2;
  p.g0 = a->w.gamma0; p.m0 = a->w.mean0; p.v0 = a->w.var0;
  p.g1 = a->w.gamma1; p.m1 = a->w.mean1; p.v1 = a->w.var1;
  size_t first = 0;
  if (tc_eligible_shape(a->d, a->h0, a->h1)) {
    if (int rc = launch_att_pack(p, a->act, packed, (cudaStream_t)stream)) return rc;
    first = (att_packed_bytes(a->d, a->h0, a->h1) + 15) / 16 * 16;
  }
  if (pair_image_wanted(a->d, a->h0, a->h1))
    if (int rc = launch_att_pair_pack(p, a->act, (char*)packed + first, (cudaStream_t)stream)) return rc;
  if (split_eligible_shape(a->d, a->h0, a->h1))
    return launch_att_split_pack(p, a->act, (char*)packed + split_image_offset(a->d, a->h0, a->h1), (cudaStream_t)stream);
  return 0;
}
