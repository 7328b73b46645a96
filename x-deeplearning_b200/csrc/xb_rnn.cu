// GRU and attention-gated GRU (AUGRU) over short behaviour sequences.
//
// One CTA owns one sequence and walks its T steps; the recurrent weights live
// in shared memory as fp32 for the whole walk, the hidden state in shared
// memory between steps. With H = 36 a step is 2 x 36 x 108 multiply-adds, so a
// sequence never leaves its SM and needs no inter-CTA synchronisation (the
// reference CUDA GRU spins on global atomics between blocks,
// blaze/blaze/operator/op/gru_op.cu:73-85; nothing here waits on another CTA).
// Latency-bound by design: throughput comes from batch-many independent CTAs.
#include <cstring>

#include "xb_common.cuh"
#include "xb_umma.cuh"

namespace xb {
namespace {

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

__device__ __forceinline__ float sigm(float v) { return 1.f / (1.f + expf(-v)); }

// x [B,T,H], y [B,T,H]; i2h, h2h [H,3H] (gate order r, z, candidate); biases [3H].
// Follows GRUKernel, blaze/blaze/operator/op/gru_op.cc:33-93: leading steps whose first H
// input pre-activations (before the bias) are all zero emit zeros and leave h at zero.
__global__ void gru_kernel(const void* x, void* y, int T, int H, const void* i2h, const void* h2h, const void* bi,
                           const void* bh, int dt) {
  extern __shared__ float sm[];
  float* Wi = sm;                    // [H][3H]
  float* Wh = Wi + H * 3 * H;        // [H][3H]
  float* h = Wh + H * 3 * H;         // [H]
  float* xs = h + H;                 // [H]
  float* pre = xs + H;               // [3H]
  float* act = pre + 3 * H;          // [3H]
  const int j = threadIdx.x, G = 3 * H;
  const int64_t b = blockIdx.x;
  for (int i = j; i < H * G; i += blockDim.x) { Wi[i] = load_as_f32(i2h, i, dt); Wh[i] = load_as_f32(h2h, i, dt); }
  if (j < H) h[j] = 0.f;
  const float bij = j < G ? load_as_f32(bi, j, dt) : 0.f, bhj = j < G ? load_as_f32(bh, j, dt) : 0.f;
  bool started = false;
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const int64_t base = (b * T + t) * H;
    if (j < H) xs[j] = load_as_f32(x, base + j, dt);
    __syncthreads();
    float p = 0.f, a = 0.f;
    if (j < G) {
      for (int k = 0; k < H; ++k) { p = fmaf(xs[k], Wi[k * G + j], p); a = fmaf(h[k], Wh[k * G + j], a); }
    }
    if (!started) started = __syncthreads_or(j < H && p != 0.f) != 0;
    if (!started) {
      if (j < H) store_from_f32(y, base + j, dt, 0.f);
      __syncthreads();
      continue;
    }
    if (j < G) { pre[j] = p + bij; act[j] = a + bhj; }
    __syncthreads();
    float out = 0.f;
    if (j < H) {
      const float r = sigm(pre[j] + act[j]);
      const float z = sigm(pre[H + j] + act[H + j]);
      const float c = tanhf(pre[2 * H + j] + r * act[2 * H + j]);
      out = c + z * (h[j] - c);
      store_from_f32(y, base + j, dt, out);
    }
    __syncthreads();
    if (j < H) h[j] = out;
  }
}

// AUGRU after VecAttGRUCell.call (xdl-algorithm-solution/DIEN/script/utils.py:139-207):
// [r|u] = sigmoid([x,h] Wg + bg); c = tanh([x, r*h] Wc + bc); u' = (1 - a_t) u; h' = u' h + (1 - u') c.
// Wg [2H, 2H] (rows x then h; columns r then u), Wc [2H, H]; att [B, T].
// `share` > 0: the input sequence is shared by groups of `share` consecutive batch entries (x is [B / share, T, H],
// the candidates of one request), and only the final state is written (y is [B, H]).
__global__ void augru_kernel(const void* x, const void* att, void* y, int T, int H, const void* Wg_, const void* bg_,
                             const void* Wc_, const void* bc_, int dt, int share) {
  extern __shared__ float sm[];
  float* Wg = sm;                     // [2H][2H]
  float* Wc = Wg + 4 * H * H;         // [2H][H]
  float* h = Wc + 2 * H * H;          // [H]
  float* xs = h + H;                  // [H]
  float* g = xs + H;                  // [2H]
  float* rh = g + 2 * H;              // [H]
  const int j = threadIdx.x, G = 2 * H;
  const int64_t b = blockIdx.x;
  for (int i = j; i < 4 * H * H; i += blockDim.x) Wg[i] = load_as_f32(Wg_, i, dt);
  for (int i = j; i < 2 * H * H; i += blockDim.x) Wc[i] = load_as_f32(Wc_, i, dt);
  if (j < H) h[j] = 0.f;
  const float bgj = j < G ? load_as_f32(bg_, j, dt) : 0.f, bcj = j < H ? load_as_f32(bc_, j, dt) : 0.f;
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const int64_t base = (b * T + t) * H;
    const int64_t xbase = share > 0 ? ((b / share) * T + t) * H : base;
    if (j < H) xs[j] = load_as_f32(x, xbase + j, dt);
    __syncthreads();
    if (j < G) {
      float s = bgj;
      for (int k = 0; k < H; ++k) s = fmaf(xs[k], Wg[k * G + j], s);
      for (int k = 0; k < H; ++k) s = fmaf(h[k], Wg[(H + k) * G + j], s);
      g[j] = sigm(s);
    }
    __syncthreads();
    if (j < H) rh[j] = g[j] * h[j];
    __syncthreads();
    float out = 0.f;
    if (j < H) {
      float s = bcj;
      for (int k = 0; k < H; ++k) s = fmaf(xs[k], Wc[k * H + j], s);
      for (int k = 0; k < H; ++k) s = fmaf(rh[k], Wc[(H + k) * H + j], s);
      const float a = load_as_f32(att, b * T + t, dt);
      const float u = (1.f - a) * g[H + j];
      out = u * h[j] + (1.f - u) * tanhf(s);
      if (share <= 0) store_from_f32(y, base + j, dt, out);
      else if (t == T - 1) store_from_f32(y, b * H + j, dt, out);
    }
    __syncthreads();
    if (j < H) h[j] = out;
  }
}

}  // namespace
}  // namespace xb

#include "xb_augru_tc.cuh"

namespace xb {
int rnn_status(int* out) { return umma::read_status_word(out); }
int rnn_clear_status() { return umma::clear_status_word(); }
int rnn_set_status_mirror(int* p) { return umma::set_status_mirror(p); }
}  // namespace xb

using namespace xb;

extern "C" int xb_gru(const void* x, void* y, int64_t batch, int32_t T, int32_t H, const void* i2h, const void* h2h,
                      const void* i2h_bias, const void* h2h_bias, int32_t dtype, xb_stream_t s) {
  XB_REQUIRE(x && y && i2h && h2h && i2h_bias && h2h_bias, XB_ERR_ARG, "xb_gru: null tensor");
  XB_REQUIRE(batch >= 0 && T >= 0 && H >= 1, XB_ERR_ARG, "xb_gru: bad sizes");
  XB_REQUIRE(H <= 64, XB_ERR_LIMIT, "xb_gru: hidden size %d, at most 64 (weights are kept in shared memory)", H);
  XB_REQUIRE(dtype == XB_F32 || dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_gru: dtype %d", dtype);
  XB_REQUIRE(batch < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_gru: batch too large");
  if (batch == 0 || T == 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)2 * H * 3 * H + 2 * H + 6 * H);
  static PerDeviceOnce attr;
  XB_SET_MAX_SMEM_ONCE(attr, 110 * 1024, (const void*)gru_kernel);
  const int threads = (3 * H + 31) / 32 * 32;
  gru_kernel<<<(unsigned)batch, threads, smem, (cudaStream_t)s>>>(x, y, T, H, i2h, h2h, i2h_bias, h2h_bias, dtype);
  return check_launch("gru_kernel");
}

extern "C" int xb_augru(const void* x, const void* att, void* y, int64_t batch, int32_t T, int32_t H, const void* Wg,
                        const void* bg, const void* Wc, const void* bc, int32_t dtype, xb_stream_t s) {
  XB_REQUIRE(x && att && y && Wg && bg && Wc && bc, XB_ERR_ARG, "xb_augru: null tensor");
  XB_REQUIRE(batch >= 0 && T >= 0 && H >= 1, XB_ERR_ARG, "xb_augru: bad sizes");
  XB_REQUIRE(H <= 64, XB_ERR_LIMIT, "xb_augru: hidden size %d, at most 64 (weights are kept in shared memory)", H);
  XB_REQUIRE(dtype == XB_F32 || dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_augru: dtype %d", dtype);
  XB_REQUIRE(batch < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_augru: batch too large");
  if (batch == 0 || T == 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)6 * H * H + 5 * H);
  static PerDeviceOnce attr;
  XB_SET_MAX_SMEM_ONCE(attr, 110 * 1024, (const void*)augru_kernel);
  const int threads = (2 * H + 31) / 32 * 32;
  augru_kernel<<<(unsigned)batch, threads, smem, (cudaStream_t)s>>>(x, att, y, T, H, Wg, bg, Wc, bc, dtype, 0);
  return check_launch("augru_kernel");
}

extern "C" int xb_augru_shared(const void* x, const void* att, void* y_final, int32_t requests, int32_t n_cand, int32_t T,
                               int32_t H, const void* Wg, const void* bg, const void* Wc, const void* bc, int32_t engine,
                               xb_stream_t s) {
  XB_REQUIRE(x && att && y_final && Wg && bg && Wc && bc, XB_ERR_ARG, "xb_augru_shared: null tensor");
  XB_REQUIRE(requests >= 0 && n_cand >= 0 && T >= 1 && H >= 1, XB_ERR_ARG, "xb_augru_shared: bad sizes");
  XB_REQUIRE(H <= 64, XB_ERR_LIMIT, "xb_augru_shared: hidden size %d, at most 64", H);
  XB_REQUIRE(engine == XB_GEMM_AUTO || engine == XB_GEMM_SIMT || engine == XB_GEMM_TCGEN05, XB_ERR_ARG, "xb_augru_shared: engine %d", engine);
  if (requests == 0 || n_cand == 0) return 0;
  const bool tc = engine != XB_GEMM_SIMT && augru_tc_eligible(H, T);
  XB_REQUIRE(tc || engine != XB_GEMM_TCGEN05, XB_ERR_UNSUPPORTED,
             "xb_augru_shared: the tcgen05 engine takes an even H <= 64 whose padding to a multiple of 8 leaves 4 slots");
  if (tc) {
    AuParams p;
    memset(&p, 0, sizeof(p));
    p.x = (const __half*)x; p.att = (const __half*)att; p.y = (__half*)y_final;
    p.Wg = (const __half*)Wg; p.bg = (const __half*)bg; p.Wc = (const __half*)Wc; p.bc = (const __half*)bc;
    p.requests = requests; p.n_cand = n_cand; p.T = T; p.H = H;
    return launch_augru_tc(p, (cudaStream_t)s);
  }
  const int64_t batch = (int64_t)requests * n_cand;
  XB_REQUIRE(batch < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_augru_shared: batch too large");
  const size_t smem = sizeof(float) * ((size_t)6 * H * H + 5 * H);
  static PerDeviceOnce attr;
  XB_SET_MAX_SMEM_ONCE(attr, 110 * 1024, (const void*)augru_kernel);
  const int threads = (2 * H + 31) / 32 * 32;
  augru_kernel<<<(unsigned)batch, threads, smem, (cudaStream_t)s>>>(x, att, y_final, T, H, Wg, bg, Wc, bc, XB_F16, n_cand);
  return check_launch("augru_kernel");
}
