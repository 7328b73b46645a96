// Stand-alone activation, normalisation, elementwise and data-movement
// operators for graphs whose ops were not fused into a GEMM epilogue, plus the
// library's error/version plumbing. All are HBM-bound streaming kernels:
// grid-stride loops sized to a multiple of the SM count.
#include <cstring>

#include "xb_common.cuh"

namespace xb {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { g_err[0] = 0; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static inline unsigned stream_grid(int64_t work_items, int per_block) {
  int64_t blocks = (work_items + per_block - 1) / per_block;
  int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

__global__ void dice_kernel(const void* x, void* y, int64_t size, int c, const void* gamma,
                            const void* mean, const void* var, int nosqrt, int dt) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < size; i += (int64_t)gridDim.x * blockDim.x) {
    int col = (int)(i % c);
    float v = load_as_f32(x, i, dt);
    float r = act_dice(v, load_as_f32(gamma, col, dt), load_as_f32(mean, col, dt),
                       dice_rstd(load_as_f32(var, col, dt), nosqrt));
    store_from_f32(y, i, dt, r);
  }
}

__global__ void prelu_kernel(const void* x, void* y, int64_t size, const void* w, int64_t inner, int dt, int wdt) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < size; i += (int64_t)gridDim.x * blockDim.x)
    store_from_f32(y, i, dt, act_prelu(load_as_f32(x, i, dt), load_as_f32(w, i % inner, wdt)));
}

__global__ void sigmoid_kernel(const void* x, void* y, int64_t size, int dt) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < size; i += (int64_t)gridDim.x * blockDim.x)
    store_from_f32(y, i, dt, act_sigmoid(load_as_f32(x, i, dt)));
}

__global__ void batchnorm_kernel(const void* x, void* y, int64_t size, int c, const void* gamma, const void* beta,
                                 const void* mean, const void* var, float eps, int nosqrt, int dt) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < size; i += (int64_t)gridDim.x * blockDim.x) {
    int col = (int)(i % c);
    float vr = load_as_f32(var, col, dt);
    float xn = (load_as_f32(x, i, dt) - load_as_f32(mean, col, dt)) / (nosqrt ? vr : sqrtf(vr + eps));
    store_from_f32(y, i, dt, load_as_f32(gamma, col, dt) * xn + load_as_f32(beta, col, dt));
  }
}

// one thread per (outer, inner) pair walks the c axis three times (max, sum, divide)
__global__ void softmax_kernel(const void* x, void* y, int64_t n, int c, int64_t w, int dt) {
  const int64_t total = n * w;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t base = (i / w) * c * w + (i % w);
    float m = load_as_f32(x, base, dt);
    for (int j = 1; j < c; ++j) m = fmaxf(m, load_as_f32(x, base + (int64_t)j * w, dt));
    float s = 0.f;
    for (int j = 0; j < c; ++j) s += __expf(load_as_f32(x, base + (int64_t)j * w, dt) - m);
    for (int j = 0; j < c; ++j)
      store_from_f32(y, base + (int64_t)j * w, dt, __expf(load_as_f32(x, base + (int64_t)j * w, dt) - m) / s);
  }
}

struct EwParams {
  int op, dt;
  const void *a, *b, *c;
  void* y;
  int64_t as[4], bs[4], cs[4], shape[4];
};

__global__ void elementwise_kernel(const __grid_constant__ EwParams p) {
  const int64_t total = p.shape[0] * p.shape[1] * p.shape[2] * p.shape[3];
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i;
    const int64_t i3 = r % p.shape[3]; r /= p.shape[3];
    const int64_t i2 = r % p.shape[2]; r /= p.shape[2];
    const int64_t i1 = r % p.shape[1]; r /= p.shape[1];
    const int64_t i0 = r;
    const int64_t ia = i0 * p.as[0] + i1 * p.as[1] + i2 * p.as[2] + i3 * p.as[3];
    const int64_t ib = i0 * p.bs[0] + i1 * p.bs[1] + i2 * p.bs[2] + i3 * p.bs[3];
    float out;
    if (p.op == XB_EW_WHERE) {
      const int64_t ic = i0 * p.cs[0] + i1 * p.cs[1] + i2 * p.cs[2] + i3 * p.cs[3];
      const int32_t cond = reinterpret_cast<const int32_t*>(p.a)[ia];
      out = cond ? load_as_f32(p.b, ib, p.dt) : load_as_f32(p.c, ic, p.dt);
    } else if (p.op == XB_EW_BROADCAST_TO) {
      out = load_as_f32(p.a, ia, p.dt);
    } else {
      const float av = load_as_f32(p.a, ia, p.dt), bv = load_as_f32(p.b, ib, p.dt);
      switch (p.op) {
        case XB_EW_ADD: out = av + bv; break;
        case XB_EW_SUB: out = av - bv; break;
        case XB_EW_MUL: out = av * bv; break;
        case XB_EW_DIV: out = av / bv; break;
        case XB_EW_MAX: out = fmaxf(av, bv); break;
        case XB_EW_MIN: out = fminf(av, bv); break;
        case XB_EW_EQ: out = av == bv ? 1.f : 0.f; break;
        default: out = av != bv ? 1.f : 0.f; break;
      }
    }
    store_from_f32(p.y, i, p.dt, out);
  }
}

__global__ void copy2d_kernel(const void* src, int64_t src_ld, int sdt, void* dst, int64_t dst_ld, int ddt,
                              int64_t rows, int64_t cols) {
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    if (sdt == XB_I32 && ddt == XB_I32)
      reinterpret_cast<int32_t*>(dst)[r * dst_ld + c] = reinterpret_cast<const int32_t*>(src)[r * src_ld + c];
    else if (sdt == XB_I64 && ddt == XB_I64)
      reinterpret_cast<int64_t*>(dst)[r * dst_ld + c] = reinterpret_cast<const int64_t*>(src)[r * src_ld + c];
    else
      store_from_f32(dst, r * dst_ld + c, ddt, load_as_f32(src, r * src_ld + c, sdt));
  }
}

__global__ void reduce_sum_kernel(const void* x, void* y, int64_t outer, int64_t r, int64_t inner, int dt) {
  const int64_t total = outer * inner;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = i / inner, in = i - o * inner;
    float s = 0.f;
    for (int64_t j = 0; j < r; ++j) s += load_as_f32(x, (o * r + j) * inner + in, dt);
    store_from_f32(y, i, dt, s);
  }
}

// W [K,N] row-major (ld ldw) -> out [N, ldk] with zero padding of k in [K, ldk)
__global__ void pack_kmajor_kernel(const void* W, int wdt, int K, int N, int64_t ldw, void* out, int odt,
                                   int64_t ldk, int64_t stride_w, int64_t stride_out) {
  const int64_t b = blockIdx.y;
  const int64_t total = (int64_t)N * ldk;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / ldk, k = i - n * ldk;
    float v = k < K ? load_as_f32(W, b * stride_w + k * ldw + n, wdt) : 0.f;
    store_from_f32(out, b * stride_out + i, odt, v);
  }
}

// one CTA per (request, 64-candidate slab); his_sum is rebuilt per CTA from the T k rows. The row is
// produced two columns (one 32-bit store) at a time when d and du are even; every feature segment then
// starts on a 4-byte boundary in X and in q / att.
__global__ void __launch_bounds__(256) din_tower_input_kernel(const __half* user, int64_t ldu, const __half* q,
                                                              int64_t ldq, const __half* k, int64_t ldk,
                                                              const __half* att, int64_t ldatt, __half* X, int64_t ldx,
                                                              int n_cand, int T, int d, int du, int pairs_ok) {
  extern __shared__ float hs[];      // [d] his_sum, then [du] user row
  float* us = hs + d;
  const int r = blockIdx.y;
  // his_sum: the block's threads split the T steps (groups of d threads take every G-th step), partial
  // sums meet in shared memory and are added in group order, so the result does not depend on timing
  float* part = us + du;             // [G][d]
  const int G = max(1, min((int)blockDim.x / d, 8));
  if ((int)threadIdx.x < G * d) {
    const int gi = threadIdx.x / d, e = threadIdx.x - gi * d;
    float s = 0.f;
    for (int t = gi; t < T; t += G) s += __half2float(k[((int64_t)r * T + t) * ldk + e]);
    part[gi * d + e] = s;
  }
  for (int e = threadIdx.x; e < du; e += blockDim.x) us[e] = __half2float(user[(int64_t)r * ldu + e]);
  __syncthreads();
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float s = 0.f;
    for (int gi = 0; gi < G; ++gi) s += part[gi * d + e];
    hs[e] = s;
  }
  __syncthreads();
  const int n0 = blockIdx.x * 64;
  const int rows = min(64, n_cand - n0);
  if (pairs_ok) {
    const int wp = (int)(ldx >> 1);                    // half2 units per row
    for (int idx = threadIdx.x; idx < rows * wp; idx += blockDim.x) {
      const int n = n0 + idx / wp, c = (idx % wp) * 2;
      const int64_t row = (int64_t)r * n_cand + n;
      float2 v = make_float2(0.f, 0.f);
      if (c < du) v = make_float2(us[c], us[c + 1]);
      else if (c < du + 5 * d) {
        const int seg = (c - du) / d, e = (c - du) - seg * d;
        if (seg == 1) v = make_float2(hs[e], hs[e + 1]);
        else if (seg == 3) v = __half22float2(*reinterpret_cast<const __half2*>(att + row * ldatt + e));
        else {
          const float2 qv = __half22float2(*reinterpret_cast<const __half2*>(q + row * ldq + e));
          if (seg == 0) v = qv;
          else if (seg == 2) v = make_float2(qv.x * hs[e], qv.y * hs[e + 1]);
          else v = make_float2(qv.x - hs[e], qv.y - hs[e + 1]);
        }
      }
      *reinterpret_cast<__half2*>(X + row * ldx + c) = __floats2half2_rn(v.x, v.y);
    }
    return;
  }
  const int width = (int)ldx;
  for (int idx = threadIdx.x; idx < rows * width; idx += blockDim.x) {
    const int n = n0 + idx / width, c = idx % width;
    const int64_t row = (int64_t)r * n_cand + n;
    float v = 0.f;
    if (c < du) v = us[c];
    else if (c < du + 5 * d) {
      const int seg = (c - du) / d, e = (c - du) % d;
      const float qv = __half2float(q[row * ldq + e]);
      if (seg == 0) v = qv;
      else if (seg == 1) v = hs[e];
      else if (seg == 2) v = qv * hs[e];
      else if (seg == 3) v = __half2float(att[row * ldatt + e]);
      else v = qv - hs[e];
    }
    X[row * ldx + c] = __float2half_rn(v);
  }
}

// Split form: per-request columns [user | his_sum] once per request, per-candidate columns
// [q | q*his_sum | att | q-his_sum] per candidate. Same CTA shape as above.
__global__ void __launch_bounds__(256) din_tower_split_kernel(const __half* user, int64_t ldu, const __half* q,
                                                              int64_t ldq, const __half* k, int64_t ldk,
                                                              const __half* att, int64_t ldatt, __half* Xu, int64_t ldxu,
                                                              __half* Xc, int64_t ldxc, int n_cand, int T, int d, int du,
                                                              int pairs_ok) {
  extern __shared__ float hs[];      // [d] his_sum, then [G][d] partial sums
  float* part = hs + d;
  const int r = blockIdx.y;
  const int G = max(1, min((int)blockDim.x / d, 8));
  if ((int)threadIdx.x < G * d) {
    const int gi = threadIdx.x / d, e = threadIdx.x - gi * d;
    float s = 0.f;
    for (int t = gi; t < T; t += G) s += __half2float(k[((int64_t)r * T + t) * ldk + e]);
    part[gi * d + e] = s;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float s = 0.f;
    for (int gi = 0; gi < G; ++gi) s += part[gi * d + e];
    hs[e] = s;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int c = threadIdx.x; c < (int)ldxu; c += blockDim.x) {
      __half v = __float2half(0.f);
      if (c < du) v = user[(int64_t)r * ldu + c];
      else if (c < du + d) v = __float2half_rn(hs[c - du]);
      Xu[(int64_t)r * ldxu + c] = v;
    }
  }
  const int n0 = blockIdx.x * 64;
  const int rows = min(64, n_cand - n0);
  if (pairs_ok) {
    const int wp = (int)(ldxc >> 1);                   // half2 units per row
    for (int idx = threadIdx.x; idx < rows * wp; idx += blockDim.x) {
      const int n = n0 + idx / wp, c = (idx % wp) * 2;
      const int64_t row = (int64_t)r * n_cand + n;
      float2 v = make_float2(0.f, 0.f);
      if (c < 4 * d) {
        const int seg = c / d, e = c - seg * d;
        if (seg == 2) v = __half22float2(*reinterpret_cast<const __half2*>(att + row * ldatt + e));
        else {
          const float2 qv = __half22float2(*reinterpret_cast<const __half2*>(q + row * ldq + e));
          if (seg == 0) v = qv;
          else if (seg == 1) v = make_float2(qv.x * hs[e], qv.y * hs[e + 1]);
          else v = make_float2(qv.x - hs[e], qv.y - hs[e + 1]);
        }
      }
      *reinterpret_cast<__half2*>(Xc + row * ldxc + c) = __floats2half2_rn(v.x, v.y);
    }
    return;
  }
  const int width = (int)ldxc;
  for (int idx = threadIdx.x; idx < rows * width; idx += blockDim.x) {
    const int n = n0 + idx / width, c = idx % width;
    const int64_t row = (int64_t)r * n_cand + n;
    float v = 0.f;
    if (c < 4 * d) {
      const int seg = c / d, e = c % d;
      if (seg == 2) v = __half2float(att[row * ldatt + e]);
      else {
        const float qv = __half2float(q[row * ldq + e]);
        v = seg == 0 ? qv : (seg == 1 ? qv * hs[e] : qv - hs[e]);
      }
    }
    Xc[row * ldxc + c] = __float2half_rn(v);
  }
}

static bool float_dtype(int dt) { return dt == XB_F32 || dt == XB_F16 || dt == XB_BF16; }

}  // namespace xb

using namespace xb;

extern "C" const char* xb_last_error(void) { return g_err; }
extern "C" const char* xb_version(void) { return "xdlb200 0.1 (sm_100a)"; }

extern "C" int xb_dice(const void* x, void* y, int64_t rows, int32_t c, const void* gamma, const void* mean,
                       const void* var, int32_t nosqrt, int32_t dtype, xb_stream_t s) {
  XB_REQUIRE(x && y && gamma && mean && var && c > 0 && rows >= 0, XB_ERR_ARG, "xb_dice: bad arguments");
  XB_REQUIRE(float_dtype(dtype), XB_ERR_UNSUPPORTED, "xb_dice: dtype %d", dtype);
  if (rows == 0) return 0;
  dice_kernel<<<stream_grid(rows * c, 256), 256, 0, (cudaStream_t)s>>>(x, y, rows * c, c, gamma, mean, var, nosqrt, dtype);
  return check_launch("dice_kernel");
}

extern "C" int xb_prelu(const void* x, void* y, int64_t size, const void* w, int64_t inner, int32_t dtype,
                        int32_t w_dtype, xb_stream_t s) {
  XB_REQUIRE(x && y && w && inner > 0 && size >= 0, XB_ERR_ARG, "xb_prelu: bad arguments");
  XB_REQUIRE(float_dtype(dtype) && float_dtype(w_dtype), XB_ERR_UNSUPPORTED, "xb_prelu: dtype %d/%d", dtype, w_dtype);
  if (size == 0) return 0;
  prelu_kernel<<<stream_grid(size, 256), 256, 0, (cudaStream_t)s>>>(x, y, size, w, inner, dtype, w_dtype);
  return check_launch("prelu_kernel");
}

extern "C" int xb_sigmoid(const void* x, void* y, int64_t size, int32_t dtype, xb_stream_t s) {
  XB_REQUIRE(x && y && size >= 0, XB_ERR_ARG, "xb_sigmoid: bad arguments");
  XB_REQUIRE(float_dtype(dtype), XB_ERR_UNSUPPORTED, "xb_sigmoid: dtype %d", dtype);
  if (size == 0) return 0;
  sigmoid_kernel<<<stream_grid(size, 256), 256, 0, (cudaStream_t)s>>>(x, y, size, dtype);
  return check_launch("sigmoid_kernel");
}

extern "C" int xb_softmax(const void* x, void* y, int64_t n, int32_t c, int64_t w, int32_t dtype, xb_stream_t s) {
  XB_REQUIRE(x && y && n >= 0 && c > 0 && w > 0, XB_ERR_ARG, "xb_softmax: bad arguments");
  XB_REQUIRE(float_dtype(dtype), XB_ERR_UNSUPPORTED, "xb_softmax: dtype %d", dtype);
  if (n == 0) return 0;
  softmax_kernel<<<stream_grid(n * w, 128), 128, 0, (cudaStream_t)s>>>(x, y, n, c, w, dtype);
  return check_launch("softmax_kernel");
}

extern "C" int xb_batchnorm(const void* x, void* y, int64_t size, int32_t c, const void* gamma, const void* beta,
                            const void* mean, const void* var, float eps, int32_t nosqrt, int32_t dtype,
                            xb_stream_t s) {
  XB_REQUIRE(x && y && gamma && beta && mean && var && c > 0 && size >= 0, XB_ERR_ARG, "xb_batchnorm: bad arguments");
  XB_REQUIRE(float_dtype(dtype), XB_ERR_UNSUPPORTED, "xb_batchnorm: dtype %d", dtype);
  if (size == 0) return 0;
  batchnorm_kernel<<<stream_grid(size, 256), 256, 0, (cudaStream_t)s>>>(x, y, size, c, gamma, beta, mean, var, eps, nosqrt, dtype);
  return check_launch("batchnorm_kernel");
}

extern "C" int xb_elementwise(int32_t op, const void* a, const int64_t* as, const void* b, const int64_t* bs,
                              const void* c, const int64_t* cs, void* y, const int64_t* shape, int32_t dtype,
                              xb_stream_t s) {
  XB_REQUIRE(op >= XB_EW_ADD && op <= XB_EW_WHERE, XB_ERR_UNSUPPORTED, "xb_elementwise: op %d", op);
  XB_REQUIRE(a && as && y && shape, XB_ERR_ARG, "xb_elementwise: null pointer");
  XB_REQUIRE(op == XB_EW_BROADCAST_TO || (b && bs), XB_ERR_ARG, "xb_elementwise: second operand missing");
  XB_REQUIRE(op != XB_EW_WHERE || (c && cs), XB_ERR_ARG, "xb_elementwise: third operand missing");
  XB_REQUIRE(float_dtype(dtype) || dtype == XB_I32, XB_ERR_UNSUPPORTED, "xb_elementwise: dtype %d", dtype);
  EwParams p;
  memset(&p, 0, sizeof(p));
  p.op = op; p.dt = dtype; p.a = a; p.b = b; p.c = c; p.y = y;
  int64_t total = 1;
  for (int i = 0; i < 4; ++i) {
    XB_REQUIRE(shape[i] >= 0, XB_ERR_ARG, "xb_elementwise: negative extent");
    p.shape[i] = shape[i]; p.as[i] = as[i];
    p.bs[i] = bs ? bs[i] : 0; p.cs[i] = cs ? cs[i] : 0;
    total *= shape[i];
  }
  if (total == 0) return 0;
  elementwise_kernel<<<stream_grid(total, 256), 256, 0, (cudaStream_t)s>>>(p);
  return check_launch("elementwise_kernel");
}

extern "C" int xb_copy2d(const void* src, int64_t src_ld, int32_t sdt, void* dst, int64_t dst_ld, int32_t ddt,
                         int64_t rows, int64_t cols, xb_stream_t s) {
  XB_REQUIRE(src && dst && rows >= 0 && cols >= 0, XB_ERR_ARG, "xb_copy2d: bad arguments");
  XB_REQUIRE(dtype_size(sdt) && dtype_size(ddt), XB_ERR_UNSUPPORTED, "xb_copy2d: dtype %d -> %d", sdt, ddt);
  XB_REQUIRE((sdt == XB_I64) == (ddt == XB_I64), XB_ERR_UNSUPPORTED, "xb_copy2d: int64 converts to nothing else");
  if (rows * cols == 0) return 0;
  copy2d_kernel<<<stream_grid(rows * cols, 256), 256, 0, (cudaStream_t)s>>>(src, src_ld, sdt, dst, dst_ld, ddt, rows, cols);
  return check_launch("copy2d_kernel");
}

// One CTA column per descriptor, blockIdx.y walks the copy in 32 KB pieces; 16-byte vectors when both ends
// and the length allow it, single bytes otherwise (id lists and segment counts of odd lengths).
constexpr int64_t COPY_PIECE = 32 * 1024;
__global__ void copy_segments_kernel(const xb_copy_item* __restrict__ items) {
  const xb_copy_item it = items[blockIdx.x];
  const int64_t begin = (int64_t)blockIdx.y * COPY_PIECE;
  if (begin >= it.bytes) return;
  const int64_t n = min(COPY_PIECE, it.bytes - begin);
  const uint8_t* src = reinterpret_cast<const uint8_t*>(it.src) + begin;
  uint8_t* dst = reinterpret_cast<uint8_t*>(it.dst) + begin;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    const int64_t nv = n / 16;
    for (int64_t i = threadIdx.x; i < nv; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
    for (int64_t i = nv * 16 + threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  } else {
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
}

extern "C" int xb_copy_segments(const xb_copy_item* items, int32_t n_items, int64_t max_bytes, xb_stream_t s) {
  XB_REQUIRE(n_items >= 0 && max_bytes >= 0 && (n_items == 0 || items), XB_ERR_ARG, "xb_copy_segments: bad arguments");
  if (n_items == 0 || max_bytes == 0) return 0;
  const int64_t pieces = (max_bytes + COPY_PIECE - 1) / COPY_PIECE;
  XB_REQUIRE(pieces <= 65535, XB_ERR_LIMIT, "xb_copy_segments: a copy of %lld bytes is too long for one call", (long long)max_bytes);
  dim3 grid((unsigned)n_items, (unsigned)pieces);
  copy_segments_kernel<<<grid, 256, 0, (cudaStream_t)s>>>(items);
  return check_launch("copy_segments_kernel");
}

extern "C" int xb_reduce_sum(const void* x, void* y, int64_t outer, int64_t r, int64_t inner, int32_t dtype,
                             xb_stream_t s) {
  XB_REQUIRE(x && y && outer >= 0 && r >= 0 && inner >= 0, XB_ERR_ARG, "xb_reduce_sum: bad arguments");
  XB_REQUIRE(float_dtype(dtype), XB_ERR_UNSUPPORTED, "xb_reduce_sum: dtype %d", dtype);
  if (outer * inner == 0) return 0;
  reduce_sum_kernel<<<stream_grid(outer * inner, 128), 128, 0, (cudaStream_t)s>>>(x, y, outer, r, inner, dtype);
  return check_launch("reduce_sum_kernel");
}

extern "C" int xb_pack_weight_kmajor(const void* W, int32_t w_dtype, int32_t K, int32_t N, int64_t ldw, void* out,
                                     int32_t out_dtype, int64_t ldk, int32_t batch, int64_t stride_w,
                                     int64_t stride_out, xb_stream_t s) {
  XB_REQUIRE(W && out && K > 0 && N > 0 && batch > 0, XB_ERR_ARG, "xb_pack_weight_kmajor: bad arguments");
  XB_REQUIRE(ldk >= K && ldw >= N, XB_ERR_ARG, "xb_pack_weight_kmajor: leading dimensions too small");
  XB_REQUIRE(float_dtype(w_dtype) && float_dtype(out_dtype), XB_ERR_UNSUPPORTED, "xb_pack_weight_kmajor: dtype");
  XB_REQUIRE(batch <= 65535, XB_ERR_LIMIT, "xb_pack_weight_kmajor: batch %d", batch);
  dim3 grid(stream_grid((int64_t)N * ldk, 256), batch);
  pack_kmajor_kernel<<<grid, 256, 0, (cudaStream_t)s>>>(W, w_dtype, K, N, ldw, out, out_dtype, ldk, stride_w, stride_out);
  return check_launch("pack_kmajor_kernel");
}

extern "C" int xb_din_tower_input(const void* user, int64_t ldu, const void* q, int64_t ldq, const void* k,
                                  int64_t ldk, const void* att, int64_t ldatt, void* X, int64_t ldx,
                                  int32_t requests, int32_t n_cand, int32_t T, int32_t d, int32_t du,
                                  xb_stream_t s) {
  XB_REQUIRE(user && q && k && att && X, XB_ERR_ARG, "xb_din_tower_input: null tensor");
  XB_REQUIRE(requests >= 0 && n_cand >= 0 && T >= 0 && d > 0 && du >= 0, XB_ERR_ARG, "xb_din_tower_input: bad sizes");
  XB_REQUIRE(d <= 256 && du <= 4096, XB_ERR_LIMIT, "xb_din_tower_input: d <= 256 and du <= 4096");
  XB_REQUIRE(ldx >= du + 5 * d && ldu >= du && ldq >= d && ldk >= d && ldatt >= d, XB_ERR_ARG,
             "xb_din_tower_input: leading dimension too small");
  XB_REQUIRE(requests <= 65535 && ldx <= 65536, XB_ERR_LIMIT, "xb_din_tower_input: more than 65535 requests per call");
  if (requests == 0 || n_cand == 0) return 0;
  dim3 grid((n_cand + 63) / 64, requests);
  // 32-bit accesses need even segment widths and leading dimensions and 4-byte aligned bases
  const int pairs_ok = d % 2 == 0 && du % 2 == 0 && ldx % 2 == 0 && ldq % 2 == 0 && ldatt % 2 == 0 &&
                       (((uintptr_t)q | (uintptr_t)att | (uintptr_t)X) & 3) == 0;
  din_tower_input_kernel<<<grid, 256, sizeof(float) * (9 * d + du + 2), (cudaStream_t)s>>>(
      (const __half*)user, ldu, (const __half*)q, ldq, (const __half*)k, ldk, (const __half*)att, ldatt, (__half*)X,
      ldx, n_cand, T, d, du, pairs_ok);
  return check_launch("din_tower_input_kernel");
}

extern "C" int xb_din_tower_input_split(const void* user, int64_t ldu, const void* q, int64_t ldq, const void* k,
                                        int64_t ldk, const void* att, int64_t ldatt, void* Xu, int64_t ldxu, void* Xc,
                                        int64_t ldxc, int32_t requests, int32_t n_cand, int32_t T, int32_t d, int32_t du,
                                        xb_stream_t s) {
  XB_REQUIRE(user && q && k && att && Xu && Xc, XB_ERR_ARG, "xb_din_tower_input_split: null tensor");
  XB_REQUIRE(requests >= 0 && n_cand >= 0 && T >= 0 && d > 0 && du >= 0, XB_ERR_ARG, "xb_din_tower_input_split: bad sizes");
  XB_REQUIRE(d <= 256 && du <= 4096, XB_ERR_LIMIT, "xb_din_tower_input_split: d <= 256 and du <= 4096");
  XB_REQUIRE(ldxu >= du + d && ldxc >= 4 * d && ldu >= du && ldq >= d && ldk >= d && ldatt >= d, XB_ERR_ARG,
             "xb_din_tower_input_split: leading dimension too small");
  XB_REQUIRE(requests <= 65535 && ldxc <= 65536 && ldxu <= 65536, XB_ERR_LIMIT,
             "xb_din_tower_input_split: more than 65535 requests per call");
  if (requests == 0) return 0;
  dim3 grid(n_cand > 0 ? (n_cand + 63) / 64 : 1, requests);
  const int pairs_ok = d % 2 == 0 && ldxc % 2 == 0 && ldq % 2 == 0 && ldatt % 2 == 0 &&
                       (((uintptr_t)q | (uintptr_t)att | (uintptr_t)Xc) & 3) == 0;
  din_tower_split_kernel<<<grid, 256, sizeof(float) * (9 * d + 2), (cudaStream_t)s>>>(
      (const __half*)user, ldu, (const __half*)q, ldq, (const __half*)k, ldk, (const __half*)att, ldatt, (__half*)Xu,
      ldxu, (__half*)Xc, ldxc, n_cand, T, d, du, pairs_ok);
  return check_launch("din_tower_split_kernel");
}
