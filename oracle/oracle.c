/*
 * oracle.c - plain-C, fp32, single-source restatement of Blaze's CPU inference
 * hot path. TEST INFRASTRUCTURE ONLY: it is the checker the CUDA kernels are
 * compared with and the timed CPU baseline; nothing in the shipped libraries
 * links or calls it.
 *
 * Every function names the reference file:line (paths inside the reference
 * project) whose arithmetic it follows. Loop order and operation order follow
 * the reference so that fp32 results agree with it to rounding.
 *
 * Pinning: tests/test_oracle_golden.py checks these functions against the
 * reference's own operator fixtures (tests/golden/blaze_op_fixtures.json) and,
 * for pooling, against the reference sparse store compiled unmodified
 * (oracle/_ref/libqed_ref.so). The AUGRU step has no reference fixture:
 * parity unpinned for orc_augru only.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------- */
/* key -> row index. The reference resolves an int64 key with a bucketed hash
 * (bucket = (uint32)key % bucket_size, linear scan of the bucket,
 * blaze/blaze/store/quick_embedding/hashtable.cc:45-64). Only hit/miss and
 * the row found matter for the arithmetic, so the restatement uses open
 * addressing over the same key set. */
typedef struct {
  int64_t cap;      /* power of two */
  int64_t* keys;
  int64_t* rows;    /* -1 = empty */
} orc_index;

static uint64_t mix64(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33; return x;
}

void* orc_index_create(const int64_t* keys, int64_t n) {
  orc_index* ix = (orc_index*)malloc(sizeof(orc_index));
  int64_t cap = 16;
  while (cap < 2 * n) cap <<= 1;
  ix->cap = cap;
  ix->keys = (int64_t*)malloc(sizeof(int64_t) * cap);
  ix->rows = (int64_t*)malloc(sizeof(int64_t) * cap);
  for (int64_t i = 0; i < cap; ++i) ix->rows[i] = -1;
  for (int64_t r = 0; r < n; ++r) {
    uint64_t h = mix64((uint64_t)keys[r]) & (uint64_t)(cap - 1);
    /* a repeated key keeps its first row, as a bucket scan would find it */
    while (ix->rows[h] != -1 && ix->keys[h] != keys[r]) h = (h + 1) & (uint64_t)(cap - 1);
    if (ix->rows[h] == -1) { ix->keys[h] = keys[r]; ix->rows[h] = r; }
  }
  return ix;
}

void orc_index_destroy(void* p) {
  orc_index* ix = (orc_index*)p;
  if (!ix) return;
  free(ix->keys); free(ix->rows); free(ix);
}

static int64_t index_lookup(const orc_index* ix, int64_t key) {
  uint64_t h = mix64((uint64_t)key) & (uint64_t)(ix->cap - 1);
  while (ix->rows[h] != -1) {
    if (ix->keys[h] == key) return ix->rows[h];
    h = (h + 1) & (uint64_t)(ix->cap - 1);
  }
  return -1;
}

/* ------------------------------------------------------------------------- */
/* Embedding pooling of one feature group into n_items output blocks.
 * Follows QuickEmbeddingDict::Get, blaze/blaze/store/quick_embedding/
 * quick_embedding_dict.cc:89-147 with the processors of udf_processor.h:41-151.
 *   index == NULL: keys are row numbers; a key outside [0, rows) misses.
 *   udf: 0 kSum, 1 kAvg, 2 kAssign; trunc_dir: 0 kOrder, 1 kReverse.
 *   outs[k] points at the item's column offset inside its block; strides[k]
 *   is the block row stride in elements. The init step zeroes the item's span
 *   (dim, or dim*trunc_num for kAssign) exactly as InitProcess does.
 *   assign_stride[k]: distance in elements between consecutive assigned rows
 *   (the reference always uses dim; a wider stride interleaves two groups).
 */
int orc_embedding_pool(const float* table, int64_t rows, int dim, const void* index,
                       const int64_t* keys, const float* values, const int32_t* key_num,
                       int64_t batch, int n_items, const int* udf, const int* trunc_dir,
                       const int* trunc_num, const int* assign_stride,
                       float* const* outs, const int64_t* strides) {
  const orc_index* ix = (const orc_index*)index;
  float** out = (float**)malloc(sizeof(float*) * (size_t)n_items);
  for (int k = 0; k < n_items; ++k) out[k] = outs[k];
  for (int64_t i = 0; i < batch; ++i) {
    size_t num = (size_t)key_num[i];
    for (int k = 0; k < n_items; ++k) {
      if (udf[k] == 2) {
        int as = assign_stride ? assign_stride[k] : dim;
        for (int t = 0; t < trunc_num[k]; ++t) memset(out[k] + (size_t)t * as, 0, sizeof(float) * dim);
      } else {
        memset(out[k], 0, sizeof(float) * dim);
      }
    }
    for (size_t j = 0; j < num; ++j) {
      int64_t row = ix ? index_lookup(ix, keys[j]) : ((keys[j] >= 0 && keys[j] < rows) ? keys[j] : -1);
      if (row < 0) continue;                       /* missing key: skipped */
      const float* w = table + row * dim;
      float value = values[j];
      for (int k = 0; k < n_items; ++k) {
        if (udf[k] == 2) {
          int as = assign_stride ? assign_stride[k] : dim;
          size_t tn = (size_t)trunc_num[k];
          if (trunc_dir[k] == 0 && j >= tn) continue;
          if (trunc_dir[k] == 1 && (num - j) > tn) continue;
          float* o = out[k] + (trunc_dir[k] == 0 ? (size_t)as * j : (size_t)as * (tn - (num - j)));
          for (int d = 0; d < dim; ++d) o[d] = value * w[d];
        } else {
          float* o = out[k];
          for (int d = 0; d < dim; ++d) o[d] = o[d] + value * w[d];
        }
      }
    }
    for (int k = 0; k < n_items; ++k) {
      if (udf[k] == 1 && num != 0) {
        float s = (float)(1.0 / (double)num);      /* multiply, not divide */
        for (int d = 0; d < dim; ++d) out[k][d] = out[k][d] * s;
      }
      out[k] += strides[k];
    }
    keys += num;
    values += num;
  }
  free(out);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* C = alpha*op(A)*op(B) + beta*C, row-major fp32. Stands in for cblas_sgemm
 * (blaze/blaze/math/gemm.cc:12-27); the BLAS itself is third-party (MKL or an
 * unpinned OpenBLAS) and absent, so the published definition is restated with
 * k ascending and fp32 accumulation. */
void orc_gemm(int transa, int transb, int64_t M, int64_t N, int64_t K, float alpha,
              const float* A, const float* B, float beta, float* C) {
  float* acc = (float*)malloc(sizeof(float) * (size_t)N);
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) acc[j] = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      float a = transa ? A[k * M + i] : A[i * K + k];
      if (!transb) {
        const float* b = B + k * N;
        for (int64_t j = 0; j < N; ++j) acc[j] += a * b[j];
      } else {
        for (int64_t j = 0; j < N; ++j) acc[j] += a * B[j * K + k];
      }
    }
    float* c = C + i * N;
    if (beta == 0.f) for (int64_t j = 0; j < N; ++j) c[j] = alpha * acc[j];
    else for (int64_t j = 0; j < N; ++j) c[j] = alpha * acc[j] + beta * c[j];
  }
  free(acc);
}

/* GemmStridedBatched (blaze/blaze/math/gemm.h:50-63): a stride of 0 re-uses
 * the operand for every batch. */
void orc_gemm_strided_batched(int transa, int transb, int64_t M, int64_t N, int64_t K,
                              float alpha, const float* A, int64_t sa, const float* B, int64_t sb,
                              float beta, float* C, int64_t sc, int64_t batch) {
  for (int64_t p = 0; p < batch; ++p)
    orc_gemm(transa, transb, M, N, K, alpha, A + p * sa, B + p * sb, beta, C + p * sc);
}

/* Gemm operator: Y <- broadcast(bias); Y = alpha*A*B + beta*Y.
 * blaze/blaze/operator/op/gemm_op.h:33-107; bias_rows is 1 for a rank-1 [N]
 * bias (every row gets it, math/broadcast.cc:14-29) or M for a full [M,N]. */
void orc_gemm_op(int transa, int transb, int64_t M, int64_t N, int64_t K, float alpha,
                 const float* A, const float* B, float beta, const float* bias,
                 int64_t bias_rows, float* Y) {
  if (bias == NULL) {
    orc_gemm(transa, transb, M, N, K, alpha, A, B, 0.f, Y);
    return;
  }
  for (int64_t i = 0; i < M; ++i)
    memcpy(Y + i * N, bias + (bias_rows == 1 ? 0 : i * N), sizeof(float) * (size_t)N);
  orc_gemm(transa, transb, M, N, K, alpha, A, B, beta, Y);
}

/* PrunedGemm: [X1|X2] x [W1;W2] = X1 x W1 + X2 x W2, blaze/blaze/operator/op/pruned_gemm_op.h:40-160.
 * Y <- broadcast(bias) (:69-77), then for operands with different row counts the long product
 * goes into Y with `beta` and the one-row product into a scratch row that is added to every
 * row of Y (:106-152, DimEqualBroadcastFMA). The reference allows a short operand of exactly
 * one row; `group` = rows of Y per row of the short product (M for the reference's case)
 * restates that per request when several requests are stacked. With equal row counts (:82-105)
 * the intended sum of both products is formed (the reference passes X2 twice there).
 * x_short [M/group, ks], w_short [ks, N], x_long [M, kl], w_long [kl, N], bias [N] or NULL. */
void orc_pruned_gemm(int64_t M, int64_t N, int64_t group, int64_t ks, int64_t kl, float alpha, float beta,
                     const float* x_short, const float* w_short, const float* x_long, const float* w_long,
                     const float* bias, float* Y) {
  int64_t m = M / group;
  float* part = (float*)malloc(sizeof(float) * (size_t)(m * N));
  orc_gemm_op(0, 0, M, N, kl, alpha, x_long, w_long, beta, bias, 1, Y);
  orc_gemm(0, 0, m, N, ks, alpha, x_short, w_short, 0.f, part);
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) Y[i * N + j] += part[(i / group) * N + j];
  free(part);
}

/* FusedParallelGemm, 2-D input: P GEMMs sharing A; W stacked [P*K,N] (or
 * [P*N,K] with transB); bias [P*N] (bias_rows 1) or [P*M,N] (bias_rows M);
 * Y [P*M,N]. blaze/blaze/operator/fused_op/fused_parallel_gemm_op.h:43-133. */
void orc_fused_parallel_gemm(int transa, int transb, int P, int64_t M, int64_t N, int64_t K,
                             float alpha, const float* A, const float* W, float beta,
                             const float* bias, int64_t bias_rows, float* Y) {
  for (int p = 0; p < P; ++p)
    orc_gemm_op(transa, transb, M, N, K, alpha, A, W + (int64_t)p * K * N, beta,
                bias ? bias + (int64_t)p * bias_rows * N : NULL, bias_rows, Y + (int64_t)p * M * N);
}

/* ------------------------------------------------------------------------- */
/* Dice, blaze/blaze/operator/op/dice_op.cc:14-34 (kDiceEpsilon 1e-8,
 * blaze/blaze/operator/common_helper.h:90). */
void orc_dice(const float* x, int64_t rows, int64_t c, const float* gamma, const float* mean,
              const float* var, int nosqrt, float* y) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * c;
    float* yr = y + r * c;
    for (int64_t j = 0; j < c; ++j) {
      float t = -1 * (xr[j] - mean[j]) / (nosqrt ? var[j] : sqrtf(var[j] + 1e-8f));
      float p = 1 / (1 + expf(t));
      float xv = xr[j];
      yr[j] = (1 - p) * gamma[j] * xv + p * xv;
    }
  }
}

/* PRelu, blaze/blaze/operator/op/prelu_op.cc:10-30 with the formula of
 * blaze/blaze/math/activation.h:36-42; w has `inner` slopes (1 = shared). */
void orc_prelu(const float* x, int64_t size, const float* w, int64_t inner, float* y) {
  for (int64_t i = 0; i < size; ++i) {
    float v = x[i];
    y[i] = v * ((v > 0) + ((v < 0) * w[i % inner]));
  }
}

/* Sigmoid, CPU form e^x/(1+e^x): blaze/blaze/operator/op/sigmoid_op.cc:15-21. */
void orc_sigmoid(const float* x, int64_t size, float* y) {
  for (int64_t i = 0; i < size; ++i) {
    float e = expf(x[i]);
    y[i] = e / (1 + e);
  }
}

/* Softmax over `c` with outer n and inner w:
 * blaze/blaze/operator/op/softmax_op.cc:21-78. */
void orc_softmax(const float* x, int64_t n, int64_t c, int64_t w, float* y) {
  for (int64_t i = 0; i < n; ++i)
    for (int64_t z = 0; z < w; ++z) {
      const float* xs = x + i * c * w + z;
      float* ys = y + i * c * w + z;
      float m = xs[0];
      for (int64_t j = 1; j < c; ++j) m = xs[j * w] > m ? xs[j * w] : m;
      float s = 0.f;
      for (int64_t j = 0; j < c; ++j) { ys[j * w] = expf(xs[j * w] - m); s += ys[j * w]; }
      for (int64_t j = 0; j < c; ++j) ys[j * w] /= s;
    }
}

/* Inference batch normalisation:
 * blaze/blaze/operator/op/batch_normalization_op.cc:12-20. */
void orc_batchnorm(const float* x, int64_t size, int64_t c, const float* gamma, const float* beta,
                   const float* mean, const float* var, float eps, int nosqrt, float* y) {
  for (int64_t i = 0; i < size; ++i) {
    int64_t o = i % c;
    float xn = (x[i] - mean[o]) / (nosqrt ? var[o] : sqrtf(var[o] + eps));
    y[i] = gamma[o] * xn + beta[o];
  }
}

/* Fuse: concat a 1-row tensor with an M-row tensor along columns.
 * blaze/blaze/operator/op/fuse_op.cc:9-30. */
void orc_fuse(const float* x1, int64_t x1_m, int64_t x1_n, const float* x2, int64_t x2_m,
              int64_t x2_n, float* y) {
  int64_t ym = x1_m > x2_m ? x1_m : x2_m;
  for (int64_t r = 0; r < ym; ++r) {
    memcpy(y + r * (x1_n + x2_n), x1 + (x1_m == 1 ? 0 : r * x1_n), sizeof(float) * (size_t)x1_n);
    memcpy(y + r * (x1_n + x2_n) + x1_n, x2 + (x2_m == 1 ? 0 : r * x2_n), sizeof(float) * (size_t)x2_n);
  }
}

/* ------------------------------------------------------------------------- */
/* DIN attention unit, composed op by op as the reference graph does
 * (blaze/tools/example_model/din/model/graph_ulf.txt: sub / multiply /
 * broadcast_to / concat [q,k,q-k,q*k] -> att_gemm0 -> act -> att_gemm1 -> act
 * -> att_gemm2 -> (where mask -> softmax) -> batchdot with k).
 *   q [n_cand, d], k [T, d]; W0 [4d,h0], W1 [h0,h1], W2 [h1,1] (+biases).
 *   act: 0 none, 1 sigmoid (shipped graph), 2 dice (dice params per layer:
 *   gamma/mean/var for h0 and h1).
 *   seq_len valid steps; with use_softmax the masked positions get the
 *   reference padding value -2^32+1 before softmax over T; without softmax
 *   masked positions contribute nothing (their k rows are zero).
 *   out [n_cand, d] = sum_t score[n,t] * k[t]; scores_out (optional) [n_cand,T].
 */
typedef struct {
  const float *W0, *b0, *W1, *b1, *W2, *b2;
  const float *g0, *m0, *v0, *g1, *m1, *v1;   /* dice statistics */
} orc_att_weights;

static void act_rows(int act, float* x, int64_t rows, int64_t c, const float* g, const float* m,
                     const float* v) {
  if (act == 1) orc_sigmoid(x, rows * c, x);
  else if (act == 2) orc_dice(x, rows, c, g, m, v, 0, x);
}

void orc_din_attention(const float* q, int64_t n_cand, const float* k, int64_t T, int d, int h0,
                       int h1, const orc_att_weights* w, int act, int seq_len, int use_softmax,
                       float* out, float* scores_out) {
  int d4 = 4 * d;
  float* x = (float*)malloc(sizeof(float) * (size_t)T * d4);
  float* y0 = (float*)malloc(sizeof(float) * (size_t)T * h0);
  float* y1 = (float*)malloc(sizeof(float) * (size_t)T * h1);
  float* s = (float*)malloc(sizeof(float) * (size_t)T);
  for (int64_t n = 0; n < n_cand; ++n) {
    const float* qn = q + n * d;
    for (int64_t t = 0; t < T; ++t) {
      const float* kt = k + t * d;
      float* xr = x + t * d4;
      for (int j = 0; j < d; ++j) {
        xr[j] = qn[j];
        xr[d + j] = kt[j];
        xr[2 * d + j] = qn[j] - kt[j];
        xr[3 * d + j] = qn[j] * kt[j];
      }
    }
    orc_gemm_op(0, 0, T, h0, d4, 1.f, x, w->W0, 1.f, w->b0, 1, y0);
    act_rows(act, y0, T, h0, w->g0, w->m0, w->v0);
    orc_gemm_op(0, 0, T, h1, h0, 1.f, y0, w->W1, 1.f, w->b1, 1, y1);
    act_rows(act, y1, T, h1, w->g1, w->m1, w->v1);
    orc_gemm_op(0, 0, T, 1, h1, 1.f, y1, w->W2, 1.f, w->b2, 1, s);
    if (use_softmax) {
      for (int64_t t = seq_len; t < T; ++t) s[t] = -4294967295.0f;
      orc_softmax(s, 1, T, 1, s);
    } else {
      for (int64_t t = seq_len; t < T; ++t) s[t] = 0.f;
    }
    if (scores_out) memcpy(scores_out + n * T, s, sizeof(float) * (size_t)T);
    float* o = out + n * d;
    for (int j = 0; j < d; ++j) o[j] = 0.f;
    /* batchdot (MatMul transA): out[j] = sum_t s[t]*k[t][j], t ascending */
    for (int64_t t = 0; t < T; ++t)
      for (int j = 0; j < d; ++j) o[j] += s[t] * k[t * d + j];
  }
  free(x); free(y0); free(y1); free(s);
}

/* ------------------------------------------------------------------------- */
/* GRU over T steps for one batch row-set, following GRUKernel
 * (blaze/blaze/operator/op/gru_op.cc:33-93): preact = X*W_i2h once, per step
 * act = h*W_h2h, gates r,z = sigmoid(first 2H), candidate tanh(i_h + r*h_h),
 * h' = c + z*(h - c). Biases i2h_bias/h2h_bias are [3H]. Gate order r,z,c.
 * x [B,T,H], y [B,T,H]. Leading steps whose first H pre-activations are all
 * zero emit zeros and keep h = 0. */
static float sigm(float v) { return 1.f / (1.f + expf(-v)); }

void orc_gru(const float* x, int64_t B, int64_t T, int H, const float* Wi, const float* Wh,
             const float* bi, const float* bh, float* y) {
  float* pre = (float*)malloc(sizeof(float) * 3 * (size_t)H);
  float* act = (float*)malloc(sizeof(float) * 3 * (size_t)H);
  float* h = (float*)malloc(sizeof(float) * (size_t)H);
  for (int64_t b = 0; b < B; ++b) {
    for (int j = 0; j < H; ++j) h[j] = 0.f;
    int started = 0;
    for (int64_t t = 0; t < T; ++t) {
      const float* xt = x + (b * T + t) * H;
      float* yt = y + (b * T + t) * H;
      orc_gemm(0, 0, 1, 3 * H, H, 1.f, xt, Wi, 0.f, pre);
      if (!started) {
        /* the reference tests the first H pre-activations, before the bias */
        int allzero = 1;
        for (int j = 0; j < H; ++j) if (pre[j] != 0.f) { allzero = 0; break; }
        if (allzero) { for (int j = 0; j < H; ++j) yt[j] = 0.f; continue; }
        started = 1;
      }
      orc_gemm(0, 0, 1, 3 * H, H, 1.f, h, Wh, 0.f, act);
      for (int j = 0; j < 3 * H; ++j) { pre[j] += bi ? bi[j] : 0.f; act[j] += bh ? bh[j] : 0.f; }
      for (int j = 0; j < H; ++j) {
        float r = sigm(pre[j] + act[j]);
        float z = sigm(pre[H + j] + act[H + j]);
        float c = tanhf(pre[2 * H + j] + r * act[2 * H + j]);
        yt[j] = c + z * (h[j] - c);
      }
      for (int j = 0; j < H; ++j) h[j] = yt[j];
    }
  }
  free(pre); free(act); free(h);
}

/* AUGRU step sequence after VecAttGRUCell.call
 * (xdl-algorithm-solution/DIEN/script/utils.py:139-207): gates over [x,h] with
 * bias, sigmoid, split r|u; candidate tanh over [x, r*h]; u' = (1-a)*u;
 * h' = u'*h + (1-u')*c. Wg [2H, 2H] (rows: x then h; cols: r then u),
 * Wc [2H, H]. att [B,T]. y [B,T,H]. Parity unpinned: no reference fixture. */
void orc_augru(const float* x, const float* att, int64_t B, int64_t T, int H, const float* Wg,
               const float* bg, const float* Wc, const float* bc, float* y) {
  float* xh = (float*)malloc(sizeof(float) * 2 * (size_t)H);
  float* g = (float*)malloc(sizeof(float) * 2 * (size_t)H);
  float* c = (float*)malloc(sizeof(float) * (size_t)H);
  float* h = (float*)malloc(sizeof(float) * (size_t)H);
  for (int64_t b = 0; b < B; ++b) {
    for (int j = 0; j < H; ++j) h[j] = 0.f;
    for (int64_t t = 0; t < T; ++t) {
      const float* xt = x + (b * T + t) * H;
      for (int j = 0; j < H; ++j) { xh[j] = xt[j]; xh[H + j] = h[j]; }
      orc_gemm_op(0, 0, 1, 2 * H, 2 * H, 1.f, xh, Wg, 1.f, bg, 1, g);
      for (int j = 0; j < 2 * H; ++j) g[j] = sigm(g[j]);
      for (int j = 0; j < H; ++j) xh[H + j] = g[j] * h[j];
      orc_gemm_op(0, 0, 1, H, 2 * H, 1.f, xh, Wc, 1.f, bc, 1, c);
      float a = att[b * T + t];
      float* yt = y + (b * T + t) * H;
      for (int j = 0; j < H; ++j) {
        float u = (1.f - a) * g[H + j];
        yt[j] = u * h[j] + (1.f - u) * tanhf(c[j]);
      }
      for (int j = 0; j < H; ++j) h[j] = yt[j];
    }
  }
  free(xh); free(g); free(c); free(h);
}

/* Row-shard routing rule of the sharded pooling path (no reference
 * counterpart; the rule is this project's): owner = (uint64)id % shards,
 * local row = id / shards. */
void orc_route(const int64_t* ids, int64_t n, int shards, int32_t* owner, int64_t* local_row) {
  for (int64_t i = 0; i < n; ++i) {
    uint64_t u = (uint64_t)ids[i];
    owner[i] = (int32_t)(u % (uint64_t)shards);
    local_row[i] = (int64_t)(u / (uint64_t)shards);
  }
}
