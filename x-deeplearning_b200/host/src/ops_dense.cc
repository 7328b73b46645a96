// CUDA operators of the dense part of the hot path: ConstantFill, Gemm (with the
// optional fused activation the fusion pass adds), FusedParallelGemm, MatMul,
// FusedParallelMatMul, Dice, PRelu, Sigmoid, Softmax, BatchNormalization and the
// fused DIN operators. Each RunOnDevice shapes its outputs the way the reference
// operator does and then makes one call into the kernel library.
#include <algorithm>
#include <cstring>

#include "runtime.h"

namespace blaze {
namespace {

// Operand of a dense operator that has to reach the kernels in another layout or
// type than the model holds it in (K-major weights, fp32 activation parameters).
// Converted once when the source is a constant, on every run otherwise.
struct Derived {
  std::unique_ptr<Blob> blob;
  const void* src = nullptr;
  bool valid = false;
};

const float* AsF32(Blob* b, Derived* d, cudaStream_t s, int* launches) {
  if (b->data_type() == kFloat) return b->as<float>();
  if (!d->blob) d->blob.reset(new Blob(b->device_option()));
  if (!(d->valid && b->is_constant && d->src == b->as<void>())) {
    d->blob->set_data_type(kFloat);
    d->blob->Reshape(b->shape());
    XB_CHECK(xb_copy2d(b->as<void>(), (int64_t)b->size(), b->data_type(), d->blob->as<void>(), (int64_t)b->size(), XB_F32,
                       1, (int64_t)b->size(), s));
    ++*launches;
    d->valid = true;
    d->src = b->as<void>();
  }
  return d->blob->as<float>();
}

// ---- ConstantFill -----------------------------------------------------------------------------
class ConstantFillOp final : public Operator<CUDAContext> {
 public:
  ConstantFillOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    Blob* out = Output(0);
    if (!constant_fresh) return;                       // another predictor of this model filled it
    const int dtype = GetSingleArgument<int>("dtype", kFloat);
    std::vector<TIndex> shape;
    for (int64_t d : GetRepeatedArgument<int64_t>("shape")) shape.push_back((TIndex)d);
    out->set_data_type(dtype);
    out->Reshape(shape);
    out->is_constant = true;
    const Argument* v = def.FindArg("value");
    BLAZE_CONDITION_THROW(v != nullptr, "ConstantFill without value", def.DebugString());
    const size_t n = out->size();
    std::vector<char>& host = out->host_copy;
    host.assign(n * DataTypeSize(dtype), 0);
    auto count = [&](size_t have) {
      BLAZE_CONDITION_THROW(have == n, "value.size()=", have, " output->size()=", n, def.DebugString());
    };
    if (dtype == kFloat || dtype == kFloat16) {
      std::vector<float> f = v->floats;
      if (f.empty() && !v->ints.empty()) f.assign(v->ints.begin(), v->ints.end());
      if (f.empty() && v->has_f) f.assign(1, v->f);
      count(f.size());
      if (dtype == kFloat) memcpy(host.data(), f.data(), n * 4);
      else for (size_t i = 0; i < n; ++i) reinterpret_cast<uint16_t*>(host.data())[i] = FloatToHalfBits(f[i]);
    } else if (dtype == kInt32 || dtype == kInt64) {
      std::vector<int64_t> iv = v->ints;
      if (iv.empty() && !v->floats.empty()) iv.assign(v->floats.begin(), v->floats.end());
      if (iv.empty() && v->has_i) iv.assign(1, v->i);
      count(iv.size());
      if (dtype == kInt64) memcpy(host.data(), iv.data(), n * 8);
      else for (size_t i = 0; i < n; ++i) reinterpret_cast<int32_t*>(host.data())[i] = (int32_t)iv[i];
    } else {
      BLAZE_THROW("ConstantFill: unsupported dtype ", dtype);
    }
    context_.Activate();
    if (n) CUDA_CHECK(cudaMemcpy(out->as<void>(), host.data(), host.size(), cudaMemcpyHostToDevice));
  }
  bool RunOnDevice() override { return true; }
};
REGISTER_CUDA_OPERATOR(ConstantFill, ConstantFillOp);
OPERATOR_SCHEMA(ConstantFill).NumInputs(0).NumOutputs(1);

// ---- Gemm family --------------------------------------------------------------------------------
struct GemmCommon {
  bool transa = false, transb = false;
  float alpha = 1.f, beta = 1.f;
};

// Weights of an fp16 model are packed once to K-major [N, ldk] so the tcgen05 engine can take them.
struct PackedWeight {
  std::unique_ptr<Blob> blob;
  const void* src = nullptr;
  int64_t ldk = 0;
};

const void* PackIfUseful(Blob* w, bool transb, int K, int N, int batch, PackedWeight* pw, cudaStream_t s,
                         int* launches, bool* now_transb, int64_t* ldb, int64_t* stride_b) {
  *now_transb = transb;
  *ldb = transb ? K : N;
  *stride_b = (int64_t)K * N;
  const bool half = w->data_type() == kFloat16;
  if (!half || !w->is_constant) return w->as<void>();
  if (transb && K % 8 == 0) return w->as<void>();        // already K-major and TMA-aligned
  if (transb) return w->as<void>();                       // K-major but unaligned: the CUDA-core engine takes it
  if (pw->src != w->as<void>()) {
    pw->ldk = (K + 7) / 8 * 8;
    pw->blob.reset(new Blob(w->device_option()));
    pw->blob->set_data_type(kFloat16);
    pw->blob->Reshape({(TIndex)batch, (TIndex)N, (TIndex)pw->ldk});
    XB_CHECK(xb_pack_weight_kmajor(w->as<void>(), XB_F16, K, N, N, pw->blob->as<void>(), XB_F16, pw->ldk, batch,
                                   (int64_t)K * N, (int64_t)N * pw->ldk, s));
    ++*launches;
    pw->src = w->as<void>();
  }
  *now_transb = true;
  *ldb = pw->ldk;
  *stride_b = (int64_t)N * pw->ldk;
  return pw->blob->as<void>();
}

class GemmOp final : public Operator<CUDAContext> {
 public:
  GemmOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    c_.transa = GetSingleArgument<bool>("transA", false);
    c_.transb = GetSingleArgument<bool>("transB", false);
    c_.alpha = GetSingleArgument<float>("alpha", 1.0f);
    c_.beta = GetSingleArgument<float>("beta", 1.0f);
    epilogue_ = GetSingleArgument<int>("epilogue", XB_EPI_NONE);
    nosqrt_ = GetSingleArgument<bool>("nosqrt", false);
  }

  bool RunOnDevice() override {
    Blob* a = Input(0);
    Blob* b = Input(1);
    const size_t n_epi = epilogue_ == XB_EPI_DICE ? 3 : (epilogue_ == XB_EPI_PRELU ? 1 : 0);
    const size_t n_plain = InputSize() - n_epi;
    Blob* c = n_plain > 2 ? Input(2) : nullptr;
    Blob* y = Output(0);
    CheckValid(a, b, c);
    const auto& as = a->shape();
    const auto& bs = b->shape();
    TIndex M = as.size() == 3 ? as[1] : as[0];
    TIndex K = as.size() == 3 ? as[2] : as[1];
    if (c_.transa) std::swap(M, K);
    const TIndex N = c_.transb ? bs[0] : bs[1];
    int batch = 1;
    int64_t stride_a = 0, stride_y = 0;
    y->set_data_type(a->data_type());
    if (as.size() == 3) {
      y->Reshape({as[0], M, N});
      if (M == 1 || !c_.transa) {
        M = as[0] * M;                         // rows are contiguous: one 2-D product
      } else {
        batch = (int)as[0]; stride_a = (int64_t)M * K; stride_y = (int64_t)M * N;
      }
    } else {
      y->Reshape({M, N});
    }
    xb_gemm_args g;
    memset(&g, 0, sizeof(g));
    cudaStream_t s = context_.cuda_stream();
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.trans_a = c_.transa;
    g.alpha = c_.alpha; g.beta = c ? c_.beta : 0.f;
    g.A = a->as<void>(); g.lda = c_.transa ? M : K; g.stride_a = stride_a;
    if (as.size() == 3 && c_.transa) g.lda = as[2];
    bool tb; int64_t ldb, sb;
    g.B = PackIfUseful(b, c_.transb, (int)K, (int)N, 1, &packed_, s, &launches, &tb, &ldb, &sb);
    g.trans_b = tb; g.ldb = ldb; g.stride_b = 0;
    if (c) {
      g.bias = c->as<void>(); g.bias_dtype = c->data_type();
      g.bias_kind = c->shape().size() == 2 ? XB_BIAS_FULL : XB_BIAS_ROW;
      g.ldbias = N; g.stride_bias = 0;
      // a full [M,N] bias of a 3-D product repeats for every batch row block
      BLAZE_CONDITION_THROW(!(g.bias_kind == XB_BIAS_FULL && as.size() == 3 && batch == 1 && as[0] > 1),
                            "Gemm: a rank-2 bias with a 3-D input is not supported");
    }
    g.Y = y->as<void>(); g.ldy = N; g.stride_y = stride_y; g.batch = batch;
    g.ab_dtype = a->data_type(); g.y_dtype = y->data_type();
    g.epilogue = epilogue_; g.dice_nosqrt = nosqrt_;
    if (epilogue_ == XB_EPI_PRELU) {
      Blob* w = Input(n_plain);
      g.ep_a = AsF32(w, &ep_[0], s, &launches);
      g.ep_count = (int)w->size();
      BLAZE_CONDITION_THROW(g.ep_count == 1 || g.ep_count == (int)N, "PRelu slopes ", g.ep_count, " for N=", N);
    } else if (epilogue_ == XB_EPI_DICE) {
      g.ep_a = AsF32(Input(n_plain), &ep_[0], s, &launches);
      g.ep_b = AsF32(Input(n_plain + 1), &ep_[1], s, &launches);
      g.ep_c = AsF32(Input(n_plain + 2), &ep_[2], s, &launches);
    }
    XB_CHECK(xb_gemm(&g, s));
    ++launches;
    return true;
  }

 private:
  void CheckValid(Blob* a, Blob* b, Blob* c) {
    BLAZE_CONDITION_THROW(a->shape().size() == 2 || a->shape().size() == 3, "a->shape.size()=", a->shape().size());
    BLAZE_CONDITION_THROW(b->shape().size() == 2, "b->shape.size()=", b->shape().size(), def_.DebugString());
    if (c) BLAZE_CONDITION_THROW(c->shape().size() <= 2, "c->shape().size()=", c->shape().size());
    const auto& as = a->shape();
    const auto& bs = b->shape();
    TIndex a_m = as.size() == 3 ? as[1] : as[0], a_k = as.size() == 3 ? as[2] : as[1];
    if (c_.transa) std::swap(a_m, a_k);
    TIndex b_k = bs[0], b_n = bs[1];
    if (c_.transb) std::swap(b_k, b_n);
    BLAZE_CONDITION_THROW(a_k == b_k, "a_k=", a_k, " b_k=", b_k, def_.DebugString());
    BLAZE_CONDITION_THROW(a->data_type() == b->data_type(), "a->data_type()=", a->data_type(), " b->data_type()=", b->data_type());
    if (c) {
      if (c->shape().size() == 2) {
        BLAZE_CONDITION_THROW(a_m == c->shape()[0], "a_m=", a_m, " c->shape()[0]=", c->shape()[0]);
        BLAZE_CONDITION_THROW(b_n == c->shape()[1], "b_n=", b_n, " c->shape()[1]=", c->shape()[1]);
      } else {
        BLAZE_CONDITION_THROW(b_n == c->shape()[0], "b_n=", b_n, " c->shape()[0]=", c->shape()[0]);
      }
    }
  }
  GemmCommon c_;
  int epilogue_;
  bool nosqrt_;
  PackedWeight packed_;
  Derived ep_[3];
};
REGISTER_CUDA_OPERATOR(Gemm, GemmOp);
OPERATOR_SCHEMA(Gemm).NumInputs(2, 6).NumOutputs(1);

// PrunedGemm: [X1 | X2] x [W1 ; W2] = X1 x W1 + X2 x W2 (+ bias), the "common features computed once"
// product (blaze/blaze/operator/op/pruned_gemm_op.h:1-163). The reference takes operands with equal
// row counts or one of them with a single row that is broadcast; here the short operand may also have
// m rows with the long one a multiple of m: row i of the long operand pairs with row i / (M/m) of the
// short one, which is the one-row case applied to m requests in one launch. The short product (with the
// bias) is kept in fp32 and added in the epilogue of the long one, before the optional fused activation
// and the single rounding to the output type. (In the equal-rows branch the reference passes X2 for both
// operands of its second Gemm, pruned_gemm_op.h:95-105; the product computed here is X2 x W2.)
class PrunedGemmOp final : public Operator<CUDAContext> {
 public:
  PrunedGemmOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    c_.transa = GetSingleArgument<bool>("transA", false);
    c_.transb = GetSingleArgument<bool>("transB", false);
    c_.alpha = GetSingleArgument<float>("alpha", 1.0f);
    c_.beta = GetSingleArgument<float>("beta", 1.0f);
    epilogue_ = GetSingleArgument<int>("epilogue", XB_EPI_NONE);
    nosqrt_ = GetSingleArgument<bool>("nosqrt", false);
    BLAZE_CONDITION_THROW(!c_.transa, "PrunedGemm: transA is not supported");
  }

  bool RunOnDevice() override {
    const size_t n_epi = epilogue_ == XB_EPI_DICE ? 3 : (epilogue_ == XB_EPI_PRELU ? 1 : 0);
    const size_t n_plain = InputSize() - n_epi;
    BLAZE_CONDITION_THROW(n_plain == 4 || n_plain == 5, "PrunedGemm takes x1, x2, w1, w2 and an optional bias");
    Blob *x1 = Input(0), *x2 = Input(1), *w1 = Input(2), *w2 = Input(3);
    Blob* bias = n_plain > 4 ? Input(4) : nullptr;
    Blob* y = Output(0);
    for (Blob* b : {x1, x2, w1, w2})
      BLAZE_CONDITION_THROW(b->shape().size() == 2, "PrunedGemm: only 2-D operands, got rank ", b->shape().size());
    BLAZE_CONDITION_THROW(x1->data_type() == x2->data_type() && x1->data_type() == w1->data_type() &&
                          w1->data_type() == w2->data_type(), "PrunedGemm: operand data types differ");
    const TIndex m1 = x1->shape()[0], k1 = x1->shape()[1], m2 = x2->shape()[0], k2 = x2->shape()[1];
    const TIndex n1 = c_.transb ? w1->shape()[0] : w1->shape()[1], n2 = c_.transb ? w2->shape()[0] : w2->shape()[1];
    BLAZE_CONDITION_THROW((c_.transb ? w1->shape()[1] : w1->shape()[0]) == k1, "x1_k=", k1, " does not match w1");
    BLAZE_CONDITION_THROW((c_.transb ? w2->shape()[1] : w2->shape()[0]) == k2, "x2_k=", k2, " does not match w2");
    BLAZE_CONDITION_THROW(n1 == n2, "w1_n=", n1, " w2_n=", n2);
    const TIndex M = std::max(m1, m2), m = std::min(m1, m2), N = n1;
    BLAZE_CONDITION_THROW(m > 0 && M % m == 0, "PrunedGemm: row counts ", m1, " and ", m2, " do not broadcast");
    if (bias) BLAZE_CONDITION_THROW(bias->size() == (size_t)N, "PrunedGemm: bias of ", bias->size(), " for N=", N);
    const bool first_short = m1 <= m2;
    Blob* xs = first_short ? x1 : x2;          // short operand: computed once per row group
    Blob* ws = first_short ? w1 : w2;
    Blob* xl = first_short ? x2 : x1;
    Blob* wl = first_short ? w2 : w1;
    const TIndex ks = first_short ? k1 : k2, kl = first_short ? k2 : k1;
    y->set_data_type(x1->data_type());
    y->Reshape({M, N});
    cudaStream_t s = context_.cuda_stream();
    if (!partial_) partial_.reset(new Blob(device_option_));
    partial_->set_data_type(kFloat);
    partial_->Reshape({m, N});

    xb_gemm_args g;
    memset(&g, 0, sizeof(g));
    bool tb; int64_t ldb, sb;
    // short product: partial = alpha * xs x ws + beta * bias, fp32
    g.M = (int)m; g.N = (int)N; g.K = (int)ks; g.alpha = c_.alpha; g.beta = bias ? c_.beta : 0.f;
    g.A = xs->as<void>(); g.lda = ks;
    g.B = PackIfUseful(ws, c_.transb, (int)ks, (int)N, 1, &packed_[0], s, &launches, &tb, &ldb, &sb);
    g.trans_b = tb; g.ldb = ldb;
    if (bias) { g.bias = bias->as<void>(); g.bias_dtype = bias->data_type(); g.bias_kind = XB_BIAS_ROW; }
    g.Y = partial_->as<void>(); g.ldy = N; g.batch = 1;
    g.ab_dtype = xs->data_type(); g.y_dtype = kFloat;
    XB_CHECK(xb_gemm(&g, s));
    ++launches;
    // long product with the short one added per row group, then the activation
    memset(&g, 0, sizeof(g));
    g.M = (int)M; g.N = (int)N; g.K = (int)kl; g.alpha = c_.alpha; g.beta = 1.f;
    g.A = xl->as<void>(); g.lda = kl;
    g.B = PackIfUseful(wl, c_.transb, (int)kl, (int)N, 1, &packed_[1], s, &launches, &tb, &ldb, &sb);
    g.trans_b = tb; g.ldb = ldb;
    g.bias = partial_->as<void>(); g.bias_dtype = kFloat; g.bias_kind = XB_BIAS_FULL; g.ldbias = N;
    g.bias_row_group = M / m;
    g.Y = y->as<void>(); g.ldy = N; g.batch = 1;
    g.ab_dtype = xl->data_type(); g.y_dtype = y->data_type();
    g.epilogue = epilogue_; g.dice_nosqrt = nosqrt_;
    if (epilogue_ == XB_EPI_PRELU) {
      Blob* w = Input(n_plain);
      g.ep_a = AsF32(w, &ep_[0], s, &launches);
      g.ep_count = (int)w->size();
      BLAZE_CONDITION_THROW(g.ep_count == 1 || g.ep_count == (int)N, "PRelu slopes ", g.ep_count, " for N=", N);
    } else if (epilogue_ == XB_EPI_DICE) {
      g.ep_a = AsF32(Input(n_plain), &ep_[0], s, &launches);
      g.ep_b = AsF32(Input(n_plain + 1), &ep_[1], s, &launches);
      g.ep_c = AsF32(Input(n_plain + 2), &ep_[2], s, &launches);
    }
    XB_CHECK(xb_gemm(&g, s));
    ++launches;
    return true;
  }

 private:
  GemmCommon c_;
  int epilogue_;
  bool nosqrt_;
  PackedWeight packed_[2];
  Derived ep_[3];
  std::unique_ptr<Blob> partial_;
};
REGISTER_CUDA_OPERATOR(PrunedGemm, PrunedGemmOp);
OPERATOR_SCHEMA(PrunedGemm).NumInputs(4, 8).NumOutputs(1);

class FusedParallelGemmOp final : public Operator<CUDAContext> {
 public:
  FusedParallelGemmOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    c_.transa = GetSingleArgument<bool>("transA", false);
    c_.transb = GetSingleArgument<bool>("transB", false);
    c_.alpha = GetSingleArgument<float>("alpha", 1.0f);
    c_.beta = GetSingleArgument<float>("beta", 1.0f);
    parallel_num_ = GetSingleArgument<int>("parallel_num", 1);
    BLAZE_CONDITION_THROW(parallel_num_ >= 1, "parallel_num=", parallel_num_);
  }
  bool RunOnDevice() override {
    Blob* a = Input(0);
    Blob* b = Input(1);
    Blob* c = InputSize() > 2 ? Input(2) : nullptr;
    Blob* y = Output(0);
    const auto& as = a->shape();
    const auto& bs = b->shape();
    BLAZE_CONDITION_THROW(as.size() == 2 || as.size() == 3, "a->shape.size()=", as.size());
    BLAZE_CONDITION_THROW(bs.size() == 2, "b->shape.size()=", bs.size());
    const int P = parallel_num_;
    TIndex M = as.size() == 3 ? as[1] : as[0], K = as.size() == 3 ? as[2] : as[1];
    if (c_.transa) std::swap(M, K);
    const TIndex N = c_.transb ? bs[0] / P : bs[1];
    const TIndex b_k = c_.transb ? bs[1] : bs[0] / P;
    BLAZE_CONDITION_THROW(b_k == K && (c_.transb ? bs[0] : bs[0]) % P == 0, "a_k=", K, " b_k=", b_k, def_.DebugString());
    y->set_data_type(a->data_type());
    TIndex outer = 1;
    if (as.size() == 3) {
      y->Reshape({as[0] * P, M, N});
      BLAZE_CONDITION_THROW(M == 1 || !c_.transa, "FusedParallelGemm: transposed 3-D input is not supported");
      outer = as[0];
      M = as[0] * M;
    } else {
      y->Reshape({M * P, N});
    }
    (void)outer;
    xb_gemm_args g;
    memset(&g, 0, sizeof(g));
    cudaStream_t s = context_.cuda_stream();
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.trans_a = c_.transa;
    g.alpha = c_.alpha; g.beta = c ? c_.beta : 0.f;
    g.A = a->as<void>(); g.lda = c_.transa ? M : K; g.stride_a = 0;       // every branch reads the same input
    bool tb; int64_t ldb, sb;
    g.B = PackIfUseful(b, c_.transb, (int)K, (int)N, P, &packed_, s, &launches, &tb, &ldb, &sb);
    g.trans_b = tb; g.ldb = ldb; g.stride_b = sb;
    if (c) {
      g.bias = c->as<void>(); g.bias_dtype = c->data_type();
      if (c->shape().size() == 2) {
        BLAZE_CONDITION_THROW(c->shape()[0] == M * P && c->shape()[1] == N, "bias shape mismatch", def_.DebugString());
        g.bias_kind = XB_BIAS_FULL; g.ldbias = N; g.stride_bias = (int64_t)M * N;
      } else {
        BLAZE_CONDITION_THROW(c->shape()[0] == N * P, "c->shape()[0]=", c->shape()[0], " N*P=", N * P);
        g.bias_kind = XB_BIAS_ROW; g.stride_bias = N;
      }
    }
    g.Y = y->as<void>(); g.ldy = N; g.stride_y = (int64_t)M * N; g.batch = P;
    g.ab_dtype = a->data_type(); g.y_dtype = y->data_type();
    XB_CHECK(xb_gemm(&g, s));
    ++launches;
    return true;
  }

 private:
  GemmCommon c_;
  int parallel_num_;
  PackedWeight packed_;
};
REGISTER_CUDA_OPERATOR(FusedParallelGemm, FusedParallelGemmOp);
OPERATOR_SCHEMA(FusedParallelGemm).NumInputs(2, 3).NumOutputs(1);

// numpy-style batched matmul with at most one leading batch dimension per operand
void BatchedMatMul(const GemmCommon& c, const void* a, const std::vector<TIndex>& as, const void* b,
                   const std::vector<TIndex>& bs, void* y, int dtype, cudaStream_t s, std::vector<TIndex>* yshape) {
  BLAZE_CONDITION_THROW(as.size() >= 2 && bs.size() >= 2, "MatMul operands need rank >= 2");
  TIndex M = as[as.size() - 2], K = as[as.size() - 1];
  if (c.transa) std::swap(M, K);
  const TIndex N = c.transb ? bs[bs.size() - 2] : bs[bs.size() - 1];
  const TIndex bk = c.transb ? bs[bs.size() - 1] : bs[bs.size() - 2];
  BLAZE_CONDITION_THROW(bk == K, "a_k=", K, " b_k=", bk);
  TIndex na = 1, nb = 1;
  for (size_t i = 0; i + 2 < as.size(); ++i) na *= as[i];
  for (size_t i = 0; i + 2 < bs.size(); ++i) nb *= bs[i];
  BLAZE_CONDITION_THROW(na == nb || na == 1 || nb == 1, "a_size=", na, " b_size=", nb);
  const TIndex batch = std::max(na, nb);
  xb_gemm_args g;
  memset(&g, 0, sizeof(g));
  g.M = (int)M; g.N = (int)N; g.K = (int)K; g.trans_a = c.transa; g.trans_b = c.transb;
  g.alpha = 1.f; g.beta = 0.f;
  g.A = a; g.lda = as[as.size() - 1]; g.stride_a = (na == 1 && batch > 1) ? 0 : (int64_t)M * K;
  g.B = b; g.ldb = bs[bs.size() - 1]; g.stride_b = (nb == 1 && batch > 1) ? 0 : (int64_t)K * N;
  g.Y = y; g.ldy = N; g.stride_y = (int64_t)M * N; g.batch = (int)batch;
  g.ab_dtype = dtype; g.y_dtype = dtype;
  XB_CHECK(xb_gemm(&g, s));
  if (yshape) {
    const std::vector<TIndex>& lead = na >= nb ? as : bs;
    yshape->assign(lead.begin(), lead.end() - 2);
    yshape->push_back(M);
    yshape->push_back(N);
  }
}

class MatMulOp final : public Operator<CUDAContext> {
 public:
  MatMulOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    c_.transa = GetSingleArgument<bool>("transA", false);
    c_.transb = GetSingleArgument<bool>("transB", false);
  }
  bool RunOnDevice() override {
    Blob* a = Input(0);
    Blob* b = Input(1);
    Blob* y = Output(0);
    // output shape first (needs the sizes), then the product
    std::vector<TIndex> as = a->shape(), bs = b->shape();
    if (as.size() == 1) as.insert(as.begin(), 1);
    if (bs.size() == 1) bs.push_back(1);
    TIndex M = as[as.size() - 2], K = as[as.size() - 1];
    if (c_.transa) std::swap(M, K);
    const TIndex N = c_.transb ? bs[bs.size() - 2] : bs[bs.size() - 1];
    TIndex na = 1, nb = 1;
    for (size_t i = 0; i + 2 < as.size(); ++i) na *= as[i];
    for (size_t i = 0; i + 2 < bs.size(); ++i) nb *= bs[i];
    std::vector<TIndex> ys((na >= nb ? as : bs).begin(), (na >= nb ? as : bs).end() - 2);
    ys.push_back(M); ys.push_back(N);
    y->set_data_type(a->data_type());
    y->Reshape(ys);
    BatchedMatMul(c_, a->as<void>(), as, b->as<void>(), bs, y->as<void>(), a->data_type(), context_.cuda_stream(), nullptr);
    ++launches;
    return true;
  }

 private:
  GemmCommon c_;
};
REGISTER_CUDA_OPERATOR(MatMul, MatMulOp);
OPERATOR_SCHEMA(MatMul).NumInputs(2).NumOutputs(1);

class FusedParallelMatMulOp final : public Operator<CUDAContext> {
 public:
  FusedParallelMatMulOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    c_.transa = GetSingleArgument<bool>("transA", false);
    c_.transb = GetSingleArgument<bool>("transB", false);
    parallel_num_ = GetSingleArgument<int>("parallel_num", 1);
  }
  bool RunOnDevice() override {
    Blob* a = Input(0);
    Blob* b = Input(1);
    Blob* y = Output(0);
    const int P = parallel_num_;
    std::vector<TIndex> as = a->shape(), bs = b->shape();
    BLAZE_CONDITION_THROW(as.size() >= 3 && bs.size() >= 3 && as[0] % P == 0 && bs[0] % P == 0,
                          "FusedParallelMatMul: leading dims must be multiples of parallel_num", def_.DebugString());
    as[0] /= P; bs[0] /= P;
    TIndex M = as[as.size() - 2], K = as[as.size() - 1];
    if (c_.transa) std::swap(M, K);
    const TIndex N = c_.transb ? bs[bs.size() - 2] : bs[bs.size() - 1];
    TIndex na = 1, nb = 1;
    for (size_t i = 0; i + 2 < as.size(); ++i) na *= as[i];
    for (size_t i = 0; i + 2 < bs.size(); ++i) nb *= bs[i];
    const TIndex per = std::max(na, nb);
    y->set_data_type(a->data_type());
    y->Reshape({per * P, M, N});
    const size_t es = DataTypeSize(a->data_type());
    for (int p = 0; p < P; ++p) {
      BatchedMatMul(c_, a->as<char>() + (size_t)p * na * M * K * es, as, b->as<char>() + (size_t)p * nb * K * N * es, bs,
                    y->as<char>() + (size_t)p * per * M * N * es, a->data_type(), context_.cuda_stream(), nullptr);
      ++launches;
    }
    return true;
  }

 private:
  GemmCommon c_;
  int parallel_num_;
};
REGISTER_CUDA_OPERATOR(FusedParallelMatMul, FusedParallelMatMulOp);
OPERATOR_SCHEMA(FusedParallelMatMul).NumInputs(2).NumOutputs(1);

// ---- activations ---------------------------------------------------------------------------------
class DiceOp final : public Operator<CUDAContext> {
 public:
  DiceOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    nosqrt_ = GetSingleArgument<bool>("nosqrt", false);
  }
  bool RunOnDevice() override {
    Blob *x = Input(0), *gamma = Input(1), *mean = Input(2), *var = Input(3), *y = Output(0);
    BLAZE_CONDITION_THROW(!x->shape().empty(), "Dice: empty shape");
    const TIndex c = x->shape().back();
    BLAZE_CONDITION_THROW(gamma->size() == c && mean->size() == c && var->size() == c, "Dice: parameter size != ", c);
    BLAZE_CONDITION_THROW(gamma->data_type() == x->data_type(), "Dice: parameter dtype differs from x");
    y->set_data_type(x->data_type());
    y->Reshape(x->shape());
    XB_CHECK(xb_dice(x->as<void>(), y->as<void>(), (int64_t)(x->size() / c), (int)c, gamma->as<void>(), mean->as<void>(),
                     var->as<void>(), nosqrt_, x->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
  bool nosqrt_;
};
REGISTER_CUDA_OPERATOR(Dice, DiceOp);
OPERATOR_SCHEMA(Dice).NumInputs(4).NumOutputs(1);

class PReluOp final : public Operator<CUDAContext> {
 public:
  using Operator<CUDAContext>::Operator;
  bool RunOnDevice() override {
    Blob *x = Input(0), *w = Input(1), *y = Output(0);
    y->set_data_type(x->data_type());
    y->Reshape(x->shape());
    XB_CHECK(xb_prelu(x->as<void>(), y->as<void>(), (int64_t)x->size(), w->as<void>(), (int64_t)w->size(), x->data_type(),
                      w->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
};
REGISTER_CUDA_OPERATOR(PRelu, PReluOp);
OPERATOR_SCHEMA(PRelu).NumInputs(2).NumOutputs(1);

class SigmoidOp final : public Operator<CUDAContext> {
 public:
  using Operator<CUDAContext>::Operator;
  bool RunOnDevice() override {
    Blob *x = Input(0), *y = Output(0);
    y->set_data_type(x->data_type());
    y->Reshape(x->shape());
    XB_CHECK(xb_sigmoid(x->as<void>(), y->as<void>(), (int64_t)x->size(), x->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
};
REGISTER_CUDA_OPERATOR(Sigmoid, SigmoidOp);
OPERATOR_SCHEMA(Sigmoid).NumInputs(1).NumOutputs(1);

class SoftmaxOp final : public Operator<CUDAContext> {
 public:
  SoftmaxOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    axis_ = GetSingleArgument<size_t>("axis", 1);
  }
  bool RunOnDevice() override {
    Blob *x = Input(0), *y = Output(0);
    BLAZE_CONDITION_THROW(axis_ < x->shape().size(), "Softmax axis ", axis_, " for rank ", x->shape().size());
    y->set_data_type(x->data_type());
    y->Reshape(x->shape());
    XB_CHECK(xb_softmax(x->as<void>(), y->as<void>(), (int64_t)x->size(0, axis_), (int)x->shape()[axis_],
                        (int64_t)x->size(axis_ + 1, x->shape().size()), x->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
  size_t axis_;
};
REGISTER_CUDA_OPERATOR(Softmax, SoftmaxOp);
OPERATOR_SCHEMA(Softmax).NumInputs(1).NumOutputs(1);

class BatchNormalizationOp final : public Operator<CUDAContext> {
 public:
  BatchNormalizationOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    nosqrt_ = GetSingleArgument<bool>("nosqrt", false);
    eps_ = GetSingleArgument<float>("eps", 0.001f);
  }
  bool RunOnDevice() override {
    Blob *x = Input(0), *y = Output(0);
    const TIndex c = x->shape().back();
    for (int i = 1; i <= 4; ++i) BLAZE_CONDITION_THROW(Input(i)->size() == c, "BatchNormalization: parameter ", i, " size != ", c);
    y->set_data_type(x->data_type());
    y->Reshape(x->shape());
    XB_CHECK(xb_batchnorm(x->as<void>(), y->as<void>(), (int64_t)x->size(), (int)c, Input(1)->as<void>(), Input(2)->as<void>(),
                          Input(3)->as<void>(), Input(4)->as<void>(), eps_, nosqrt_, x->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
  bool nosqrt_;
  float eps_;
};
REGISTER_CUDA_OPERATOR(BatchNormalization, BatchNormalizationOp);
OPERATOR_SCHEMA(BatchNormalization).NumInputs(5).NumOutputs(1);

// ---- GRU -----------------------------------------------------------------------------------------
// from_deepnet layout: inputs x, h2h, i2h, h2h_bias, i2h_bias; otherwise x, i2h, h2h, bias [i2h_bias | h2h_bias]
// and the sequence is output 1 (blaze/blaze/operator/op/gru_op.h:66-150).
class GRUOp final : public Operator<CUDAContext> {
 public:
  GRUOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    from_deepnet_ = GetSingleArgument<bool>("from_deepnet", false);
  }
  bool RunOnDevice() override {
    Blob* x = Input(0);
    const auto& xs = x->shape();
    BLAZE_CONDITION_THROW(xs.size() == 2 || xs.size() == 3, "x_shape.size()=", xs.size());
    Blob *h2h, *i2h, *y;
    const void *bi, *bh;
    if (from_deepnet_) {
      BLAZE_CONDITION_THROW(InputSize() == 5, "GRU(from_deepnet) takes 5 inputs");
      h2h = Input(1); i2h = Input(2); bh = Input(3)->as<void>(); bi = Input(4)->as<void>(); y = Output(0);
    } else {
      BLAZE_CONDITION_THROW(InputSize() == 4 && OutputSize() >= 2, "GRU takes 4 inputs and writes output 1");
      i2h = Input(1); h2h = Input(2); y = Output(1);
      Blob* bias = Input(3);
      bi = bias->as<void>();
      bh = bias->as<char>() + bias->size() / 2 * DataTypeSize(bias->data_type());
    }
    const TIndex batch = xs.size() < 3 ? 1 : xs[0], T = xs[xs.size() - 2], H = h2h->shape()[0];
    BLAZE_CONDITION_THROW(xs.back() == H && i2h->shape()[0] == H && h2h->shape()[1] == 3 * H, "GRU: input dim must equal hidden ", H);
    y->set_data_type(x->data_type());
    y->Reshape({batch, T, H});
    XB_CHECK(xb_gru(x->as<void>(), y->as<void>(), (int64_t)batch, (int)T, (int)H, i2h->as<void>(), h2h->as<void>(), bi, bh,
                    x->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
  bool from_deepnet_;
};
REGISTER_CUDA_OPERATOR(GRU, GRUOp);
OPERATOR_SCHEMA(GRU).NumInputs(4, 5).NumOutputs(1, 2);

// ---- fused DIN operators (no reference operator: they replace whole sub-graphs) -------------------
// DinAttention: inputs q [R*n, d] | [R, n, d], k [R, T, d], W0 [4d,h0], b0, W1 [h0,h1], b1, W2 [h1,1], b2,
// then for act=dice gamma0, mean0, var0, gamma1, mean1, var1; optional last input seq_len int32 [R].
class DinAttentionOp final : public Operator<CUDAContext> {
 public:
  DinAttentionOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    act_ = GetSingleArgument<int>("act", XB_ACT_DICE);
    softmax_ = GetSingleArgument<bool>("softmax", false);
    engine_ = GetSingleArgument<int>("engine", XB_GEMM_AUTO);
  }
  bool RunOnDevice() override {
    Blob *q = Input(0), *k = Input(1), *y = Output(0);
    BLAZE_CONDITION_THROW(q->data_type() == kFloat16 && k->data_type() == kFloat16, "DinAttention needs fp16 q and k");
    BLAZE_CONDITION_THROW(k->shape().size() == 3, "k must be [requests, T, d]");
    const int R = (int)k->shape()[0], T = (int)k->shape()[1], d = (int)k->shape()[2];
    BLAZE_CONDITION_THROW(q->shape().back() == (TIndex)d && q->size() % ((size_t)R * d) == 0, "q shape does not match k");
    const int n_cand = (int)(q->size() / ((size_t)R * d));
    const size_t n_w = act_ == XB_ACT_DICE ? 12 : 6;
    BLAZE_CONDITION_THROW(InputSize() == 2 + n_w || InputSize() == 3 + n_w, "DinAttention: ", InputSize(), " inputs");
    cudaStream_t s = context_.cuda_stream();
    Blob *W0 = Input(2), *W1 = Input(4), *W2 = Input(6);
    const int h0 = (int)W0->shape()[1], h1 = (int)W1->shape()[1];
    BLAZE_CONDITION_THROW(W0->shape()[0] == (TIndex)4 * d && W1->shape()[0] == (TIndex)h0 && W2->size() == (size_t)h1,
                          "DinAttention: weight shapes do not chain");
    xb_din_att_args a;
    memset(&a, 0, sizeof(a));
    // weights: K-major fp16 copies, packed once
    bool tb; int64_t ld, sb;
    a.w.W0 = Pack(W0, 4 * d, h0, &pw0_, s);
    a.w.W1 = Pack(W1, h0, h1, &pw1_, s);
    (void)tb; (void)ld; (void)sb;
    a.w.W2 = AsF32(W2, &f_[0], s, &launches);
    a.w.b0 = AsF32(Input(3), &f_[1], s, &launches);
    a.w.b1 = AsF32(Input(5), &f_[2], s, &launches);
    a.w.b2 = HostScalar(Input(7));
    if (act_ == XB_ACT_DICE) {
      a.w.gamma0 = AsF32(Input(8), &f_[3], s, &launches); a.w.mean0 = AsF32(Input(9), &f_[4], s, &launches);
      a.w.var0 = AsF32(Input(10), &f_[5], s, &launches); a.w.gamma1 = AsF32(Input(11), &f_[6], s, &launches);
      a.w.mean1 = AsF32(Input(12), &f_[7], s, &launches); a.w.var1 = AsF32(Input(13), &f_[8], s, &launches);
    }
    if (InputSize() == 3 + n_w) a.seq_len = Input(2 + n_w)->as<int32_t>();
    y->set_data_type(kFloat16);
    y->Reshape({(TIndex)R * n_cand, (TIndex)d});
    a.q = q->as<void>(); a.ldq = d; a.k = k->as<void>(); a.ldk = d; a.out = y->as<void>(); a.ldo = d;
    a.requests = R; a.n_cand = n_cand; a.T = T; a.d = d; a.h0 = h0; a.h1 = h1;
    a.act = act_; a.use_softmax = softmax_; a.engine = engine_;
    if (!operands_) {
      // all weights are constants (checked in HostScalar/Pack): lay the MMA operands out once
      const size_t n = xb_din_attention_packed_bytes(d, h0, h1);
      operands_.reset(new Blob(q->device_option()));
      operands_->set_data_type(kFloat);
      operands_->Reshape({(TIndex)((n + 3) / 4)});
      has_operands_ = n != 0 && W0->is_constant && W1->is_constant && W2->is_constant;
      if (has_operands_) {
        XB_CHECK(xb_din_attention_pack(&a, operands_->as<void>(), n, s));
        ++launches;
      }
    }
    if (has_operands_) a.w.packed = operands_->as<void>();
    XB_CHECK(xb_din_attention(&a, s));
    ++launches;
    return true;
  }

 private:
  // exact-size K-major fp16 copy [N, K] of a [K, N] weight
  const void* Pack(Blob* w, int K, int N, PackedWeight* pw, cudaStream_t s) {
    if (pw->src != w->as<void>() || !w->is_constant) {
      if (!pw->blob) pw->blob.reset(new Blob(w->device_option()));
      pw->blob->set_data_type(kFloat16);
      pw->blob->Reshape({(TIndex)N, (TIndex)K});
      XB_CHECK(xb_pack_weight_kmajor(w->as<void>(), w->data_type(), K, N, N, pw->blob->as<void>(), XB_F16, K, 1, 0, 0, s));
      ++launches;
      pw->src = w->as<void>();
    }
    return pw->blob->as<void>();
  }
  float HostScalar(Blob* b) {
    BLAZE_CONDITION_THROW(b->is_constant && !b->host_copy.empty(), "DinAttention: b2 must be a constant");
    if (b->data_type() == kFloat16) return HalfBitsToFloat(*reinterpret_cast<const uint16_t*>(b->host_copy.data()));
    return *reinterpret_cast<const float*>(b->host_copy.data());
  }
  int act_, engine_;
  bool softmax_;
  PackedWeight pw0_, pw1_;
  std::unique_ptr<Blob> operands_;
  bool has_operands_ = false;
  Derived f_[9];
};
REGISTER_CUDA_OPERATOR(DinAttention, DinAttentionOp);
OPERATOR_SCHEMA(DinAttention).NumInputs(8, 15).NumOutputs(1);

// DinTowerInput: inputs user [R, du], q [R*n, d], k [R, T, d], att [R*n, d] -> X [R*n, ld] with
// ld = roundup(du + 5d, 8) (argument "ld" overrides).
class DinTowerInputOp final : public Operator<CUDAContext> {
 public:
  DinTowerInputOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    ld_ = GetSingleArgument<int>("ld", 0);
  }
  bool RunOnDevice() override {
    Blob *u = Input(0), *q = Input(1), *k = Input(2), *att = Input(3), *x = Output(0);
    if (OutputSize() == 2) return RunSplit(u, q, k, att);
    for (int i = 0; i < 4; ++i) BLAZE_CONDITION_THROW(Input(i)->data_type() == kFloat16, "DinTowerInput needs fp16 inputs");
    BLAZE_CONDITION_THROW(k->shape().size() == 3 && u->shape().size() == 2, "DinTowerInput: k [R,T,d], user [R,du]");
    const int R = (int)k->shape()[0], T = (int)k->shape()[1], d = (int)k->shape()[2], du = (int)u->shape()[1];
    const int n_cand = (int)(q->size() / ((size_t)R * d));
    const int ld = ld_ ? ld_ : (du + 5 * d + 7) / 8 * 8;
    x->set_data_type(kFloat16);
    x->Reshape({(TIndex)R * n_cand, (TIndex)ld});
    XB_CHECK(xb_din_tower_input(u->as<void>(), du, q->as<void>(), d, k->as<void>(), d, att->as<void>(), d, x->as<void>(), ld,
                                R, n_cand, T, d, du, context_.cuda_stream()));
    ++launches;
    return true;
  }
  // two outputs: [user | his_sum] per request and [q | q*his_sum | att | q-his_sum] per candidate, the two
  // operands of a PrunedGemm
  bool RunSplit(Blob* u, Blob* q, Blob* k, Blob* att) {
    for (int i = 0; i < 4; ++i) BLAZE_CONDITION_THROW(Input(i)->data_type() == kFloat16, "DinTowerInput needs fp16 inputs");
    BLAZE_CONDITION_THROW(k->shape().size() == 3 && u->shape().size() == 2, "DinTowerInput: k [R,T,d], user [R,du]");
    const int R = (int)k->shape()[0], T = (int)k->shape()[1], d = (int)k->shape()[2], du = (int)u->shape()[1];
    const int n_cand = (int)(q->size() / ((size_t)R * d));
    const int ldu = (du + d + 7) / 8 * 8, ldc = (4 * d + 7) / 8 * 8;
    Blob *xu = Output(0), *xc = Output(1);
    xu->set_data_type(kFloat16);
    xu->Reshape({(TIndex)R, (TIndex)ldu});
    xc->set_data_type(kFloat16);
    xc->Reshape({(TIndex)R * n_cand, (TIndex)ldc});
    XB_CHECK(xb_din_tower_input_split(u->as<void>(), du, q->as<void>(), d, k->as<void>(), d, att->as<void>(), d,
                                      xu->as<void>(), ldu, xc->as<void>(), ldc, R, n_cand, T, d, du,
                                      context_.cuda_stream()));
    ++launches;
    return true;
  }
  int ld_;
};
// DinTower: the whole tower of the DIN-style model as one operator - feature assembly, Gemm + Dice twice,
// the output Gemm and Softmax - computed by the fused tcgen05 tower kernel.
// Inputs: uid_emb [R, du], ad_emb [R*n, d], his_emb [R, T, d], att [R*n, d], then the constants
// W1 [du+5d, n1], b1, gamma1, mean1, var1, W2 [n1, n2], b2, gamma2, mean2, var2, W3 [n2, n3], b3.
class DinTowerOp final : public Operator<CUDAContext> {
 public:
  DinTowerOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    softmax_ = GetSingleArgument<bool>("softmax", true);
  }
  bool RunOnDevice() override {
    Blob *u = Input(0), *q = Input(1), *k = Input(2), *att = Input(3), *y = Output(0);
    for (int i = 0; i < 4; ++i) BLAZE_CONDITION_THROW(Input(i)->data_type() == kFloat16, "DinTower needs fp16 inputs");
    BLAZE_CONDITION_THROW(k->shape().size() == 3 && u->shape().size() == 2, "DinTower: his_emb [R,T,d], uid_emb [R,du]");
    const int R = (int)k->shape()[0], T = (int)k->shape()[1], d = (int)k->shape()[2], du = (int)u->shape()[1];
    const int n_cand = (int)(q->size() / ((size_t)R * d));
    Blob *W1 = Input(4), *W2 = Input(9), *W3 = Input(14);
    for (Blob* w : {W1, W2, W3})
      BLAZE_CONDITION_THROW(w->shape().size() == 2 && w->data_type() == kFloat16 && w->is_constant,
                            "DinTower: weights must be fp16 rank-2 constants");
    const int n1 = (int)W1->shape()[1], n2 = (int)W2->shape()[1], n3 = (int)W3->shape()[1];
    BLAZE_CONDITION_THROW(W1->shape()[0] == (TIndex)(du + 5 * d) && W2->shape()[0] == (TIndex)n1 && W3->shape()[0] == (TIndex)n2,
                          "DinTower: weight shapes do not chain: ", W1->shape()[0], "x", n1, ", ", W2->shape()[0], "x", n2,
                          ", ", W3->shape()[0], "x", n3);
    cudaStream_t s = context_.cuda_stream();
    xb_din_tower_args a;
    memset(&a, 0, sizeof(a));
    a.d = d; a.du = du; a.n1 = n1; a.n2 = n2; a.n3 = n3; a.softmax = softmax_;
    a.W1 = W1->as<void>(); a.W2 = W2->as<void>(); a.W3 = W3->as<void>();
    a.b1 = AsF32(Input(5), &f_[0], s, &launches);
    a.gamma1 = AsF32(Input(6), &f_[1], s, &launches); a.mean1 = AsF32(Input(7), &f_[2], s, &launches);
    a.var1 = AsF32(Input(8), &f_[3], s, &launches);
    a.b2 = AsF32(Input(10), &f_[4], s, &launches);
    a.gamma2 = AsF32(Input(11), &f_[5], s, &launches); a.mean2 = AsF32(Input(12), &f_[6], s, &launches);
    a.var2 = AsF32(Input(13), &f_[7], s, &launches);
    a.b3 = AsF32(Input(15), &f_[8], s, &launches);
    if (!image_) {
      const size_t n = xb_din_tower_packed_bytes(d, n1, n2, n3);
      BLAZE_CONDITION_THROW(n != 0, "DinTower: d=", d, " n1=", n1, " n2=", n2, " n3=", n3, " is outside the fused tower kernel");
      image_.reset(new Blob(device_option_));
      image_->set_data_type(kFloat);
      image_->Reshape({(TIndex)((n + 3) / 4)});
      XB_CHECK(xb_din_tower_pack(&a, image_->as<void>(), n, s));
      ++launches;
    }
    a.packed = image_->as<void>();
    const size_t wbytes = xb_din_tower_workspace_bytes(R, d, n1);
    if (!scratch_) scratch_.reset(new Blob(device_option_));
    scratch_->set_data_type(kFloat);
    scratch_->Reshape({(TIndex)((wbytes + 3) / 4)});
    y->set_data_type(kFloat);
    y->Reshape({(TIndex)R * n_cand, (TIndex)n3});
    a.user = u->as<void>(); a.ldu = du; a.q = q->as<void>(); a.ldq = d; a.k = k->as<void>(); a.ldk = d;
    a.att = att->as<void>(); a.ldatt = d; a.prob = y->as<float>();
    a.requests = R; a.n_cand = n_cand; a.T = T;
    XB_CHECK(xb_din_tower(&a, scratch_->as<void>(), wbytes, s));
    launches += 2;
    return true;
  }

 private:
  bool softmax_;
  Derived f_[9];
  std::unique_ptr<Blob> image_, scratch_;
};
REGISTER_CUDA_OPERATOR(DinTower, DinTowerOp);
OPERATOR_SCHEMA(DinTower).NumInputs(16).NumOutputs(1);

REGISTER_CUDA_OPERATOR(DinTowerInput, DinTowerInputOp);
OPERATOR_SCHEMA(DinTowerInput).NumInputs(4).NumOutputs(1, 2);

}  // namespace
}  // namespace blaze
