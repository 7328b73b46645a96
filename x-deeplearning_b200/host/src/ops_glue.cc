// CUDA operators of the glue around the dense path: Embedding, Reshape, Concat,
// Slice, Split, FusedSliceConcat, Fuse, ReduceSum, the broadcasting elementwise
// family and the FusedParallelMul pair. Shapes follow the reference operators;
// data movement is expressed with xb_copy2d / xb_elementwise / xb_reduce_sum.
#include <algorithm>
#include <cstring>

#include "runtime.h"

namespace blaze {
namespace {

size_t Prod(const std::vector<TIndex>& s, size_t from, size_t to) {
  size_t n = 1;
  for (size_t i = from; i < to; ++i) n *= s[i];
  return n;
}

// numpy broadcasting of up to 4 dims: right-aligned shapes, element strides (0 where broadcast)
bool BroadcastShape(const std::vector<TIndex>& a, const std::vector<TIndex>& b, std::vector<TIndex>* out) {
  const size_t r = std::max(a.size(), b.size());
  out->assign(r, 1);
  for (size_t i = 0; i < r; ++i) {
    const TIndex da = i < r - a.size() ? 1 : a[i - (r - a.size())];
    const TIndex db = i < r - b.size() ? 1 : b[i - (r - b.size())];
    if (da != db && da != 1 && db != 1) return false;
    (*out)[i] = std::max(da, db);
  }
  return true;
}
void Strides4(const std::vector<TIndex>& shape, const std::vector<TIndex>& out, int64_t (&st)[4], int64_t (&osh)[4]) {
  BLAZE_CONDITION_THROW(out.size() <= 4, "elementwise operators support at most 4 dims, got ", out.size());
  const size_t r = out.size();
  std::vector<TIndex> s(r, 1);
  for (size_t i = 0; i < shape.size(); ++i) s[r - shape.size() + i] = shape[i];
  int64_t run = 1;
  int64_t tmp[4] = {0, 0, 0, 0};
  for (int i = (int)r - 1; i >= 0; --i) {
    tmp[i] = s[i] == 1 && out[i] != 1 ? 0 : run;
    if (s[i] == 1) tmp[i] = 0;
    run *= (int64_t)s[i];
  }
  for (int i = 0; i < 4; ++i) { st[i] = 0; osh[i] = 1; }
  for (size_t i = 0; i < r; ++i) { st[4 - r + i] = tmp[i]; osh[4 - r + i] = (int64_t)out[i]; }
}

// ---- Reshape ---------------------------------------------------------------------------------
class ReshapeOp final : public Operator<CUDAContext> {
 public:
  using Operator<CUDAContext>::Operator;
  bool RunOnDevice() override {
    Blob *x = Input(0), *y = Output(0);
    std::vector<int64_t> rshape = GetRepeatedArgument<int64_t>("shape");
    if (rshape.empty()) {
      BLAZE_CONDITION_THROW(InputSize() == 2, "Reshape needs a shape input or argument");
      Blob* sb = Input(1);
      BLAZE_CONDITION_THROW(sb->is_constant && !sb->host_copy.empty(), "Reshape: the shape operand must be a constant");
      for (size_t i = 0; i < sb->size(); ++i)
        rshape.push_back(sb->data_type() == kInt64 ? reinterpret_cast<const int64_t*>(sb->host_copy.data())[i]
                                                    : reinterpret_cast<const int32_t*>(sb->host_copy.data())[i]);
    }
    const auto& shape = x->shape();
    std::vector<TIndex> ns(rshape.size());
    int unknown = -1;
    size_t known = 1;
    for (size_t i = 0; i < rshape.size(); ++i) {
      if (rshape[i] == 0) { BLAZE_CONDITION_THROW(i < shape.size(), "Reshape: 0 beyond the input rank"); ns[i] = shape[i]; known *= ns[i]; }
      else if (rshape[i] < 0) { BLAZE_CONDITION_THROW(unknown == -1, "can not support two unknown dims"); unknown = (int)i; }
      else { ns[i] = (TIndex)rshape[i]; known *= ns[i]; }
    }
    if (unknown >= 0) ns[unknown] = known ? x->size() / known : 0;
    else BLAZE_CONDITION_THROW(known == x->size(), "known_size=", known, " x->size()=", x->size());
    y->RefReshape(x, ns);
    return true;
  }
};
REGISTER_CUDA_OPERATOR(Reshape, ReshapeOp);
OPERATOR_SCHEMA(Reshape).NumInputs(1, 2).NumOutputs(1);

// ---- Concat / Slice / Split / FusedSliceConcat / Fuse -----------------------------------------
class ConcatOp final : public Operator<CUDAContext> {
 public:
  ConcatOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) { axis_ = GetSingleArgument<size_t>("axis", 1); }
  bool RunOnDevice() override {
    Blob* y = Output(0);
    const auto& s0 = Input(0)->shape();
    BLAZE_CONDITION_THROW(axis_ < s0.size(), "Concat axis ", axis_, " for rank ", s0.size());
    std::vector<TIndex> ys = s0;
    TIndex total = 0;
    for (size_t i = 0; i < InputSize(); ++i) {
      const auto& s = Input(i)->shape();
      BLAZE_CONDITION_THROW(s.size() == s0.size(), "Concat: rank mismatch");
      for (size_t d = 0; d < s.size(); ++d) BLAZE_CONDITION_THROW(d == axis_ || s[d] == s0[d], "Concat: dim ", d, " mismatch");
      BLAZE_CONDITION_THROW(Input(i)->data_type() == Input(0)->data_type(), "Concat: dtype mismatch");
      total += s[axis_];
    }
    ys[axis_] = total;
    y->set_data_type(Input(0)->data_type());
    y->Reshape(ys);
    const size_t outer = Prod(s0, 0, axis_), inner = Prod(s0, axis_ + 1, s0.size());
    const size_t es = DataTypeSize(y->data_type());
    size_t off = 0;
    for (size_t i = 0; i < InputSize(); ++i) {
      const size_t cols = Input(i)->shape()[axis_] * inner;
      XB_CHECK(xb_copy2d(Input(i)->as<void>(), (int64_t)cols, y->data_type(), y->as<char>() + off * es, (int64_t)(total * inner),
                         y->data_type(), (int64_t)outer, (int64_t)cols, context_.cuda_stream()));
      ++launches;
      off += cols;
    }
    return true;
  }
  size_t axis_;
};
REGISTER_CUDA_OPERATOR(Concat, ConcatOp);
OPERATOR_SCHEMA(Concat).NumInputs(1, 128).NumOutputs(1);

void SliceCopy(Blob* x, size_t axis, size_t start, size_t end, void* dst, cudaStream_t s) {
  const auto& sh = x->shape();
  const size_t outer = Prod(sh, 0, axis), inner = Prod(sh, axis + 1, sh.size());
  const size_t es = DataTypeSize(x->data_type());
  XB_CHECK(xb_copy2d(x->as<char>() + start * inner * es, (int64_t)(sh[axis] * inner), x->data_type(), dst,
                     (int64_t)((end - start) * inner), x->data_type(), (int64_t)outer, (int64_t)((end - start) * inner), s));
}

class SliceOp final : public Operator<CUDAContext> {
 public:
  SliceOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    axis_ = GetSingleArgument<size_t>("axis", 1);
    start_ = GetSingleArgument<size_t>("start", 0);
    end_ = GetSingleArgument<size_t>("end", 0);
  }
  bool RunOnDevice() override {
    Blob *x = Input(0), *y = Output(0);
    BLAZE_CONDITION_THROW(axis_ < x->shape().size() && start_ < end_ && end_ <= x->shape()[axis_], "Slice [", start_, ",", end_,
                          ") on axis ", axis_, " of extent ", axis_ < x->shape().size() ? x->shape()[axis_] : 0);
    std::vector<TIndex> ys = x->shape();
    ys[axis_] = end_ - start_;
    y->set_data_type(x->data_type());
    y->Reshape(ys);
    SliceCopy(x, axis_, start_, end_, y->as<void>(), context_.cuda_stream());
    ++launches;
    return true;
  }
  size_t axis_, start_, end_;
};
REGISTER_CUDA_OPERATOR(Slice, SliceOp);
OPERATOR_SCHEMA(Slice).NumInputs(1).NumOutputs(1);

class SplitOp final : public Operator<CUDAContext> {
 public:
  SplitOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    axis_ = GetSingleArgument<size_t>("axis", 0);
    split_ = GetRepeatedArgument<int64_t>("split");
  }
  bool RunOnDevice() override {
    Blob* x = Input(0);
    BLAZE_CONDITION_THROW(axis_ < x->shape().size(), "Split axis ", axis_);
    std::vector<int64_t> sizes = split_;
    if (sizes.empty()) {
      BLAZE_CONDITION_THROW(x->shape()[axis_] % OutputSize() == 0, "Split: extent ", x->shape()[axis_], " not divisible by ", OutputSize());
      sizes.assign(OutputSize(), (int64_t)(x->shape()[axis_] / OutputSize()));
    }
    BLAZE_CONDITION_THROW(sizes.size() == OutputSize(), "Split: ", sizes.size(), " sizes for ", OutputSize(), " outputs");
    size_t off = 0;
    for (size_t i = 0; i < OutputSize(); ++i) {
      std::vector<TIndex> ys = x->shape();
      ys[axis_] = (TIndex)sizes[i];
      Output(i)->set_data_type(x->data_type());
      Output(i)->Reshape(ys);
      SliceCopy(x, axis_, off, off + sizes[i], Output(i)->as<void>(), context_.cuda_stream());
      ++launches;
      off += sizes[i];
    }
    BLAZE_CONDITION_THROW(off == x->shape()[axis_], "Split sizes sum to ", off, ", extent is ", x->shape()[axis_]);
    return true;
  }
  size_t axis_;
  std::vector<int64_t> split_;
};
REGISTER_CUDA_OPERATOR(Split, SplitOp);
OPERATOR_SCHEMA(Split).NumInputs(1).NumOutputs(1, 128);

class FusedSliceConcatOp final : public Operator<CUDAContext> {
 public:
  FusedSliceConcatOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws), tmp_(device_option_) {
    slice_axis_ = GetSingleArgument<size_t>("slice_axis", 1);
    concat_axis_ = GetSingleArgument<size_t>("concat_axis", 1);
    start_ = GetRepeatedArgument<int64_t>("start");
    end_ = GetRepeatedArgument<int64_t>("end");
    BLAZE_CONDITION_THROW(start_.size() == end_.size() && !start_.empty(), "FusedSliceConcat: start/end sizes differ");
  }
  bool RunOnDevice() override {
    Blob *x = Input(0), *y = Output(0);
    const auto& sh = x->shape();
    BLAZE_CONDITION_THROW(slice_axis_ < sh.size() && concat_axis_ < sh.size(), "FusedSliceConcat: axis out of range");
    const size_t len = (size_t)(end_[0] - start_[0]);
    for (size_t i = 0; i < start_.size(); ++i)
      BLAZE_CONDITION_THROW((size_t)(end_[i] - start_[i]) == len && end_[i] <= (int64_t)sh[slice_axis_], "FusedSliceConcat: slices differ in length");
    std::vector<TIndex> piece = sh;
    piece[slice_axis_] = len;
    std::vector<TIndex> ys = piece;
    ys[concat_axis_] = piece[concat_axis_] * start_.size();
    y->set_data_type(x->data_type());
    y->Reshape(ys);
    tmp_.set_data_type(x->data_type());
    tmp_.Reshape(piece);
    const size_t es = DataTypeSize(x->data_type());
    const size_t outer = Prod(piece, 0, concat_axis_), cols = piece[concat_axis_] * Prod(piece, concat_axis_ + 1, piece.size());
    for (size_t i = 0; i < start_.size(); ++i) {
      // slice i as a dense tensor, then placed at its column range of the concatenation
      SliceCopy(x, slice_axis_, start_[i], end_[i], tmp_.as<void>(), context_.cuda_stream());
      XB_CHECK(xb_copy2d(tmp_.as<void>(), (int64_t)cols, x->data_type(), y->as<char>() + i * cols * es,
                         (int64_t)(cols * start_.size()), x->data_type(), (int64_t)outer, (int64_t)cols, context_.cuda_stream()));
      launches += 2;
    }
    return true;
  }
  size_t slice_axis_, concat_axis_;
  std::vector<int64_t> start_, end_;
  Blob tmp_;
};
REGISTER_CUDA_OPERATOR(FusedSliceConcat, FusedSliceConcatOp);
OPERATOR_SCHEMA(FusedSliceConcat).NumInputs(1).NumOutputs(1);

class FuseOp final : public Operator<CUDAContext> {
 public:
  FuseOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    comm_index_ = GetSingleArgument<int>("comm_index", 0);
    BLAZE_CONDITION_THROW(comm_index_ >= 0 && comm_index_ <= 1, "comm_index_=", comm_index_);
  }
  bool RunOnDevice() override {
    Blob *x1 = Input(0), *x2 = Input(1), *y = Output(0);
    BLAZE_CONDITION_THROW(x1->shape().size() == 2 && x2->shape().size() == 2, "Fuse needs 2-D inputs");
    BLAZE_CONDITION_THROW(Input(comm_index_)->shape()[0] == 1, "the common input must have one row");
    BLAZE_CONDITION_THROW(x1->data_type() == x2->data_type(), "Fuse: dtype mismatch");
    const TIndex m1 = x1->shape()[0], n1 = x1->shape()[1], m2 = x2->shape()[0], n2 = x2->shape()[1];
    const TIndex ym = std::max(m1, m2);
    y->set_data_type(x1->data_type());
    y->Reshape({ym, n1 + n2});
    const size_t es = DataTypeSize(y->data_type());
    XB_CHECK(xb_copy2d(x1->as<void>(), m1 == 1 ? 0 : (int64_t)n1, y->data_type(), y->as<void>(), (int64_t)(n1 + n2),
                       y->data_type(), (int64_t)ym, (int64_t)n1, context_.cuda_stream()));
    XB_CHECK(xb_copy2d(x2->as<void>(), m2 == 1 ? 0 : (int64_t)n2, y->data_type(), y->as<char>() + n1 * es, (int64_t)(n1 + n2),
                       y->data_type(), (int64_t)ym, (int64_t)n2, context_.cuda_stream()));
    launches += 2;
    return true;
  }
  int comm_index_;
};
REGISTER_CUDA_OPERATOR(Fuse, FuseOp);
OPERATOR_SCHEMA(Fuse).NumInputs(2).NumOutputs(1);

// ---- ReduceSum ----------------------------------------------------------------------------------
class ReduceSumOp final : public Operator<CUDAContext> {
 public:
  ReduceSumOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    axis_ = GetSingleArgument<size_t>("axis", 0);
    keepdims_ = GetSingleArgument<bool>("keepdims", true);
  }
  bool RunOnDevice() override {
    Blob *x = Input(0), *y = Output(0);
    const auto& sh = x->shape();
    BLAZE_CONDITION_THROW(axis_ < sh.size(), "ReduceSum axis ", axis_, " for rank ", sh.size());
    std::vector<TIndex> ys;
    for (size_t i = 0; i < sh.size(); ++i) {
      if (i != axis_) ys.push_back(sh[i]);
      else if (keepdims_) ys.push_back(1);
    }
    y->set_data_type(x->data_type());
    y->Reshape(ys);
    XB_CHECK(xb_reduce_sum(x->as<void>(), y->as<void>(), (int64_t)Prod(sh, 0, axis_), (int64_t)sh[axis_],
                           (int64_t)Prod(sh, axis_ + 1, sh.size()), x->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
  size_t axis_;
  bool keepdims_;
};
REGISTER_CUDA_OPERATOR(ReduceSum, ReduceSumOp);
OPERATOR_SCHEMA(ReduceSum).NumInputs(1).NumOutputs(1);

// ---- elementwise ------------------------------------------------------------------------------
template <int OP>
class ElementwiseOp final : public Operator<CUDAContext> {
 public:
  using Operator<CUDAContext>::Operator;
  bool RunOnDevice() override {
    Blob *a = Input(0), *b = Input(1), *y = Output(0);
    std::vector<TIndex> ys;
    BLAZE_CONDITION_THROW(BroadcastShape(a->shape(), b->shape(), &ys), "can not broadcast", def_.DebugString());
    BLAZE_CONDITION_THROW(a->data_type() == b->data_type(), "elementwise: dtype mismatch");
    y->set_data_type(a->data_type());
    y->Reshape(ys);
    int64_t as[4], bs[4], osh[4];
    Strides4(a->shape(), ys, as, osh);
    Strides4(b->shape(), ys, bs, osh);
    XB_CHECK(xb_elementwise(OP, a->as<void>(), as, b->as<void>(), bs, nullptr, nullptr, y->as<void>(), osh, a->data_type(),
                            context_.cuda_stream()));
    ++launches;
    return true;
  }
};
typedef ElementwiseOp<XB_EW_ADD> AddOp;
typedef ElementwiseOp<XB_EW_SUB> SubOp;
typedef ElementwiseOp<XB_EW_MUL> MulOp;
typedef ElementwiseOp<XB_EW_DIV> DivOp;
typedef ElementwiseOp<XB_EW_MAX> MaxOp;
typedef ElementwiseOp<XB_EW_MIN> MinOp;
typedef ElementwiseOp<XB_EW_EQ> EqualOp;
typedef ElementwiseOp<XB_EW_NE> NotEqualOp;
REGISTER_CUDA_OPERATOR(Add, AddOp);
REGISTER_CUDA_OPERATOR(Sub, SubOp);
REGISTER_CUDA_OPERATOR(Mul, MulOp);
REGISTER_CUDA_OPERATOR(Div, DivOp);
REGISTER_CUDA_OPERATOR(Max, MaxOp);
REGISTER_CUDA_OPERATOR(Min, MinOp);
REGISTER_CUDA_OPERATOR(Equal, EqualOp);
REGISTER_CUDA_OPERATOR(NotEqual, NotEqualOp);
OPERATOR_SCHEMA(Add).NumInputs(2).NumOutputs(1);
OPERATOR_SCHEMA(Sub).NumInputs(2).NumOutputs(1);
OPERATOR_SCHEMA(Mul).NumInputs(2).NumOutputs(1);
OPERATOR_SCHEMA(Div).NumInputs(2).NumOutputs(1);
OPERATOR_SCHEMA(Max).NumInputs(2).NumOutputs(1);
OPERATOR_SCHEMA(Min).NumInputs(2).NumOutputs(1);
OPERATOR_SCHEMA(Equal).NumInputs(2).NumOutputs(1);
OPERATOR_SCHEMA(NotEqual).NumInputs(2).NumOutputs(1);

class BroadcastToOp final : public Operator<CUDAContext> {
 public:
  using Operator<CUDAContext>::Operator;
  bool RunOnDevice() override {
    Blob *a = Input(0), *like = Input(1), *y = Output(0);
    std::vector<TIndex> ys;
    BLAZE_CONDITION_THROW(BroadcastShape(a->shape(), like->shape(), &ys) && ys == like->shape(), "can not broadcast to the target shape");
    y->set_data_type(a->data_type());
    y->Reshape(ys);
    int64_t as[4], osh[4];
    Strides4(a->shape(), ys, as, osh);
    XB_CHECK(xb_elementwise(XB_EW_BROADCAST_TO, a->as<void>(), as, nullptr, nullptr, nullptr, nullptr, y->as<void>(), osh,
                            a->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
};
REGISTER_CUDA_OPERATOR(BroadcastTo, BroadcastToOp);
OPERATOR_SCHEMA(BroadcastTo).NumInputs(2).NumOutputs(1);

class WhereOp final : public Operator<CUDAContext> {
 public:
  using Operator<CUDAContext>::Operator;
  bool RunOnDevice() override {
    Blob *c = Input(0), *a = Input(1), *b = Input(2), *y = Output(0);
    BLAZE_CONDITION_THROW(c->data_type() == kInt32, "Where: the condition must be int32");
    std::vector<TIndex> t, ys;
    BLAZE_CONDITION_THROW(BroadcastShape(a->shape(), b->shape(), &t) && BroadcastShape(t, c->shape(), &ys), "can not broadcast");
    y->set_data_type(a->data_type());
    y->Reshape(ys);
    int64_t cs[4], as[4], bs[4], osh[4];
    Strides4(c->shape(), ys, cs, osh);
    Strides4(a->shape(), ys, as, osh);
    Strides4(b->shape(), ys, bs, osh);
    XB_CHECK(xb_elementwise(XB_EW_WHERE, c->as<void>(), cs, a->as<void>(), as, b->as<void>(), bs, y->as<void>(), osh,
                            a->data_type(), context_.cuda_stream()));
    ++launches;
    return true;
  }
};
REGISTER_CUDA_OPERATOR(Where, WhereOp);
OPERATOR_SCHEMA(Where).NumInputs(3).NumOutputs(1);

// ---- FusedParallelMul / FusedParallelMulReduceSum --------------------------------------------------
class FusedParallelMulOp : public Operator<CUDAContext> {
 public:
  FusedParallelMulOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    parallel_num_ = GetSingleArgument<int>("parallel_num", 2);
  }
  bool RunOnDevice() override { return Multiply(Output(0)); }

 protected:
  bool Multiply(Blob* c) {
    Blob *a = Input(0), *b = Input(1);
    const int P = parallel_num_;
    BLAZE_CONDITION_THROW(a->shape().size() >= 2 && b->shape().size() >= 2, "FusedParallelMul needs rank >= 2");
    std::vector<TIndex> as = a->shape(), bs = b->shape();
    BLAZE_CONDITION_THROW(as[0] % P == 0 && bs[0] % P == 0, "leading dims must be multiples of parallel_num");
    as[0] /= P; bs[0] /= P;
    BLAZE_CONDITION_THROW(BroadcastShape(as, bs, &branch_), "can not broadcast for Mul");
    std::vector<TIndex> cs = branch_;
    cs[0] *= P;
    c->set_data_type(a->data_type());
    c->Reshape(cs);
    int64_t ast[4], bst[4], osh[4];
    Strides4(as, branch_, ast, osh);
    Strides4(bs, branch_, bst, osh);
    const size_t es = DataTypeSize(a->data_type());
    const size_t la = Prod(as, 0, as.size()), lb = Prod(bs, 0, bs.size()), lc = Prod(branch_, 0, branch_.size());
    for (int p = 0; p < P; ++p) {
      XB_CHECK(xb_elementwise(XB_EW_MUL, a->as<char>() + p * la * es, ast, b->as<char>() + p * lb * es, bst, nullptr, nullptr,
                              c->as<char>() + p * lc * es, osh, a->data_type(), context_.cuda_stream()));
      ++launches;
    }
    return true;
  }
  int parallel_num_;
  std::vector<TIndex> branch_;
};
REGISTER_CUDA_OPERATOR(FusedParallelMul, FusedParallelMulOp);
OPERATOR_SCHEMA(FusedParallelMul).NumInputs(2).NumOutputs(1);

class FusedParallelMulReduceSumOp final : public FusedParallelMulOp {
 public:
  FusedParallelMulReduceSumOp(const OperatorDef& def, Workspace* ws) : FusedParallelMulOp(def, ws), tmp_(device_option_) {
    axis_ = GetSingleArgument<size_t>("axis", 0);
    keepdims_ = GetSingleArgument<bool>("keepdims", true);
  }
  bool RunOnDevice() override {
    if (!Multiply(&tmp_)) return false;
    Blob* y = Output(0);
    const int P = parallel_num_;
    BLAZE_CONDITION_THROW(axis_ < branch_.size(), "axis ", axis_, " for rank ", branch_.size());
    std::vector<TIndex> red;
    for (size_t i = 0; i < branch_.size(); ++i) {
      if (i != axis_) red.push_back(branch_[i]);
      else if (keepdims_) red.push_back(1);
    }
    if (red.empty()) red.push_back(1);
    std::vector<TIndex> ys = red;
    ys[0] *= P;
    y->set_data_type(tmp_.data_type());
    y->Reshape(ys);
    const size_t es = DataTypeSize(tmp_.data_type());
    const size_t lc = Prod(branch_, 0, branch_.size()), lr = Prod(red, 0, red.size());
    for (int p = 0; p < P; ++p) {
      XB_CHECK(xb_reduce_sum(tmp_.as<char>() + p * lc * es, y->as<char>() + p * lr * es, (int64_t)Prod(branch_, 0, axis_),
                             (int64_t)branch_[axis_], (int64_t)Prod(branch_, axis_ + 1, branch_.size()), tmp_.data_type(),
                             context_.cuda_stream()));
      ++launches;
    }
    return true;
  }
  size_t axis_;
  bool keepdims_;
  Blob tmp_;
};
REGISTER_CUDA_OPERATOR(FusedParallelMulReduceSum, FusedParallelMulReduceSumOp);
OPERATOR_SCHEMA(FusedParallelMulReduceSum).NumInputs(2).NumOutputs(1);

// ---- Embedding ------------------------------------------------------------------------------------
// CUDA registration of the operator the reference ships for CPU only
// (blaze/blaze/operator/sparse_op/embedding/embedding_op.cc:87). Inputs are triples
// <feature_group>.ids / .values / .segments; outputs one blob per block_config.
class EmbeddingOp final : public Operator<CUDAContext> {
 public:
  EmbeddingOp(const OperatorDef& def, Workspace* ws) : Operator<CUDAContext>(def, ws) {
    puller_ = ws->GetSparsePuller();
    BLAZE_CONDITION_THROW(puller_ != nullptr, "sparse puller is not set: call LoadSparseModelWeight first");
    const std::string conf = GetSingleArgument<std::string>("embedding_config", "");
    TextNode root;
    std::string err;
    BLAZE_CONDITION_THROW(ParseTextProto(conf, &root, &err), "parse embedding config failed: ", err);
    for (const TextNode* n : root.Children("feature_group_config")) {
      FeatureGroup fg;
      BLAZE_CONDITION_THROW(n->Get("feature_group", &fg.name) && n->Get("table_name", &fg.table), "feature_group_config needs feature_group and table_name");
      fg.dim = (int)n->GetInt("dim", 18);
      fg_index_[fg.name] = groups_.size();
      groups_.push_back(fg);
    }
    // input name -> feature group ("<fg>.ids" at 3p, ".values" at 3p+1, ".segments" at 3p+2)
    BLAZE_CONDITION_THROW(def.input.size() % 3 == 0, "embedding op input size=", def.input.size());
    for (size_t i = 0; i < def.input.size(); i += 3) {
      const std::string& n = def.input[i];
      const size_t dot = n.rfind('.');
      BLAZE_CONDITION_THROW(dot != std::string::npos, "input ", n, " is not <feature_group>.ids");
      input_fg_[n.substr(0, dot)] = i / 3;
    }
    const auto blocks = root.Children("block_config");
    BLAZE_CONDITION_THROW(blocks.size() == def.output.size(), "block_config count ", blocks.size(), " != outputs ", def.output.size());
    for (size_t b = 0; b < blocks.size(); ++b) {
      Block blk;
      size_t offset = 0;
      for (const TextNode* it : blocks[b]->Children("embedding_block_config_item")) {
        Item item;
        std::string fg;
        BLAZE_CONDITION_THROW(it->Get("feature_group", &fg), "block item without feature_group");
        auto f = fg_index_.find(fg);
        BLAZE_CONDITION_THROW(f != fg_index_.end(), "feature group config not exist, fg: ", fg);
        item.fg = f->second;
        item.udf = (int)it->GetInt("udf_type", 0);
        std::string td;
        item.trunc_dir = store::kReverse;
        if (it->Get("trunc_direction", &td)) item.trunc_dir = (td == "kInorder" || td == "0") ? store::kOrder : store::kReverse;
        item.trunc_num = (int)it->GetInt("trunc_num", 0);
        item.offset = offset;
        const int dim = groups_[item.fg].dim;
        switch (item.udf) {
          case store::kSum: case store::kAvg: offset += dim; break;
          case store::kAssign: offset += (size_t)dim * item.trunc_num; break;
          default: BLAZE_THROW("Unsupported udf type: ", item.udf);
        }
        groups_[item.fg].uses.emplace_back(b, blk.items.size());
        if (!input_fg_.count(fg)) blk.needs_clear = true;          // nothing will write this item
        blk.items.push_back(item);
      }
      blk.stride = offset;
      blocks_.push_back(blk);
    }
  }

  bool RunOnDevice() override {
    cudaStream_t s = context_.cuda_stream();
    // CheckValid
    for (size_t i = 0; i < InputSize(); i += 3) {
      Blob *ids = Input(i), *vals = Input(i + 1), *seg = Input(i + 2);
      BLAZE_CONDITION_THROW(ids->size() == vals->size(), "id_blob->size()=", ids->size(), " value_blob->size()=", vals->size(), def_.DebugString());
      BLAZE_CONDITION_THROW(ids->data_type() == kInt64 || ids->data_type() == kInt32, "Unsupported key type:", ids->data_type());
      BLAZE_CONDITION_THROW(seg->data_type() == kInt32, "Unsupported num type:", seg->data_type());
      BLAZE_CONDITION_THROW(vals->data_type() == Input(1)->data_type(), "x->data_type()=", Input(1)->data_type(), " y->data_type()=", vals->data_type());
    }
    const int vtype = InputSize() ? Input(1)->data_type() : kFloat;
    BLAZE_CONDITION_THROW(vtype == kFloat || vtype == kFloat16, "Unsupported value type:", vtype);
    // Setup: shape the output blocks
    for (size_t b = 0; b < blocks_.size(); ++b) {
      size_t batch = 0;
      for (const Item& it : blocks_[b].items) {
        auto f = input_fg_.find(groups_[it.fg].name);
        BLAZE_CONDITION_THROW(f != input_fg_.end(), "feature group of block item is not in input list, fg: ", groups_[it.fg].name);
        const size_t n = Input(f->second * 3 + 2)->size();
        BLAZE_CONDITION_THROW(batch == 0 || n == batch, "batch size of each feature group in block must be equal");
        batch = n;
      }
      Blob* out = Output(b);
      out->set_data_type(vtype);
      out->Reshape({(TIndex)batch, (TIndex)blocks_[b].stride});
      if (blocks_[b].needs_clear && out->bytes()) CUDA_CHECK(cudaMemsetAsync(out->as<void>(), 0, out->bytes(), s));
    }
    // RunEmbedding: one puller input/output pair per configured feature group
    std::vector<store::SparsePullerInput> in(groups_.size());
    std::vector<store::SparsePullerOutput> out(groups_.size());
    for (size_t g = 0; g < groups_.size(); ++g) {
      const FeatureGroup& fg = groups_[g];
      in[g].name = fg.table;
      auto f = input_fg_.find(fg.name);
      if (f == input_fg_.end()) continue;
      Blob *ids = Input(f->second * 3), *vals = Input(f->second * 3 + 1), *seg = Input(f->second * 3 + 2);
      in[g].key = ids->as<void>(); in[g].key_size = ids->size();
      in[g].key_num = seg->as<void>(); in[g].key_num_size = seg->size();
      in[g].value = vals->as<void>();
      in[g].key_type = ids->data_type(); in[g].value_type = vtype; in[g].num_type = seg->data_type();
      in[g].dim = fg.dim;
      for (const auto& use : fg.uses) {
        const Item& it = blocks_[use.first].items[use.second];
        store::SparsePullerInput::Param p;
        p.udf_type = (store::UDFType)it.udf; p.trunc_direction = (store::TruncDirection)it.trunc_dir; p.trunc_num = it.trunc_num;
        in[g].in_item.push_back(p);
        store::SparsePullerOutput::OutItem o;
        o.out = Output(use.first)->as<char>() + it.offset * DataTypeSize(vtype);
        o.stride = blocks_[use.first].stride;
        out[g].out_item.push_back(o);
      }
    }
    const store::Status st = puller_->GetAsync(in, out, context_.device_id(), s, &launches);
    BLAZE_CONDITION_THROW(st == store::kOK, "pull data failed, status=", (int)st);
    return true;
  }

 private:
  struct Item { size_t fg; int udf; int trunc_dir; int trunc_num; size_t offset; };
  struct Block { std::vector<Item> items; size_t stride = 0; bool needs_clear = false; };
  struct FeatureGroup { std::string name, table; int dim = 18; std::vector<std::pair<size_t, size_t>> uses; };
  std::shared_ptr<store::SparsePuller> puller_;
  std::vector<FeatureGroup> groups_;
  std::vector<Block> blocks_;
  std::unordered_map<std::string, size_t> fg_index_, input_fg_;
};
REGISTER_CUDA_OPERATOR(Embedding, EmbeddingOp);
OPERATOR_SCHEMA(Embedding).NumInputs(3, 384).NumOutputs(1, 128);

}  // namespace
}  // namespace blaze
