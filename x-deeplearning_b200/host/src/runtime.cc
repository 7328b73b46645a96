// Blob, CUDA context, workspace, operator registries, the sequential net and the
// Gemm+activation fusion pass.
#include "runtime.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <set>

namespace blaze {

void LogError(const std::string& msg) { fprintf(stderr, "[blaze-b200][ERROR] %s\n", msg.c_str()); }

size_t DataTypeSize(int dtype) {
  switch (dtype) {
    case kFloat: case kInt32: return 4;
    case kInt64: case kDouble: return 8;
    case kFloat16: return 2;
    case kBool: return 1;
    default: BLAZE_THROW("unsupported data type ", dtype);
  }
}

uint16_t FloatToHalfBits(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return (uint16_t)(sign | h);
}

float HalfBitsToFloat(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, x;
  if (exp == 0) {
    if (man == 0) x = sign;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) x = sign | 0x7f800000u | (man << 13);
  else x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  float f;
  memcpy(&f, &x, 4);
  return f;
}

// ---- Blob ---------------------------------------------------------------------------------------
Blob::~Blob() {
  if (data_) {
    if (opt_.device_type == kCUDA) cudaFree(data_);
    else free(data_);
  }
}

size_t Blob::size() const {
  size_t n = 1;
  for (auto d : shape_) n *= d;
  return n;
}
size_t Blob::size(size_t from, size_t to) const {
  size_t n = 1;
  for (size_t i = from; i < to && i < shape_.size(); ++i) n *= shape_[i];
  return n;
}

void Blob::Reshape(const std::vector<TIndex>& shape) {
  shape_ = shape;
  ref_ = nullptr;
  const size_t need = size() * DataTypeSize(dtype_);
  if (need <= capacity_) return;
  // grow-only, like the reference Blob; not stream ordered, so sized before a net's first run
  if (data_) {
    if (opt_.device_type == kCUDA) { CUDA_CHECK(cudaDeviceSynchronize()); cudaFree(data_); }
    else free(data_);
    data_ = nullptr;
  }
  const size_t cap = std::max<size_t>(need, 256);
  if (opt_.device_type == kCUDA) {
    CUDA_CHECK(cudaSetDevice(opt_.device_id));
    CUDA_CHECK(cudaMalloc(&data_, cap));
  } else {
    data_ = malloc(cap);
    BLAZE_CONDITION_THROW(data_ != nullptr, "host allocation of ", cap, " bytes failed");
  }
  capacity_ = cap;
}

void Blob::RefReshape(Blob* src, const std::vector<TIndex>& shape) {
  shape_ = shape;
  dtype_ = src->dtype_;
  ref_ = src->ref_ ? src->ref_ : src;
}

// ---- context ------------------------------------------------------------------------------------
namespace {
// one non-blocking stream per (thread, device): predictors are per-thread objects in Blaze's model
cudaStream_t ThreadStream(int device) {
  thread_local cudaStream_t streams[64] = {nullptr};
  BLAZE_CONDITION_THROW(device >= 0 && device < 64, "device id ", device, " out of range");
  if (!streams[device]) {
    CUDA_CHECK(cudaSetDevice(device));
    CUDA_CHECK(cudaStreamCreateWithFlags(&streams[device], cudaStreamNonBlocking));
  }
  return streams[device];
}
}  // namespace

CUDAContext::CUDAContext(const DeviceOption& opt) : device_id_(opt.device_id), stream_(nullptr) {
  BLAZE_CONDITION_THROW(opt.device_type == kCUDA, "device_type=", opt.device_type,
                        ": this runtime has CUDA operators only (there is no CPU fallback)");
  stream_ = ThreadStream(device_id_);
}
void CUDAContext::Activate() const { CUDA_CHECK(cudaSetDevice(device_id_)); }
void CUDAContext::FinishDeviceComputation() const { CUDA_CHECK(cudaStreamSynchronize(stream_)); }

// ---- sparse puller registry -----------------------------------------------------------------------
namespace store {
SparsePullerCreationRegisterer* SparsePullerCreationRegisterer::Get() {
  static SparsePullerCreationRegisterer inst;
  return &inst;
}
bool SparsePullerCreationRegisterer::Register(const std::string& name, FCreateSparsePuller fcs) {
  if (fcs_map_.count(name)) BLAZE_THROW("SparsePullerCreation name=", name, " is already registered");
  fcs_map_[name] = fcs;
  return true;
}
SparsePuller* SparsePullerCreationRegisterer::CreateSparsePuller(const std::string& name) {
  auto it = fcs_map_.find(name);
  return it == fcs_map_.end() ? nullptr : it->second();
}
}  // namespace store

// ---- workspace ------------------------------------------------------------------------------------
Blob* Workspace::CreateBlob(const std::string& name, const DeviceOption& opt) {
  if (Blob* b = GetBlob(name)) return b;
  blobs_[name].reset(new Blob(opt));
  return blobs_[name].get();
}

Blob* Workspace::CreateConstantBlob(const std::string& name, const DeviceOption& opt, bool* fresh) {
  *fresh = false;
  auto own = blobs_.find(name);
  if (own != blobs_.end()) return own->second.get();
  auto sh = shared_.find(name);
  if (sh != shared_.end()) return sh->second.get();
  if (!constants_) {
    *fresh = true;
    return CreateBlob(name, opt);
  }
  std::lock_guard<std::mutex> lock(constants_->mu);
  auto it = constants_->blobs.find(name);
  if (it == constants_->blobs.end()) {
    it = constants_->blobs.emplace(name, std::make_shared<Blob>(opt)).first;
    *fresh = true;
  }
  shared_[name] = it->second;
  return it->second.get();
}

Blob* Workspace::GetBlob(const std::string& name) const {
  auto it = blobs_.find(name);
  if (it != blobs_.end()) return it->second.get();
  auto sh = shared_.find(name);
  return sh == shared_.end() ? nullptr : sh->second.get();
}

std::vector<std::string> Workspace::BlobNames() const {
  std::vector<std::string> names;
  for (const auto& kv : blobs_) names.push_back(kv.first);
  for (const auto& kv : shared_) names.push_back(kv.first);
  std::sort(names.begin(), names.end());
  return names;
}

std::unique_ptr<Net> Workspace::CreateNet() {
  const std::string& mode = net_def_.run_mode;
  // "dag" and "hybrid" schedule the same operators over several streams / devices in the
  // reference; here every operator is a CUDA operator, so one in-order stream runs them all.
  BLAZE_CONDITION_THROW(mode == "simple" || mode == "dag" || mode == "hybrid" || mode.empty(), "unknown run_mode ", mode);
  return std::unique_ptr<Net>(new Net(net_def_, this));
}

// ---- operators ------------------------------------------------------------------------------------
OperatorBase::OperatorBase(const OperatorDef& def, Workspace* ws) : def_(def), workspace_(ws) {
  device_option_ = def.has_device_option ? def.device_option : ws->net_def().device_option;
  if (const OpSchema* s = FindSchema(def.type)) {
    BLAZE_CONDITION_THROW((int)def.input.size() >= s->min_in && (int)def.input.size() <= s->max_in, "operator ",
                          def.type, " has ", def.input.size(), " inputs", def.DebugString());
    BLAZE_CONDITION_THROW((int)def.output.size() >= s->min_out && (int)def.output.size() <= s->max_out, "operator ",
                          def.type, " has ", def.output.size(), " outputs", def.DebugString());
  }
  for (const auto& n : def.input) inputs_.push_back(ws->CreateBlob(n, device_option_));
  for (const auto& n : def.output) {
    if (def.type == "ConstantFill") {
      // constants live in the per-device store shared by all predictors of a model
      outputs_.push_back(ws->CreateConstantBlob(n, device_option_, &constant_fresh));
      continue;
    }
    Blob* b = ws->GetBlob(n);
    outputs_.push_back(b ? b : ws->CreateBlob(n, device_option_));
  }
  // type inference default: outputs take the first input's type
  if (!inputs_.empty())
    for (Blob* o : outputs_)
      if (std::find(inputs_.begin(), inputs_.end(), o) == inputs_.end()) o->set_data_type(inputs_[0]->data_type());
}

template <> float OperatorBase::GetSingleArgument<float>(const std::string& name, const float& def) const {
  const Argument* a = def_.FindArg(name);
  if (!a) return def;
  return a->has_f ? a->f : (a->has_i ? (float)a->i : def);
}
template <> int64_t OperatorBase::GetSingleArgument<int64_t>(const std::string& name, const int64_t& def) const {
  const Argument* a = def_.FindArg(name);
  if (!a) return def;
  return a->has_i ? a->i : (a->has_f ? (int64_t)a->f : def);
}
template <> int OperatorBase::GetSingleArgument<int>(const std::string& name, const int& def) const {
  return (int)GetSingleArgument<int64_t>(name, def);
}
template <> size_t OperatorBase::GetSingleArgument<size_t>(const std::string& name, const size_t& def) const {
  return (size_t)GetSingleArgument<int64_t>(name, (int64_t)def);
}
template <> bool OperatorBase::GetSingleArgument<bool>(const std::string& name, const bool& def) const {
  return GetSingleArgument<int64_t>(name, def ? 1 : 0) != 0;
}
template <> std::string OperatorBase::GetSingleArgument<std::string>(const std::string& name, const std::string& def) const {
  const Argument* a = def_.FindArg(name);
  return (a && a->has_s) ? a->s : def;
}
template <> std::vector<int64_t> OperatorBase::GetRepeatedArgument<int64_t>(const std::string& name) const {
  const Argument* a = def_.FindArg(name);
  return a ? a->ints : std::vector<int64_t>();
}
template <> std::vector<float> OperatorBase::GetRepeatedArgument<float>(const std::string& name) const {
  const Argument* a = def_.FindArg(name);
  return a ? a->floats : std::vector<float>();
}

void OperatorRegistry::Register(const std::string& name, OperatorCreator c) {
  if (map_.count(name)) BLAZE_THROW("Key ", name, " already registered");
  map_[name] = c;
}
std::unique_ptr<OperatorBase> OperatorRegistry::Create(const std::string& name, const OperatorDef& def, Workspace* ws) const {
  auto it = map_.find(name);
  if (it == map_.end()) return nullptr;
  return it->second(def, ws);
}
std::vector<std::string> OperatorRegistry::Names() const {
  std::vector<std::string> n;
  for (const auto& kv : map_) n.push_back(kv.first);
  std::sort(n.begin(), n.end());
  return n;
}
OperatorRegistry* CUDAOperatorRegistry() { static OperatorRegistry r; return &r; }
OperatorRegistry* CPUOperatorRegistry() { static OperatorRegistry r; return &r; }

namespace {
std::unordered_map<std::string, OpSchema>& Schemas() {
  static std::unordered_map<std::string, OpSchema> m;
  return m;
}
}  // namespace
OpSchema& RegisterSchema(const std::string& name) {
  if (Schemas().count(name)) BLAZE_THROW("schema ", name, " already registered");
  return Schemas()[name];
}
const OpSchema* FindSchema(const std::string& name) {
  auto it = Schemas().find(name);
  return it == Schemas().end() ? nullptr : &it->second;
}

std::unique_ptr<OperatorBase> CreateOperator(const OperatorDef& def, Workspace* ws) {
  const DeviceOption& opt = def.has_device_option ? def.device_option : ws->net_def().device_option;
  OperatorRegistry* reg = opt.device_type == kCUDA ? CUDAOperatorRegistry() : CPUOperatorRegistry();
  std::unique_ptr<OperatorBase> op = reg->Create(def.type, def, ws);
  BLAZE_CONDITION_THROW(op != nullptr, "operator ", def.type, " is not registered for device_type ", opt.device_type,
                        opt.device_type == kCUDA ? "" : " (this runtime registers CUDA operators only)");
  return op;
}

// ---- net ------------------------------------------------------------------------------------------
Net::Net(const NetDef& def, Workspace* ws) : def_(def), ws_(ws) {
  for (const auto& v : def.external_input) ext_in_.push_back(v.name);
  for (const auto& v : def.external_output) ext_out_.push_back(v.name);
  // typed external inputs exist before the operators that read them are built
  for (const auto& v : def.external_input) ws->CreateBlob(v.name, def.device_option)->set_data_type(v.dtype);
  for (const auto& od : def.op) ops_.push_back(CreateOperator(od, ws));
  CUDA_CHECK(cudaSetDevice(def.device_option.device_id));
  BLAZE_CONDITION_THROW(xb_device_status_mirror(&status_word_) == 0, "device status word: ", xb_last_error());
}

void Net::CheckDeviceStatus() {
  const int st = status_word_ ? *status_word_ : 0;
  if (st == 0) return;
  xb_device_status_clear();
  BLAZE_THROW("a bounded wait ran out inside a tensor-core kernel on device ", device_id(), " (site ", st >> 8,
              "): the results of this run are invalid");
}

cudaStream_t Net::stream() const {
  DeviceOption opt = def_.device_option;
  CUDAContext ctx(opt);
  return ctx.cuda_stream();
}

bool Net::Run() {
  last_launches = 0;
  if (profile) op_ms.clear();
  for (auto& op : ops_) {
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (profile) {
      cudaEventCreate(&e0); cudaEventCreate(&e1);
      cudaEventRecord(e0, stream());
    }
    if (!op->Run()) return false;
    last_launches += op->launches;
    if (profile) {
      cudaEventRecord(e1, stream());
      cudaEventSynchronize(e1);
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      op_ms.emplace_back(op->operator_def().type + ":" + op->operator_def().name, ms);
      cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
  }
  return true;
}

// ---- BatchNormalization folding ---------------------------------------------------------------------
namespace {
// Values of a ConstantFill operator as fp32 (what the operator itself would upload), or false.
bool ConstantValues(const OperatorDef& op, std::vector<float>* out, std::vector<int64_t>* shape, int* dtype) {
  if (op.type != "ConstantFill" || op.output.size() != 1) return false;
  const Argument* v = op.FindArg("value");
  const Argument* sh = op.FindArg("shape");
  const Argument* dt = op.FindArg("dtype");
  if (!v || !sh) return false;
  *dtype = dt && dt->has_i ? (int)dt->i : kFloat;
  if (*dtype != kFloat && *dtype != kFloat16) return false;
  *shape = sh->ints;
  size_t n = 1;
  for (int64_t d : *shape) n *= (size_t)d;
  *out = v->floats;
  if (out->empty() && !v->ints.empty()) out->assign(v->ints.begin(), v->ints.end());
  if (out->empty() && v->has_f) out->assign(1, v->f);
  if (out->size() != n) return false;
  if (*dtype == kFloat16)                                   // the operator rounds to fp16 when it uploads
    for (float& f : *out) f = HalfBitsToFloat(FloatToHalfBits(f));
  return true;
}

OperatorDef MakeConstant(const std::string& name, const std::vector<float>& values, const std::vector<int64_t>& shape, int dtype) {
  OperatorDef op;
  op.type = "ConstantFill";
  op.name = name;
  op.output.push_back(name);
  Argument a;
  a.name = "shape"; a.ints = shape;
  op.arg.push_back(a);
  Argument d;
  d.name = "dtype"; d.has_i = true; d.i = dtype;
  op.arg.push_back(d);
  Argument v;
  v.name = "value"; v.floats = values;
  op.arg.push_back(v);
  return op;
}
}  // namespace

// A BatchNormalization with constant parameters next to a Gemm with a constant weight is an affine map of the
// Gemm's K (BN before) or N (BN after) axis: it folds into the weight and bias, computed here in fp32 from
// the constants' values, and the BN node disappears. The reference DIN graph has this shape (bn_layer feeding
// the first inner_product_layer, blaze/tools/example_model/din/model/graph_ulf.txt).
void FoldBatchNorm(NetDef* def) {
  bool changed = true;
  int serial = 0;
  while (changed) {
    changed = false;
    std::map<std::string, int> consumers, producer;
    for (size_t i = 0; i < def->op.size(); ++i) {
      for (const auto& in : def->op[i].input) ++consumers[in];
      for (const auto& out : def->op[i].output) producer[out] = (int)i;
    }
    std::set<std::string> ext_out;
    for (const auto& v : def->external_output) ext_out.insert(v.name);
    auto constant = [&](const std::string& name, std::vector<float>* v, std::vector<int64_t>* sh, int* dt) {
      auto it = producer.find(name);
      return it != producer.end() && ConstantValues(def->op[it->second], v, sh, dt);
    };
    for (size_t bi = 0; bi < def->op.size() && !changed; ++bi) {
      const OperatorDef bn = def->op[bi];
      if (bn.type != "BatchNormalization" || bn.input.size() != 5 || bn.output.size() != 1) continue;
      std::vector<float> gamma, beta, mean, var;
      std::vector<int64_t> sh;
      int dt = 0;
      if (!constant(bn.input[1], &gamma, &sh, &dt) || !constant(bn.input[2], &beta, &sh, &dt) ||
          !constant(bn.input[3], &mean, &sh, &dt) || !constant(bn.input[4], &var, &sh, &dt)) continue;
      const size_t c = gamma.size();
      if (beta.size() != c || mean.size() != c || var.size() != c) continue;
      const Argument* ns = bn.FindArg("nosqrt");
      const Argument* ep = bn.FindArg("eps");
      const bool nosqrt = ns && (ns->has_i ? ns->i != 0 : ns->f != 0.f);
      const float eps = ep && ep->has_f ? ep->f : 0.001f;
      std::vector<float> scale(c), shift(c);               // y = x * scale + shift
      for (size_t i = 0; i < c; ++i) {
        scale[i] = gamma[i] / (nosqrt ? var[i] : sqrtf(var[i] + eps));
        shift[i] = beta[i] - mean[i] * scale[i];
      }
      // the Gemm on the other side of the BN: its only consumer (BN first) or its producer (Gemm first)
      int gi = -1;
      bool bn_first = false;
      const std::string& x = bn.input[0];
      const std::string& y = bn.output[0];
      if (consumers[y] == 1 && !ext_out.count(y)) {
        for (size_t j = 0; j < def->op.size(); ++j)
          if (def->op[j].type == "Gemm" && !def->op[j].input.empty() && def->op[j].input[0] == y) { gi = (int)j; bn_first = true; }
      }
      if (gi < 0 && consumers[x] == 1 && !ext_out.count(x) && producer.count(x) && def->op[producer[x]].type == "Gemm" &&
          !def->op[producer[x]].FindArg("epilogue"))
        gi = producer[x];
      if (gi < 0) continue;
      OperatorDef& g = def->op[gi];
      if (g.input.size() < 2 || g.input.size() > 3 || g.output.size() != 1) continue;
      auto flag = [&](const char* name) {
        const Argument* a = g.FindArg(name);
        return a && (a->has_i ? a->i != 0 : a->f != 0.f);
      };
      auto scalar = [&](const char* name) {
        const Argument* a = g.FindArg(name);
        return a ? (a->has_f ? a->f : (a->has_i ? (float)a->i : 1.f)) : 1.f;
      };
      if (flag("transA") || scalar("alpha") != 1.f || scalar("beta") != 1.f) continue;
      const bool tb = flag("transB");
      std::vector<float> W, bias;
      std::vector<int64_t> wsh, bsh;
      int wdt = 0, bdt = 0;
      if (!constant(g.input[1], &W, &wsh, &wdt) || wsh.size() != 2) continue;
      const size_t K = (size_t)(tb ? wsh[1] : wsh[0]), N = (size_t)(tb ? wsh[0] : wsh[1]);
      const bool has_bias = g.input.size() == 3;
      if (has_bias && (!constant(g.input[2], &bias, &bsh, &bdt) || bias.size() != N)) continue;
      if (!has_bias) { bias.assign(N, 0.f); bdt = wdt; }
      if (c != (bn_first ? K : N)) continue;
      auto w = [&](size_t k, size_t n) -> float& { return tb ? W[n * K + k] : W[k * N + n]; };
      if (bn_first) {
        // (x * scale + shift) W + b = x (diag(scale) W) + (shift W + b)
        for (size_t n = 0; n < N; ++n) {
          double acc = bias[n];
          for (size_t k = 0; k < K; ++k) acc += (double)shift[k] * w(k, n);
          bias[n] = (float)acc;
        }
        for (size_t k = 0; k < K; ++k)
          for (size_t n = 0; n < N; ++n) w(k, n) *= scale[k];
      } else {
        // (x W + b) * scale + shift = x (W diag(scale)) + (b * scale + shift)
        for (size_t k = 0; k < K; ++k)
          for (size_t n = 0; n < N; ++n) w(k, n) *= scale[n];
        for (size_t n = 0; n < N; ++n) bias[n] = bias[n] * scale[n] + shift[n];
      }
      const std::string tag = "__bn" + std::to_string(serial++);
      OperatorDef cw = MakeConstant(g.input[1] + tag, W, wsh, wdt);
      OperatorDef cb = MakeConstant((has_bias ? g.input[2] : g.output[0] + "_bias") + tag, bias, {(int64_t)N}, bdt);
      g.input.resize(3);
      g.input[1] = cw.output[0];
      g.input[2] = cb.output[0];
      if (bn_first) g.input[0] = x; else g.output[0] = y;
      // the BN node goes; the new constants are placed before every operator
      def->op.erase(def->op.begin() + bi);
      def->op.insert(def->op.begin(), cb);
      def->op.insert(def->op.begin(), cw);
      changed = true;
    }
  }
  if (serial == 0) return;
  // constants that only the folded nodes read (old weights, the BN parameters) would still be uploaded
  std::map<std::string, int> consumers;
  for (const auto& op : def->op)
    for (const auto& in : op.input) ++consumers[in];
  std::set<std::string> ext_out;
  for (const auto& v : def->external_output) ext_out.insert(v.name);
  for (size_t i = def->op.size(); i-- > 0;) {
    const OperatorDef& op = def->op[i];
    if (op.type == "ConstantFill" && op.output.size() == 1 && consumers[op.output[0]] == 0 && !ext_out.count(op.output[0]))
      def->op.erase(def->op.begin() + i);
  }
}

// ---- Gemm + activation fusion -----------------------------------------------------------------------
void FuseGemmActivation(NetDef* def) {
  bool changed = true;
  while (changed) {
    changed = false;
    std::map<std::string, int> consumers;
    for (const auto& op : def->op)
      for (const auto& in : op.input) ++consumers[in];
    std::set<std::string> ext_out;
    for (const auto& v : def->external_output) ext_out.insert(v.name);
    for (size_t i = 0; i < def->op.size() && !changed; ++i) {
      OperatorDef& g = def->op[i];
      const bool gemm = g.type == "Gemm" && g.input.size() == 3, pruned = g.type == "PrunedGemm" && g.input.size() == 5;
      if (!(gemm || pruned) || g.FindArg("epilogue") || g.output.size() != 1) continue;
      const std::string& y = g.output[0];
      if (consumers[y] != 1 || ext_out.count(y)) continue;
      for (size_t j = i + 1; j < def->op.size(); ++j) {
        OperatorDef& a = def->op[j];
        if (a.input.empty() || a.input[0] != y) continue;
        int kind = 0;
        if (a.type == "PRelu" && a.input.size() == 2) kind = XB_EPI_PRELU;
        else if (a.type == "Dice" && a.input.size() == 4) kind = XB_EPI_DICE;
        else if (a.type == "Sigmoid" && a.input.size() == 1) kind = XB_EPI_SIGMOID;
        if (!kind || a.output.size() != 1) break;
        if (a.has_device_option != g.has_device_option) break;
        Argument e;
        e.name = "epilogue"; e.has_i = true; e.i = kind;
        g.arg.push_back(e);
        if (const Argument* ns = a.FindArg("nosqrt")) g.arg.push_back(*ns);
        for (size_t k = 1; k < a.input.size(); ++k) g.input.push_back(a.input[k]);
        g.output[0] = a.output[0];
        def->op.erase(def->op.begin() + j);
        changed = true;
        break;
      }
    }
  }
}

}  // namespace blaze
