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
