// Predictor / PredictorManager / InitScheduler and the Blaze_* C API.
// Behaviour follows blaze/blaze/api/cpp_api/predictor_impl.cc:14-225 and
// predictor_manager_impl.cc:18-177: exceptions raised by operators are caught at
// the API boundary, logged and turned into `false` / nullptr.
#include <cstring>
#include <fstream>

#include "blaze/api/c_api/c_api_predictor.h"
#include "blaze/api/cpp_api/predictor.h"
#include "batching.h"
#include "runtime.h"

namespace blaze {

namespace {
thread_local std::string g_last_error;
void SetError(const std::string& e) {
  g_last_error = e;
  LOG_ERROR(e);
}
const std::vector<size_t> kEmptyShape;
}  // namespace

// ---- impl classes ---------------------------------------------------------------------------------
class PredictorImpl {
 public:
  PredictorImpl(const NetDef& def, std::shared_ptr<store::SparsePuller> puller, std::shared_ptr<ConstantStore> constants) {
    ws_.Init(def);
    ws_.SetSparsePuller(puller);
    ws_.SetConstantStore(constants);
    CUDA_CHECK(cudaSetDevice(def.device_option.device_id));
    net_ = ws_.CreateNet();
    for (const auto& v : def.external_input) in_types_[v.name] = v.dtype;
    for (const auto& v : def.external_input) feed_cfg_[v.name] = v;
  }

  Blob* InputBlob(const char* name) {
    Blob* b = ws_.GetBlob(name);
    BLAZE_CONDITION_THROW(b != nullptr && in_types_.count(name), "input ", name, " does not exist");
    return b;
  }

  Workspace ws_;
  std::unique_ptr<Net> net_;
  std::unordered_map<std::string, int> in_types_;
  std::unordered_map<std::string, ValueInfo> feed_cfg_;
  std::vector<char> staging_;
  std::vector<size_t> scratch_shape_;
  bool profile_ = false;
  // request batching (InitScheduler(enable_batching = true)): the queue of this model and device, and
  // what the last batched Forward reported
  std::shared_ptr<BatchQueue> queue_;
  std::string async_error_;
};

class PredictorManagerImpl {
 public:
  bool LoadSparse(const char* uri, const char* type) {
    puller_.reset(store::SparsePullerCreationRegisterer::Get()->CreateSparsePuller(type ? type : "qed_sparse_puller"));
    if (!puller_) { SetError(MakeString("sparse puller type ", type ? type : "(null)", " is not registered")); return false; }
    if (uri == nullptr || !*uri) {
      if (std::string(type ? type : "") == "qed_sparse_puller") { SetError("qed_sparse_puller needs a file"); return false; }
      return true;
    }
    const store::Status st = puller_->Load(uri);
    if (st != store::kOK) { SetError(MakeString("load sparse model weight failed, uri=", uri)); return false; }
    return true;
  }

  bool SetNet(const NetDef& def, bool optimize) {
    net_def_ = def;
    if (optimize) {
      FoldBatchNorm(&net_def_);
      FuseDinSubgraphs(&net_def_);
      FuseGemmActivation(&net_def_);
    }
    loaded_ = true;
    return true;
  }

  bool LoadText(const std::string& text, bool optimize) {
    NetDef def;
    std::string err;
    if (!ParseNetDefText(text, &def, &err)) { SetError("parse NetDef text failed: " + err); return false; }
    return SetNet(def, optimize);
  }

  bool LoadFile(const char* filename, bool optimize) {
    std::ifstream is(filename, std::ios::binary);
    if (!is.is_open()) { SetError(MakeString("open model file failed: ", filename)); return false; }
    std::string bytes((std::istreambuf_iterator<char>(is)), std::istreambuf_iterator<char>());
    NetDef def;
    std::string err;
    // a .blaze file is the protobuf wire format; text-format NetDefs are accepted as well
    if (ParseNetDefBinary(bytes, &def, &err) && !def.op.empty()) return SetNet(def, optimize);
    if (ParseNetDefText(bytes, &def, &err) && !def.op.empty()) return SetNet(def, optimize);
    SetError(MakeString("model file ", filename, " is neither a binary nor a text NetDef: ", err));
    return false;
  }

  Predictor* Create(PredictDeviceType type, int device_id);
  // PredictorManagerImpl is a friend of Predictor: the C API extensions reach the implementation through it
  static PredictorImpl* ImplOf(Predictor* p) { return p->impl_; }

  NetDef net_def_;
  bool loaded_ = false;
  int data_type_ = kPDT_Float;
  std::string run_mode_;
  std::shared_ptr<store::SparsePuller> puller_;
  std::mutex mu_;
  std::map<int, std::shared_ptr<ConstantStore>> constants_;      // per device
  std::map<int, std::shared_ptr<BatchQueue>> queues_;            // per device, as the reference keeps one per NetDef
};

struct ManagerAccess {
  static PredictorManagerImpl* impl(PredictorManager* m) { return m->impl_; }
};

Predictor* PredictorManagerImpl::Create(PredictDeviceType type, int device_id) {
  std::lock_guard<std::mutex> lock(mu_);
  try {
    BLAZE_CONDITION_THROW(loaded_, "no model loaded");
    NetDef def = net_def_;
    // kPDT_Unkown keeps the device written in the model; there are no CPU operators to fall back to
    if (type == kPDT_CUDA || type == kPDT_Unkown) {
      if (type == kPDT_CUDA || def.device_option.device_type == kCPU) def.device_option.device_type = kCUDA;
      def.device_option.device_id = device_id;
      for (auto& op : def.op)
        if (op.has_device_option) { op.device_option.device_type = kCUDA; op.device_option.device_id = device_id; }
    } else {
      BLAZE_THROW("kPDT_CPU predictors are not available: this backend runs on CUDA devices only");
    }
    if (!run_mode_.empty()) def.run_mode = run_mode_;
    auto& store = constants_[device_id];
    if (!store) store.reset(new ConstantStore());
    std::unique_ptr<PredictorImpl> impl(new PredictorImpl(def, puller_, store));
    if (GlobalSchedulerOptions().enable_batching) {
      auto& queue = queues_[device_id];
      if (!queue) queue.reset(new BatchQueue(def, puller_, store, GlobalSchedulerOptions()));
      impl->queue_ = queue;
    }
    return new Predictor(impl.release());
  } catch (const std::exception& e) {
    SetError(MakeString("create predictor failed: ", e.what()));
    return nullptr;
  }
}

// ---- FeedNameUtility ------------------------------------------------------------------------------
std::string FeedNameUtility::SparseFeatureName2FeedName(const std::string& n, SparseFeatureType sft) {
  switch (sft) {
    case kSparseFeatureId: return n + ".ids";
    case kSparseFeatureValue: return n + ".values";
    default: return n + ".segments";
  }
}
std::string FeedNameUtility::IndicatorLevel2FeedName(int level) { return "indicator." + std::to_string(level); }

// ---- Predictor ------------------------------------------------------------------------------------
Predictor::Predictor(PredictorImpl* impl) : impl_(impl) {}
Predictor::~Predictor() { delete impl_; }

FeedNameConfig Predictor::GetFeedNameConfig(const std::string& feed_name) {
  FeedNameConfig c;
  c.feature_name = feed_name; c.feature_type = kDenseFeature; c.level = 0; c.sparse_feature_type = kSparseFeatureId;
  auto ends = [&](const char* suf) {
    const size_t n = strlen(suf);
    return feed_name.size() > n && feed_name.compare(feed_name.size() - n, n, suf) == 0;
  };
  if (feed_name.compare(0, 10, "indicator.") == 0) {
    c.feature_type = kAuxIndicator; c.level = atoi(feed_name.c_str() + 10);
  } else if (ends(".ids")) { c.feature_type = kSparseFeature; c.sparse_feature_type = kSparseFeatureId; c.feature_name = feed_name.substr(0, feed_name.size() - 4); }
  else if (ends(".values")) { c.feature_type = kSparseFeature; c.sparse_feature_type = kSparseFeatureValue; c.feature_name = feed_name.substr(0, feed_name.size() - 7); }
  else if (ends(".segments")) { c.feature_type = kSparseFeature; c.sparse_feature_type = kAuxSparseFeatureSegment; c.feature_name = feed_name.substr(0, feed_name.size() - 9); }
  return c;
}

bool Predictor::ReshapeInput(const char* name, const std::vector<size_t>& shape) {
  try {
    Blob* b = impl_->InputBlob(name);
    b->set_data_type(impl_->in_types_[name]);
    b->Reshape(shape);
    return true;
  } catch (const std::exception& e) { SetError(e.what()); return false; }
}
bool Predictor::ReshapeInput(size_t idx, const std::vector<size_t>& shape) {
  if (idx >= impl_->net_->external_input().size()) { SetError("input index out of range"); return false; }
  return ReshapeInput(impl_->net_->external_input()[idx].c_str(), shape);
}

bool Predictor::Feed(const char* name, const void* data, size_t len) {
  try {
    Blob* b = impl_->InputBlob(name);
    BLAZE_CONDITION_THROW(len == b->bytes(), "feed of ", name, ": len=", len, " blob bytes=", b->bytes());
    if (len == 0) return true;
    CUDA_CHECK(cudaSetDevice(impl_->net_->device_id()));
    CUDA_CHECK(cudaMemcpyAsync(b->as<void>(), data, len, cudaMemcpyHostToDevice, impl_->net_->stream()));
    return true;
  } catch (const std::exception& e) { SetError(e.what()); return false; }
}
bool Predictor::Feed(size_t idx, const void* data, size_t len) {
  if (idx >= impl_->net_->external_input().size()) { SetError("input index out of range"); return false; }
  return Feed(impl_->net_->external_input()[idx].c_str(), data, len);
}

size_t Predictor::InputSize() const { return impl_->net_->external_input().size(); }
PredictDataType Predictor::InputDataType(const char* name) const {
  auto it = impl_->in_types_.find(name);
  return it == impl_->in_types_.end() ? kPDT_Invalid : (PredictDataType)it->second;
}
PredictDataType Predictor::InputDataType(size_t idx) const {
  return idx < InputSize() ? InputDataType(impl_->net_->external_input()[idx].c_str()) : kPDT_Invalid;
}
const std::vector<std::string>& Predictor::ListInputName() const { return impl_->net_->external_input(); }

bool Predictor::Forward(const PredictorCallback&& cb) {
  try {
    CUDA_CHECK(cudaSetDevice(impl_->net_->device_id()));
    impl_->async_error_.clear();
    if (cb && impl_->queue_) {
      // asynchronous: the batch thread stacks this request with others of the same model, runs them
      // as one net and calls cb once this predictor's outputs are in place
      BatchQueue::Task task;
      task.ws = &impl_->ws_;
      BatchQueue::Describe(impl_->net_->net_def(), &task);
      CUDA_CHECK(cudaEventCreateWithFlags(&task.ready, cudaEventDisableTiming));
      CUDA_CHECK(cudaEventRecord(task.ready, impl_->net_->stream()));
      PredictorImpl* impl = impl_;
      PredictorCallback user_cb = cb;
      task.done = [impl, user_cb](const std::string& error) {
        impl->async_error_ = error;
        user_cb();
      };
      cudaEvent_t ready = task.ready;
      std::string why;
      if (!impl_->queue_->Schedule(&task, &why)) {
        cudaEventDestroy(ready);
        SetError(MakeString("forward failed: ", why));
        return false;
      }
      return true;
    }
    impl_->net_->profile = impl_->profile_;
    if (!impl_->net_->Run()) return false;
    CUDA_CHECK(cudaStreamSynchronize(impl_->net_->stream()));
    impl_->net_->CheckDeviceStatus();
    if (cb) cb();
    return true;
  } catch (const std::exception& e) {
    SetError(MakeString("forward failed: ", e.what()));
    return false;
  }
}

bool Predictor::Output(const char* name, void** data, size_t* len) {
  try {
    BLAZE_CONDITION_THROW(impl_->async_error_.empty(), impl_->async_error_);
    Blob* b = impl_->ws_.GetBlob(name);
    BLAZE_CONDITION_THROW(b != nullptr, "output ", name, " does not exist");
    impl_->staging_.resize(std::max<size_t>(b->bytes(), 1));
    if (b->bytes()) {
      CUDA_CHECK(cudaMemcpyAsync(impl_->staging_.data(), b->as<void>(), b->bytes(), cudaMemcpyDeviceToHost, impl_->net_->stream()));
      CUDA_CHECK(cudaStreamSynchronize(impl_->net_->stream()));
    }
    *data = impl_->staging_.data();
    *len = b->bytes();
    return true;
  } catch (const std::exception& e) { SetError(e.what()); return false; }
}
bool Predictor::Output(size_t idx, void** data, size_t* len) {
  if (idx >= OutputSize()) { SetError("output index out of range"); return false; }
  return Output(impl_->net_->external_output()[idx].c_str(), data, len);
}
const std::vector<size_t>& Predictor::OutputShape(const char* name) const {
  Blob* b = impl_->ws_.GetBlob(name);
  return b ? b->shape() : kEmptyShape;
}
const std::vector<size_t>& Predictor::OutputShape(size_t idx) const {
  return idx < OutputSize() ? OutputShape(impl_->net_->external_output()[idx].c_str()) : kEmptyShape;
}
PredictDataType Predictor::OutputDataType(const char* name) const {
  Blob* b = impl_->ws_.GetBlob(name);
  return b ? (PredictDataType)b->data_type() : kPDT_Invalid;
}
PredictDataType Predictor::OutputDataType(size_t idx) const {
  return idx < OutputSize() ? OutputDataType(impl_->net_->external_output()[idx].c_str()) : kPDT_Invalid;
}
size_t Predictor::OutputSize() const { return impl_->net_->external_output().size(); }
const std::vector<std::string>& Predictor::ListOutputName() const { return impl_->net_->external_output(); }

std::vector<std::string> Predictor::ListInternalName() const { return impl_->ws_.BlobNames(); }
bool Predictor::InternalParam(const char* name, void** data, size_t* len) { return Output(name, data, len); }
const std::vector<size_t>& Predictor::InternalShape(const char* name) const { return OutputShape(name); }
int Predictor::InternalDataType(const char* name) const {
  Blob* b = impl_->ws_.GetBlob(name);
  return b ? b->data_type() : -1;
}

void Predictor::RegisterObservers(const std::vector<std::string>& names) {
  for (const auto& n : names)
    if (n == "profile" || n == "cost") impl_->profile_ = true;
}
void Predictor::DumpObservers(std::unordered_map<std::string, std::string>* dump_map) {
  if (!dump_map) return;
  std::ostringstream os;
  os << "[";
  bool first = true;
  for (const auto& kv : impl_->net_->op_ms) {
    os << (first ? "" : ",") << "{\"op\":\"" << kv.first << "\",\"ms\":" << kv.second << "}";
    first = false;
  }
  os << "]";
  (*dump_map)["profile"] = os.str();
}

// ---- PredictorManager -----------------------------------------------------------------------------
PredictorManager::PredictorManager() : impl_(new PredictorManagerImpl()) {}
PredictorManager::~PredictorManager() { delete impl_; }
void PredictorManager::SetDataType(PredictDataType t) { impl_->data_type_ = t; }
void PredictorManager::SetRunMode(const char* m) { impl_->run_mode_ = m ? m : ""; }
bool PredictorManager::LoadSparseModelWeight(const char* uri, const char* type) { return impl_->LoadSparse(uri, type); }
bool PredictorManager::LoadModel(const char* filename, bool optimization_pass) { return impl_->LoadFile(filename, optimization_pass); }
bool PredictorManager::LoadDeepNetModel(const char*, const char*, bool) {
  SetError("ULF (DeepNet) model files are not read by this backend: convert the model to a Blaze NetDef first");
  return false;
}
bool PredictorManager::LoadModel(const char* conf_file, const char*, ModelType model_type, bool optimization_pass) {
  if (model_type == kBlaze) return impl_->LoadFile(conf_file, optimization_pass);
  SetError("only Blaze NetDef models (ModelType kBlaze) are read by this backend");
  return false;
}
Predictor* PredictorManager::CreatePredictor(PredictDeviceType type, int device_id) { return impl_->Create(type, device_id); }

bool InitScheduler(bool enable_batching, int max_batch_size, int batch_timeout_micros, int, int, int) {
  // Every operator runs in stream order on the predictor's own stream, so the thread counts have
  // nothing to size. Batching applies to predictors created after this call: their Forward(cb) goes
  // through the model's batch queue (one batch thread per model and device).
  if (enable_batching && max_batch_size < 1) { SetError("InitScheduler: max_batch_size must be at least 1"); return false; }
  SchedulerOptions& o = GlobalSchedulerOptions();
  o.enable_batching = enable_batching;
  if (enable_batching) {
    o.max_batch_size = max_batch_size;
    o.batch_timeout_micros = batch_timeout_micros < 0 ? 0 : batch_timeout_micros;
  }
  return true;
}

}  // namespace blaze

// ---- C API ------------------------------------------------------------------------------------------
using namespace blaze;

namespace {
struct CPredictor {
  Predictor* p;
  std::vector<size_t> shape;
  std::vector<std::string> names;
  std::vector<const char*> name_ptrs;
  std::unordered_map<std::string, std::string> dump;
  std::vector<std::string> dump_k, dump_v;
  std::vector<const char*> dump_kp, dump_vp;
};
#define API_BEGIN() try {
#define API_END()                                  \
  }                                                \
  catch (const std::exception& e) {                \
    SetError(e.what());                            \
    return -1;                                     \
  }                                                \
  return 0;
inline int Ret(bool ok) { return ok ? 0 : -1; }
}  // namespace

extern "C" {

const char* Blaze_GetLastErrorString(void) { return g_last_error.c_str(); }

int Blaze_InitScheduler(int a, int b, int c, int d, int e, int f) { return Ret(InitScheduler(a != 0, b, c, d, e, f)); }
int Blaze_PredictorManagerCreate(PredictorManagerHandle* handle) {
  API_BEGIN();
  *handle = new PredictorManager();
  API_END();
}
int Blaze_PredictorManagerDelete(PredictorManagerHandle handle) {
  delete static_cast<PredictorManager*>(handle);
  return 0;
}
int Blaze_PredictorManagerSetDataType(PredictorManagerHandle h, int data_type) {
  static_cast<PredictorManager*>(h)->SetDataType((PredictDataType)data_type);
  return 0;
}
int Blaze_PredictorManagerSetRunMode(PredictorManagerHandle h, const char* run_mode) {
  static_cast<PredictorManager*>(h)->SetRunMode(run_mode);
  return 0;
}
int Blaze_LoadSparseModelWeight(PredictorManagerHandle h, const char* file) {
  return Ret(static_cast<PredictorManager*>(h)->LoadSparseModelWeight(file));
}
int Blaze_PredcitorManagerLoadModel(PredictorManagerHandle h, const char* file, int optimization_pass) {
  return Ret(static_cast<PredictorManager*>(h)->LoadModel(file, optimization_pass != 0));
}
int Blaze_PredictorManagerLoadDeepNetModel(PredictorManagerHandle h, const char* conf, const char* param, int opt) {
  return Ret(static_cast<PredictorManager*>(h)->LoadDeepNetModel(conf, param, opt != 0));
}
int Blaze_PredictorCreate(PredictorManagerHandle mgr, int device_type, int device_id, PredictorHandle* handle) {
  Predictor* p = static_cast<PredictorManager*>(mgr)->CreatePredictor((PredictDeviceType)device_type, device_id);
  if (!p) return -1;
  CPredictor* c = new CPredictor();
  c->p = p;
  *handle = c;
  return 0;
}
int Blaze_PredictorDelete(PredictorHandle handle) {
  CPredictor* c = static_cast<CPredictor*>(handle);
  if (c) { delete c->p; delete c; }
  return 0;
}
int Blaze_PredictorReshapeInput(PredictorHandle h, const char* name, const int* data, int num) {
  std::vector<size_t> shape(data, data + num);
  return Ret(static_cast<CPredictor*>(h)->p->ReshapeInput(name, shape));
}
int Blaze_PredictorFeed(PredictorHandle h, const char* name, void* data, int len) {
  return Ret(static_cast<CPredictor*>(h)->p->Feed(name, data, (size_t)len));
}
int Blaze_PredictorForward(PredictorHandle h) { return Ret(static_cast<CPredictor*>(h)->p->Forward()); }
int Blaze_PredictorOutputShape(PredictorHandle h, const char* name, size_t* ndim, size_t** shape) {
  CPredictor* c = static_cast<CPredictor*>(h);
  c->shape = c->p->OutputShape(name);
  *ndim = c->shape.size();
  *shape = c->shape.data();
  return 0;
}
int Blaze_PredictorOutputDataType(PredictorHandle h, const char* name, int* data_type) {
  *data_type = static_cast<CPredictor*>(h)->p->OutputDataType(name);
  return *data_type == kPDT_Invalid ? -1 : 0;
}
int Blaze_PredictorOutput(PredictorHandle h, const char* name, void* data, size_t len) {
  void* src = nullptr;
  size_t n = 0;
  if (!static_cast<CPredictor*>(h)->p->Output(name, &src, &n)) return -1;
  if (n != len) { SetError(MakeString("output ", name, " has ", n, " bytes, the caller asked for ", len)); return -1; }
  memcpy(data, src, n);
  return 0;
}
static int ListNames(CPredictor* c, const std::vector<std::string>& names, size_t* ndim, const char*** out) {
  c->names = names;
  c->name_ptrs.clear();
  for (const auto& n : c->names) c->name_ptrs.push_back(n.c_str());
  *ndim = c->names.size();
  *out = c->name_ptrs.data();
  return 0;
}
int Blaze_PredictorParamName(PredictorHandle h, size_t* ndim, const char*** name) {
  CPredictor* c = static_cast<CPredictor*>(h);
  return ListNames(c, c->p->ListInternalName(), ndim, name);
}
int Blaze_PredictorParamShape(PredictorHandle h, const char* name, size_t* ndim, size_t** shape) {
  return Blaze_PredictorOutputShape(h, name, ndim, shape);
}
int Blaze_PredictorParamDataType(PredictorHandle h, const char* name, int* data_type) {
  *data_type = static_cast<CPredictor*>(h)->p->InternalDataType(name);
  return *data_type < 0 ? -1 : 0;
}
int Blaze_PredictorParam(PredictorHandle h, const char* name, void* data, size_t len) {
  return Blaze_PredictorOutput(h, name, data, len);
}
int Blaze_PredictorListInputNames(PredictorHandle h, size_t* ndim, const char*** names) {
  CPredictor* c = static_cast<CPredictor*>(h);
  return ListNames(c, c->p->ListInputName(), ndim, names);
}
int Blaze_PredictorListOutputNames(PredictorHandle h, size_t* ndim, const char*** names) {
  CPredictor* c = static_cast<CPredictor*>(h);
  return ListNames(c, c->p->ListOutputName(), ndim, names);
}
int Blaze_PredictorRegisterObservers(PredictorHandle h, size_t ndim, const char** names) {
  std::vector<std::string> v(names, names + ndim);
  static_cast<CPredictor*>(h)->p->RegisterObservers(v);
  return 0;
}
int Blaze_PredictorDumpObservers(PredictorHandle h, size_t* ndim, const char*** key, const char*** value) {
  CPredictor* c = static_cast<CPredictor*>(h);
  c->dump.clear();
  c->p->DumpObservers(&c->dump);
  c->dump_k.clear(); c->dump_v.clear(); c->dump_kp.clear(); c->dump_vp.clear();
  for (const auto& kv : c->dump) { c->dump_k.push_back(kv.first); c->dump_v.push_back(kv.second); }
  for (size_t i = 0; i < c->dump_k.size(); ++i) { c->dump_kp.push_back(c->dump_k[i].c_str()); c->dump_vp.push_back(c->dump_v[i].c_str()); }
  *ndim = c->dump_k.size();
  *key = c->dump_kp.data();
  *value = c->dump_vp.data();
  return 0;
}

// ---- extensions -------------------------------------------------------------------------------------
int Blaze_B200_LoadModelFromText(PredictorManagerHandle h, const char* text, int optimization_pass) {
  return Ret(ManagerAccess::impl(static_cast<PredictorManager*>(h))->LoadText(text ? text : "", optimization_pass != 0));
}
int Blaze_B200_LoadSparseModelWeight(PredictorManagerHandle h, const char* uri, const char* type) {
  return Ret(static_cast<PredictorManager*>(h)->LoadSparseModelWeight(uri, type ? type : "b200_sparse_puller"));
}
int Blaze_B200_AddTable(PredictorManagerHandle h, const char* table_name, int64_t rows, int dim, int storage_dtype,
                        const float* weights, const int64_t* keys) {
  API_BEGIN();
  PredictorManagerImpl* m = ManagerAccess::impl(static_cast<PredictorManager*>(h));
  if (!m->puller_) BLAZE_CONDITION_THROW(m->LoadSparse(nullptr, "b200_sparse_puller"), "cannot create the sparse puller");
  BLAZE_CONDITION_THROW(m->puller_->AddTable(table_name, rows, dim, storage_dtype, weights, keys) == store::kOK,
                        "AddTable ", table_name, " failed");
  API_END();
}
int Blaze_B200_ShardedInit(PredictorManagerHandle h, int rank, int world, const void* unique_id128, int64_t max_ids_per_step,
                           int partial_dtype, float capacity_factor) {
  API_BEGIN();
  PredictorManagerImpl* m = ManagerAccess::impl(static_cast<PredictorManager*>(h));
  if (!m->puller_) BLAZE_CONDITION_THROW(m->LoadSparse(nullptr, "b200_sharded_sparse_puller"), "cannot create the sharded puller");
  BLAZE_CONDITION_THROW(m->puller_->InitSharded(rank, world, unique_id128, max_ids_per_step, partial_dtype, capacity_factor) == store::kOK,
                        "the loaded sparse puller does not shard tables (load b200_sharded_sparse_puller) or the arguments are invalid");
  API_END();
}
int Blaze_B200_ShardUniqueId(void* unique_id128) {
  if (xb_shard_unique_id(unique_id128) != 0) { SetError(xb_last_error()); return -1; }
  return 0;
}
int Blaze_B200_AddDeviceShard(PredictorManagerHandle h, const char* table_name, int64_t rows, int dim, int storage_dtype,
                              const void* device_weights, int64_t pitch_bytes) {
  API_BEGIN();
  PredictorManagerImpl* m = ManagerAccess::impl(static_cast<PredictorManager*>(h));
  BLAZE_CONDITION_THROW(m->puller_ != nullptr, "no sparse puller loaded");
  BLAZE_CONDITION_THROW(m->puller_->AddDeviceShard(table_name, rows, dim, storage_dtype, device_weights, pitch_bytes) == store::kOK,
                        "AddDeviceShard ", table_name, " failed (only the sharded puller takes device shards)");
  API_END();
}
int Blaze_B200_ModelOpTypes(PredictorManagerHandle h, char* buffer, size_t capacity) {
  // operator types of the loaded (and, with optimization_pass, rewritten) NetDef, comma separated
  PredictorManagerImpl* m = ManagerAccess::impl(static_cast<PredictorManager*>(h));
  std::string s;
  for (const auto& op : m->net_def_.op) s += (s.empty() ? "" : ",") + op.type;
  if (!buffer || capacity < s.size() + 1) return (int)s.size() + 1;
  memcpy(buffer, s.c_str(), s.size() + 1);
  return 0;
}
int Blaze_B200_PredictorFeedDevice(PredictorHandle h, const char* name, const void* device_data, size_t len) {
  API_BEGIN();
  PredictorImpl* impl = PredictorManagerImpl::ImplOf(static_cast<CPredictor*>(h)->p);
  Blob* b = impl->InputBlob(name);
  BLAZE_CONDITION_THROW(len == b->bytes(), "feed of ", name, ": len=", len, " blob bytes=", b->bytes());
  if (len) CUDA_CHECK(cudaMemcpyAsync(b->as<void>(), device_data, len, cudaMemcpyDeviceToDevice, impl->net_->stream()));
  API_END();
}
int Blaze_B200_PredictorOutputDevice(PredictorHandle h, const char* name, void** device_data, size_t* len) {
  API_BEGIN();
  PredictorImpl* impl = PredictorManagerImpl::ImplOf(static_cast<CPredictor*>(h)->p);
  Blob* b = impl->ws_.GetBlob(name);
  BLAZE_CONDITION_THROW(b != nullptr, "output ", name, " does not exist");
  *device_data = b->as<void>();
  *len = b->bytes();
  API_END();
}
int Blaze_B200_PredictorLastLaunchCount(PredictorHandle h, int* count) {
  API_BEGIN();
  PredictorImpl* impl = PredictorManagerImpl::ImplOf(static_cast<CPredictor*>(h)->p);
  *count = impl->net_->last_launches;
  API_END();
}
int Blaze_B200_PredictorForwardAsync(PredictorHandle h, void (*cb)(void*), void* arg) {
  if (cb == nullptr) { SetError("Blaze_B200_PredictorForwardAsync needs a callback"); return -1; }
  return Ret(static_cast<CPredictor*>(h)->p->Forward([cb, arg] { cb(arg); }));
}
int Blaze_B200_PlanBatch(const int64_t* rows, int n_tasks, int n_inputs, int max_tasks, int* picked) {
  if (!rows || !picked || n_tasks < 0 || n_inputs < 0) { SetError("Blaze_B200_PlanBatch: bad arguments"); return -1; }
  std::deque<BatchQueue::Task> queue((size_t)n_tasks);
  for (int t = 0; t < n_tasks; ++t)
    for (int j = 0; j < n_inputs; ++j) queue[t].rows.push_back((TIndex)rows[(size_t)t * n_inputs + j]);
  const std::vector<size_t> got = BatchQueue::PickBatch(queue, (size_t)std::max(max_tasks, 0));
  for (size_t i = 0; i < got.size(); ++i) picked[i] = (int)got[i];
  return (int)got.size();
}
int Blaze_B200_BatchingStats(int64_t* batches, int64_t* tasks) {
  if (batches) *batches = GlobalBatchingStats().batches.load();
  if (tasks) *tasks = GlobalBatchingStats().tasks.load();
  return 0;
}

}  // extern "C"
