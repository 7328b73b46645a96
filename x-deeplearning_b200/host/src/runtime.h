// Internal runtime of the B200 host library: NetDef model, Blob, Workspace,
// operator framework and nets. It mirrors the structure an operator author sees
// in Blaze (blaze/blaze/operator/operator.h:21-292, blaze/blaze/common/blob.h:17-103,
// blaze/blaze/graph/workspace.h:26-196, blaze/blaze/graph/net.h:21-182) so that the
// CUDA operator classes read like Blaze operators, but it is written from scratch
// and only knows one device type for compute: CUDA on sm_100a.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "xdlb200.h"

namespace blaze {

// ---- errors -----------------------------------------------------------------------------------
class Exception : public std::runtime_error {
 public:
  explicit Exception(const std::string& m) : std::runtime_error(m) {}
};

template <typename... Args>
inline std::string MakeString(const Args&... args) {
  std::ostringstream os;
  int dummy[] = {0, ((os << args), 0)...};
  (void)dummy;
  return os.str();
}

#define BLAZE_THROW(...) throw ::blaze::Exception(::blaze::MakeString("[", __FILE__, ":", __LINE__, "] ", __VA_ARGS__))
#define BLAZE_CONDITION_THROW(cond, ...) \
  do {                                   \
    if (!(cond)) BLAZE_THROW(__VA_ARGS__); \
  } while (0)
#define CUDA_CHECK(call)                                                                          \
  do {                                                                                            \
    cudaError_t e__ = (call);                                                                     \
    if (e__ != cudaSuccess) BLAZE_THROW("cuda error status=", (int)e__, " msg=", cudaGetErrorString(e__)); \
  } while (0)
#define XB_CHECK(call)                                                        \
  do {                                                                        \
    int rc__ = (call);                                                        \
    if (rc__ != 0) BLAZE_THROW("kernel library error ", rc__, ": ", xb_last_error()); \
  } while (0)

void LogError(const std::string& msg);
#define LOG_ERROR(...) ::blaze::LogError(::blaze::MakeString(__VA_ARGS__))

// ---- types (numbering of blaze/blaze/proto/blaze.proto:6-20) -----------------------------------
enum DataType { kFloat = 1, kInt32 = 2, kBool = 5, kInt64 = 10, kFloat16 = 12, kDouble = 13 };
enum DeviceType { kCPU = 0, kCUDA = 1 };
typedef size_t TIndex;
size_t DataTypeSize(int dtype);

// ---- NetDef -----------------------------------------------------------------------------------
struct Argument {
  std::string name;
  bool has_f = false, has_i = false, has_s = false;
  float f = 0;
  int64_t i = 0;
  std::string s;
  std::vector<float> floats;
  std::vector<int64_t> ints;
  std::vector<std::string> strings;
};

struct DeviceOption {
  int device_type = kCPU;
  int device_id = 0;
  bool is_pipe = false;
};

struct NetDef;
struct OperatorDef {
  std::string type, name;
  std::vector<std::string> input, output;
  std::vector<Argument> arg;
  bool has_device_option = false;
  DeviceOption device_option;
  const Argument* FindArg(const std::string& n) const;
  std::string DebugString() const;
};

struct ValueInfo {
  std::string name, feature_name;
  int dtype = kFloat, level = 0, input_type = 0;
};

struct NetDef {
  std::string name, run_mode = "simple";
  std::vector<OperatorDef> op;
  std::vector<Argument> arg;
  DeviceOption device_option;
  std::vector<ValueInfo> external_input, external_output;
};

// Protobuf text format (what the reference's operator tests are written in).
bool ParseNetDefText(const std::string& text, NetDef* out, std::string* err);
// Protobuf wire format of message blaze.NetDef (what LoadModel reads from a .blaze file).
bool ParseNetDefBinary(const std::string& bytes, NetDef* out, std::string* err);
// Generic text-format reader used for EmbeddingConfig as well: a tree of fields.
struct TextNode {
  std::multimap<std::string, std::string> scalars;
  std::vector<std::pair<std::string, std::unique_ptr<TextNode>>> children;
  std::vector<const TextNode*> Children(const std::string& name) const;
  bool Get(const std::string& name, std::string* v) const;
  int64_t GetInt(const std::string& name, int64_t def) const;
};
bool ParseTextProto(const std::string& text, TextNode* root, std::string* err);

// ---- Blob -------------------------------------------------------------------------------------
// Shape + dtype + device memory. Growth-only reallocation, like Blaze's Blob.
class Blob {
 public:
  explicit Blob(const DeviceOption& opt) : opt_(opt) {}
  ~Blob();
  Blob(const Blob&) = delete;
  Blob& operator=(const Blob&) = delete;

  void Reshape(const std::vector<TIndex>& shape);
  // Alias of another blob's memory with a new shape (Blaze's RefReshape): no copy.
  void RefReshape(Blob* src, const std::vector<TIndex>& shape);
  const std::vector<TIndex>& shape() const { return shape_; }
  size_t size() const;
  size_t size(size_t from, size_t to) const;
  int data_type() const { return dtype_; }
  void set_data_type(int dt) { dtype_ = dt; }
  const DeviceOption& device_option() const { return opt_; }
  template <typename T = void>
  T* as() const { return reinterpret_cast<T*>(ref_ ? ref_->data_ : data_); }
  size_t bytes() const { return size() * DataTypeSize(dtype_); }
  bool is_constant = false;      // written once by ConstantFill: safe to cache derived layouts
  std::vector<char> host_copy;   // constants keep their host image (shape operands are read from it)

 private:
  DeviceOption opt_;
  std::vector<TIndex> shape_;
  int dtype_ = kFloat;
  void* data_ = nullptr;
  size_t capacity_ = 0;
  Blob* ref_ = nullptr;
};

// ---- contexts ---------------------------------------------------------------------------------
class CUDAContext {
 public:
  explicit CUDAContext(const DeviceOption& opt);
  void Activate() const;
  cudaStream_t cuda_stream() const { return stream_; }
  void FinishDeviceComputation() const;
  int device_id() const { return device_id_; }
  static int device_type() { return kCUDA; }

 private:
  int device_id_;
  cudaStream_t stream_;
};

// ---- sparse store -----------------------------------------------------------------------------
namespace store {
enum Status { kOK = 0, kTimeout, kFail };
enum UDFType { kSum = 0, kAvg, kAssign };
enum TruncDirection { kOrder = 0, kReverse };

// Same fields as blaze/blaze/store/sparse_puller.h:42-74. When a CUDA operator calls Get,
// key / key_num / value / out are DEVICE pointers and `stream` is the operator's stream.
struct SparsePullerInput {
  std::string version, name;
  void* key = nullptr;
  void* key_num = nullptr;
  size_t key_num_size = 0;
  size_t key_size = 0;             // number of ids (extension: the device path cannot count them)
  void* value = nullptr;
  int key_type = kInt64, value_type = kFloat, num_type = kInt32;
  int dim = 0;
  struct Param {
    UDFType udf_type = kSum;
    TruncDirection trunc_direction = kReverse;
    int trunc_num = 0;
  };
  std::vector<Param> in_item;
};
struct SparsePullerOutput {
  struct OutItem {
    void* out = nullptr;
    size_t stride = 0;
  };
  std::vector<OutItem> out_item;
};

class SparsePuller {
 public:
  virtual ~SparsePuller() {}
  virtual Status Load(const std::string& url) { return kFail; }
  virtual Status Get(const std::vector<SparsePullerInput>& input, std::vector<SparsePullerOutput>& output) {
    return kFail;
  }
  // Device-side pooling of all groups of one Embedding operator in one call.
  virtual Status GetAsync(const std::vector<SparsePullerInput>& input, std::vector<SparsePullerOutput>& output,
                          int device_id, cudaStream_t stream, int* launches) {
    return kFail;
  }
  // In-memory registration (host fp32 rows, optional int64 keys).
  virtual Status AddTable(const std::string& name, int64_t rows, int dim, int storage_dtype, const float* w,
                          const int64_t* keys) {
    return kFail;
  }
  // A device-resident shard registered without a host copy (row-sharded tables are generated or loaded shard by
  // shard): `rows` local rows of `dim` elements at `device_weights`, `pitch_bytes` apart, identity keys.
  virtual Status AddDeviceShard(const std::string& name, int64_t rows, int dim, int storage_dtype, const void* device_weights,
                                int64_t pitch_bytes) {
    return kFail;
  }
  // Row-sharded pullers: this process is shard `rank` of `world`; `unique_id` (128 bytes, xb_shard_unique_id) is the
  // same on every rank. Tables registered afterwards are this rank's shards (row r of the table lives on rank
  // r % world at local row r / world).
  virtual Status InitSharded(int rank, int world, const void* unique_id, int64_t max_ids_per_step, int partial_dtype,
                             float capacity_factor) {
    return kFail;
  }
};

using FCreateSparsePuller = std::function<SparsePuller*(void)>;
struct SparsePullerCreationRegisterer {
  static SparsePullerCreationRegisterer* Get();
  bool Register(const std::string& name, FCreateSparsePuller fcs);
  SparsePuller* CreateSparsePuller(const std::string& name);
  std::unordered_map<std::string, FCreateSparsePuller> fcs_map_;
};
#define REGISTER_SPARSE_PULLER_CREATION(name, fcs) \
  static bool status = ::blaze::store::SparsePullerCreationRegisterer::Get()->Register(name, fcs);
}  // namespace store

// ---- Workspace --------------------------------------------------------------------------------
class Net;
// Constants (ConstantFill outputs) are shared by all predictors of one device.
struct ConstantStore {
  std::mutex mu;
  std::unordered_map<std::string, std::shared_ptr<Blob>> blobs;
};

class Workspace {
 public:
  Workspace() {}
  void Init(const NetDef& def) { net_def_ = def; }
  const NetDef& net_def() const { return net_def_; }
  Blob* CreateBlob(const std::string& name, const DeviceOption& opt);
  // A blob owned by the per-device constant store; *fresh tells the caller to fill it.
  Blob* CreateConstantBlob(const std::string& name, const DeviceOption& opt, bool* fresh);
  Blob* GetBlob(const std::string& name) const;
  bool HasBlob(const std::string& name) const { return GetBlob(name) != nullptr; }
  void SetSparsePuller(std::shared_ptr<store::SparsePuller> p) { puller_ = p; }
  std::shared_ptr<store::SparsePuller> GetSparsePuller() const { return puller_; }
  void SetConstantStore(std::shared_ptr<ConstantStore> s) { constants_ = s; }
  std::unique_ptr<Net> CreateNet();
  std::vector<std::string> BlobNames() const;

 private:
  NetDef net_def_;
  std::unordered_map<std::string, std::unique_ptr<Blob>> blobs_;
  std::unordered_map<std::string, std::shared_ptr<Blob>> shared_;
  std::shared_ptr<store::SparsePuller> puller_;
  std::shared_ptr<ConstantStore> constants_;
};

// ---- operators --------------------------------------------------------------------------------
class OperatorBase {
 public:
  OperatorBase(const OperatorDef& def, Workspace* ws);
  virtual ~OperatorBase() {}
  virtual bool Run(int stream_id = 0) = 0;
  const OperatorDef& operator_def() const { return def_; }
  size_t InputSize() const { return inputs_.size(); }
  size_t OutputSize() const { return outputs_.size(); }
  Blob* Input(size_t i) const { return inputs_.at(i); }
  Blob* Output(size_t i) const { return outputs_.at(i); }
  bool HasArgument(const std::string& name) const { return def_.FindArg(name) != nullptr; }
  template <typename T>
  T GetSingleArgument(const std::string& name, const T& def) const;
  template <typename T>
  std::vector<T> GetRepeatedArgument(const std::string& name) const;
  int launches = 0;             // kernel-library calls made by the last Run
  bool constant_fresh = true;   // ConstantFill: this operator has to fill the (shared) output blob

 protected:
  OperatorDef def_;
  DeviceOption device_option_;
  Workspace* workspace_;
  std::vector<Blob*> inputs_, outputs_;
};

template <class Context>
class Operator : public OperatorBase {
 public:
  Operator(const OperatorDef& def, Workspace* ws) : OperatorBase(def, ws), context_(device_option_) {}
  bool Run(int stream_id = 0) final {
    context_.Activate();
    launches = 0;
    return RunOnDevice();
  }
  virtual bool RunOnDevice() = 0;
  Context* context() { return &context_; }

 protected:
  Context context_;
};

#define USE_OPERATOR_FUNCTIONS(Context)        \
  using OperatorBase::Input;                   \
  using OperatorBase::Output;                  \
  using OperatorBase::InputSize;               \
  using OperatorBase::OutputSize;              \
  using Operator<Context>::context_

typedef std::function<std::unique_ptr<OperatorBase>(const OperatorDef&, Workspace*)> OperatorCreator;
class OperatorRegistry {
 public:
  // At most one registration per name: a second one throws, as Blaze's Registry does.
  void Register(const std::string& name, OperatorCreator c);
  bool Has(const std::string& name) const { return map_.count(name) != 0; }
  std::unique_ptr<OperatorBase> Create(const std::string& name, const OperatorDef& def, Workspace* ws) const;
  std::vector<std::string> Names() const;

 private:
  std::unordered_map<std::string, OperatorCreator> map_;
};
OperatorRegistry* CUDAOperatorRegistry();
OperatorRegistry* CPUOperatorRegistry();

struct OperatorRegisterer {
  OperatorRegisterer(OperatorRegistry* r, const std::string& name, OperatorCreator c) { r->Register(name, c); }
};
#define BLAZE_CONCAT_(a, b) a##b
#define BLAZE_CONCAT(a, b) BLAZE_CONCAT_(a, b)
#define REGISTER_CUDA_OPERATOR(name, ...)                                                             \
  static ::blaze::OperatorRegisterer BLAZE_CONCAT(g_cuda_op_reg_, __COUNTER__)(                       \
      ::blaze::CUDAOperatorRegistry(), #name, [](const ::blaze::OperatorDef& d, ::blaze::Workspace* w) { \
        return std::unique_ptr<::blaze::OperatorBase>(new __VA_ARGS__(d, w));                         \
      })

// Schema: input/output count limits checked when an operator is created.
struct OpSchema {
  int min_in = 0, max_in = 1 << 20, min_out = 0, max_out = 1 << 20;
  OpSchema& NumInputs(int n) { min_in = max_in = n; return *this; }
  OpSchema& NumInputs(int lo, int hi) { min_in = lo; max_in = hi; return *this; }
  OpSchema& NumOutputs(int n) { min_out = max_out = n; return *this; }
  OpSchema& NumOutputs(int lo, int hi) { min_out = lo; max_out = hi; return *this; }
};
OpSchema& RegisterSchema(const std::string& name);
const OpSchema* FindSchema(const std::string& name);
#define OPERATOR_SCHEMA(name) \
  static ::blaze::OpSchema& BLAZE_CONCAT(g_schema_, __COUNTER__) = ::blaze::RegisterSchema(#name)

std::unique_ptr<OperatorBase> CreateOperator(const OperatorDef& def, Workspace* ws);

// ---- nets -------------------------------------------------------------------------------------
class Net {
 public:
  Net(const NetDef& def, Workspace* ws);
  virtual ~Net() {}
  bool Run();
  const std::vector<std::string>& external_input() const { return ext_in_; }
  const std::vector<std::string>& external_output() const { return ext_out_; }
  const NetDef& net_def() const { return def_; }
  Workspace* workspace() { return ws_; }
  cudaStream_t stream() const;
  int device_id() const { return def_.device_option.device_id; }
  // After the stream was synchronised: throws when a bounded wait inside a tensor-core kernel of this
  // device ran out since the last check (the outputs of that run are not to be trusted), naming the
  // site, and clears the device's status word so that later runs wait with their full limits again.
  void CheckDeviceStatus();
  int last_launches = 0;
  // per-operator wall time of the last Run when profiling is on (observer "profile")
  bool profile = false;
  std::vector<std::pair<std::string, float>> op_ms;

 protected:
  NetDef def_;
  Workspace* ws_;
  std::vector<std::unique_ptr<OperatorBase>> ops_;
  std::vector<std::string> ext_in_, ext_out_;
  const volatile int* status_word_ = nullptr;   // host-mapped mirror of the device's status word
};

// Graph rewrite run by LoadModel(optimization_pass = true): folds Dice / PRelu / Sigmoid nodes
// into the producing Gemm's epilogue when the Gemm output has no other consumer.
void FuseGemmActivation(NetDef* def);
// Run before it: folds a BatchNormalization with constant parameters into the weight and bias of the Gemm it
// feeds or follows (constants re-computed in fp32), so the node disappears from the graph.
void FoldBatchNorm(NetDef* def);
// Run between the two: recognises the op-by-op attention unit (Sub, Mul, BroadcastTo x2, Concat, three Gemm layers
// with their activations, Reshape, MatMul, Reshape) and the op-by-op tower (ReduceSum, Mul, Sub, BroadcastTo,
// Concat, Fuse, Gemm + Dice x2, Gemm, Softmax) of an fp16 DIN-style graph and replaces them by DinAttention and
// DinTower. Returns the number of sub-graphs replaced.
int FuseDinSubgraphs(NetDef* def);

// fp32 <-> fp16 on the host (round to nearest even)
uint16_t FloatToHalfBits(float f);
float HalfBitsToFloat(uint16_t h);

}  // namespace blaze
