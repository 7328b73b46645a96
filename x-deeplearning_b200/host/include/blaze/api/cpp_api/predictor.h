// Public C++ API of the B200 host runtime.
//
// Same enums, class names, method names, argument meaning and return
// conventions as Blaze's installed header blaze/blaze/api/cpp_api/predictor.h
// (Predictor :92-215, PredictorManager :217-275, InitScheduler :281-286), so
// code written against Blaze compiles and runs against this library unchanged.
// Differences are confined to what is behind the interface: models are Blaze
// NetDefs (binary or text protobuf), operators run on sm_100a kernels.
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace blaze {

class PredictorImpl;
class PredictorManagerImpl;

enum PredictDeviceType { kPDT_Unkown = -1, kPDT_CPU, kPDT_CUDA };
enum PredictDataType { kPDT_Invalid = -1, kPDT_Float = 1, kPDT_Float16 = 12 };
enum ModelType { kBlaze = 0, kUlf, kOnnx, kMxnet, kTensorFlow, kXDL, kXDLUlf };
enum FeatureType { kDenseFeature = 0, kSparseFeature, kAuxIndicator };
enum SparseFeatureType { kSparseFeatureId = 0, kSparseFeatureValue, kAuxSparseFeatureSegment };

struct FeedNameConfig {
  std::string feature_name;
  FeatureType feature_type;
  int level;                                   // indicator level
  SparseFeatureType sparse_feature_type;
};

class FeedNameUtility {
 public:
  // "<feature>.ids" / ".values" / ".segments"
  static std::string SparseFeatureName2FeedName(const std::string& sparse_feature_name, SparseFeatureType sft);
  // "indicator.<level>"
  static std::string IndicatorLevel2FeedName(int level);
};

using PredictorCallback = std::function<void()>;

// Not thread safe: one Predictor per serving thread.
class Predictor {
 public:
  virtual ~Predictor();

  FeedNameConfig GetFeedNameConfig(const std::string& feed_name);
  bool ReshapeInput(const char* name, const std::vector<size_t>& shape);
  bool ReshapeInput(size_t idx, const std::vector<size_t>& shape);
  // `data` is host memory of `len` bytes; it is copied to the device.
  bool Feed(const char* name, const void* data, size_t len);
  bool Feed(size_t idx, const void* data, size_t len);

  size_t InputSize() const;
  PredictDataType InputDataType(const char* name) const;
  PredictDataType InputDataType(size_t idx) const;
  const std::vector<std::string>& ListInputName() const;

  bool Forward(const PredictorCallback&& cb = nullptr);

  // *data points at a host copy owned by the predictor, valid until the next call.
  bool Output(const char* name, void** data, size_t* len);
  bool Output(size_t idx, void** data, size_t* len);
  const std::vector<size_t>& OutputShape(size_t idx) const;
  const std::vector<size_t>& OutputShape(const char* name) const;
  PredictDataType OutputDataType(size_t idx) const;
  PredictDataType OutputDataType(const char* name) const;
  size_t OutputSize() const;
  const std::vector<std::string>& ListOutputName() const;

  std::vector<std::string> ListInternalName() const;
  bool InternalParam(const char* name, void** data, size_t* len);
  const std::vector<size_t>& InternalShape(const char* name) const;
  int InternalDataType(const char* name) const;

  void RegisterObservers(const std::vector<std::string>& oberver_names);
  void DumpObservers(std::unordered_map<std::string, std::string>* dump_map);

 protected:
  explicit Predictor(PredictorImpl* impl);
  PredictorImpl* impl_;
  friend class PredictorManagerImpl;
};

class PredictorManager {
 public:
  PredictorManager();
  virtual ~PredictorManager();

  void SetDataType(PredictDataType data_type);
  void SetRunMode(const char* run_mode);
  // type "qed_sparse_puller" loads a QED file into HBM; "mock_sparse_puller" needs no file.
  bool LoadSparseModelWeight(const char* uri, const char* type = "qed_sparse_puller");
  bool LoadModel(const char* filename, bool optimization_pass = true);
  bool LoadDeepNetModel(const char* model_conf, const char* model_data, bool optimization_pass = true);
  bool LoadModel(const char* conf_file, const char* data_file, ModelType model_type, bool optimization_pass = true);
  // The caller owns the returned predictor.
  Predictor* CreatePredictor(PredictDeviceType predict_device_type = kPDT_Unkown, int device_id = 0);

 protected:
  PredictorManagerImpl* impl_;
  friend struct ManagerAccess;
};

bool InitScheduler(bool enable_batching, int max_batch_size, int batch_timeout_micros, int num_threads_for_cpu,
                   int num_threads_for_cuda, int num_threads_for_pipe);

}  // namespace blaze
