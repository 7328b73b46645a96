// Request batching for the predictor API: queue, merge, run, split (see batching.h).
#include "batching.h"

#include <algorithm>
#include <cstring>

namespace blaze {

SchedulerOptions& GlobalSchedulerOptions() {
  static SchedulerOptions options;
  return options;
}

BatchingStats& GlobalBatchingStats() {
  static BatchingStats stats;
  return stats;
}

namespace {
bool EndsWith(const std::string& s, const char* suffix) {
  const size_t n = strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}
// Id and value lists have one entry per id, not per sample: their lengths say nothing about how many
// samples a task carries.
bool IsRagged(const std::string& input_name) { return EndsWith(input_name, ".ids") || EndsWith(input_name, ".values"); }
}  // namespace

void BatchQueue::Describe(const NetDef& def, Task* task) {
  task->rows.clear();
  task->rest.clear();
  task->solo = false;
  for (const auto& v : def.external_input) {
    if (v.input_type == 4) task->solo = true;          // kInputIndicator
    const Blob* b = task->ws->GetBlob(v.name);
    BLAZE_CONDITION_THROW(b != nullptr, "input ", v.name, " does not exist");
    const auto& shape = b->shape();
    if (!IsRagged(v.name)) task->rows.push_back(shape.empty() ? 1 : shape[0]);
    task->rest.push_back(shape.size());
    for (size_t i = 1; i < shape.size(); ++i) task->rest.push_back(shape[i]);
    task->rest.push_back((TIndex)b->data_type());
  }
}

std::vector<size_t> BatchQueue::PickBatch(const std::deque<Task>& queue, size_t max_tasks) {
  std::vector<size_t> picked;
  if (queue.empty() || max_tasks == 0) return picked;
  picked.push_back(0);
  const Task& head = queue[0];
  if (head.solo) return picked;
  size_t pivot = head.rows.size();
  for (size_t j = 0; j < head.rows.size(); ++j)
    if (head.rows[j] > 0) { pivot = j; break; }
  for (size_t i = 1; i < queue.size() && picked.size() < max_tasks; ++i) {
    const Task& t = queue[i];
    if (t.solo || t.rest != head.rest || t.rows.size() != head.rows.size()) continue;
    bool same = true;
    for (size_t j = 0; j < head.rows.size() && same; ++j) {
      if (pivot == head.rows.size()) same = t.rows[j] == 0;
      else same = t.rows[j] * head.rows[pivot] == head.rows[j] * t.rows[pivot];
    }
    if (same && pivot != head.rows.size() && t.rows[pivot] == 0) same = false;   // an empty task against a non-empty head
    if (same) picked.push_back(i);
  }
  return picked;
}

// Descriptor table of one merge or split step: filled in pinned host memory, copied to the device on the
// batch stream, consumed by one kernel. The two halves alternate so that the split step's table does not
// overwrite the merge step's while its copy may still be in flight.
struct BatchQueue::CopyTable {
  std::vector<xb_copy_item> items;
  xb_copy_item* host[2] = {nullptr, nullptr};
  xb_copy_item* device[2] = {nullptr, nullptr};
  size_t capacity[2] = {0, 0};
  int turn = 0;
  int64_t max_bytes = 0;
  ~CopyTable() {
    for (int i = 0; i < 2; ++i) {
      if (host[i]) cudaFreeHost(host[i]);
      if (device[i]) cudaFree(device[i]);
    }
  }
};

void BatchQueue::AddCopy(const void* src, void* dst, size_t bytes) {
  if (bytes == 0) return;
  xb_copy_item it;
  it.src = src; it.dst = dst; it.bytes = (int64_t)bytes;
  copies_->items.push_back(it);
  copies_->max_bytes = std::max<int64_t>(copies_->max_bytes, (int64_t)bytes);
}

void BatchQueue::FlushCopies(cudaStream_t stream) {
  CopyTable& c = *copies_;
  const size_t n = c.items.size();
  if (n == 0) return;
  const int h = c.turn;
  c.turn ^= 1;
  if (c.capacity[h] < n) {
    // the stream is idle or only runs work of this batch that does not read the old table any more
    CUDA_CHECK(cudaStreamSynchronize(stream));
    if (c.host[h]) cudaFreeHost(c.host[h]);
    if (c.device[h]) cudaFree(c.device[h]);
    c.host[h] = nullptr; c.device[h] = nullptr; c.capacity[h] = 0;
    const size_t cap = std::max<size_t>(2 * n, 256);
    CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&c.host[h]), cap * sizeof(xb_copy_item)));
    CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&c.device[h]), cap * sizeof(xb_copy_item)));
    c.capacity[h] = cap;
  }
  memcpy(c.host[h], c.items.data(), n * sizeof(xb_copy_item));
  CUDA_CHECK(cudaMemcpyAsync(c.device[h], c.host[h], n * sizeof(xb_copy_item), cudaMemcpyHostToDevice, stream));
  BLAZE_CONDITION_THROW(xb_copy_segments(c.device[h], (int32_t)n, c.max_bytes, stream) == 0, xb_last_error());
  c.items.clear();
  c.max_bytes = 0;
}

BatchQueue::BatchQueue(const NetDef& def, std::shared_ptr<store::SparsePuller> puller,
                       std::shared_ptr<ConstantStore> constants, const SchedulerOptions& options)
    : def_(def), puller_(puller), constants_(constants), options_(options), copies_(new CopyTable()) {
  if (options_.max_batch_size < 1) options_.max_batch_size = 1;
  if (options_.batch_timeout_micros < 0) options_.batch_timeout_micros = 0;
  if (options_.max_enqueued_batches < 1) options_.max_enqueued_batches = 1;
  thread_ = std::thread([this] { Loop(); });
}

BatchQueue::~BatchQueue() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

bool BatchQueue::Schedule(Task* task, std::string* why) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    if (stop_) { *why = "the batch queue is shutting down"; return false; }
    if (queue_.size() >= (size_t)options_.max_enqueued_batches * (size_t)options_.max_batch_size) {
      *why = "the batch queue is full";
      return false;
    }
    task->enqueued = std::chrono::steady_clock::now();
    queue_.push_back(std::move(*task));
  }
  cv_.notify_all();
  return true;
}

void BatchQueue::Loop() {
  for (;;) {
    std::vector<Task> batch;
    {
      std::unique_lock<std::mutex> lock(mu_);
      cv_.wait(lock, [this] { return stop_ || !queue_.empty(); });
      if (queue_.empty()) break;                       // stop requested and nothing left to run
      const auto deadline = queue_.front().enqueued + std::chrono::microseconds(options_.batch_timeout_micros);
      cv_.wait_until(lock, deadline, [this] { return stop_ || queue_.size() >= (size_t)options_.max_batch_size; });
      const std::vector<size_t> picked = PickBatch(queue_, (size_t)options_.max_batch_size);
      for (size_t i : picked) batch.push_back(std::move(queue_[i]));
      for (size_t k = picked.size(); k-- > 0;) queue_.erase(queue_.begin() + picked[k]);
    }
    RunBatch(&batch);
  }
  // the merged net's operators and blobs belong to this thread's stream: release them here
  net_.reset();
  ws_.reset();
  copies_.reset();
}

void BatchQueue::MergeInputs(const std::vector<Task>& batch, cudaStream_t stream) {
  for (const auto& v : def_.external_input) {
    Blob* dst = ws_->GetBlob(v.name);
    BLAZE_CONDITION_THROW(dst != nullptr, "merged net has no input ", v.name);
    const Blob* first = batch[0].ws->GetBlob(v.name);
    std::vector<TIndex> shape = first->shape();
    dst->set_data_type(first->data_type());
    if (shape.empty()) {                               // a scalar cannot be stacked: the head's value stands
      dst->Reshape(shape);
      AddCopy(first->as<void>(), dst->as<void>(), first->bytes());
      continue;
    }
    TIndex total = 0;
    for (const auto& t : batch) total += t.ws->GetBlob(v.name)->shape()[0];
    shape[0] = total;
    dst->Reshape(shape);
    size_t offset = 0;
    for (const auto& t : batch) {
      const Blob* src = t.ws->GetBlob(v.name);
      AddCopy(src->as<void>(), dst->as<char>() + offset, src->bytes());
      offset += src->bytes();
    }
  }
  FlushCopies(stream);
}

void BatchQueue::SplitOutputs(const std::vector<Task>& batch, cudaStream_t stream) {
  for (const auto& o : def_.external_output) {
    const Blob* src = ws_->GetBlob(o.name);
    BLAZE_CONDITION_THROW(src != nullptr && !src->shape().empty(), "merged net has no output ", o.name);
    const TIndex total = src->shape()[0];
    // an output row belongs to the task that fed the matching input row: the input whose stacked
    // first dimension equals the output's says how many rows each task gets (per-sample inputs first)
    const std::string* by = nullptr;
    for (int ragged = 0; ragged < 2 && !by; ++ragged) {
      for (const auto& v : def_.external_input) {
        if (IsRagged(v.name) != (ragged == 1)) continue;
        TIndex sum = 0;
        bool stackable = true;
        for (const auto& t : batch) {
          const auto& s = t.ws->GetBlob(v.name)->shape();
          if (s.empty()) { stackable = false; break; }
          sum += s[0];
        }
        if (stackable && sum == total) { by = &v.name; break; }
      }
    }
    BLAZE_CONDITION_THROW(by != nullptr, "output ", o.name, " has ", total,
                          " rows, which no input's stacked first dimension matches: its rows cannot be split");
    const size_t row_bytes = total ? src->bytes() / total : 0;
    size_t offset = 0;
    for (const auto& t : batch) {
      Blob* dst = t.ws->GetBlob(o.name);
      BLAZE_CONDITION_THROW(dst != nullptr, "predictor has no output ", o.name);
      std::vector<TIndex> shape = src->shape();
      shape[0] = t.ws->GetBlob(*by)->shape()[0];
      dst->set_data_type(src->data_type());
      dst->Reshape(shape);
      const size_t n = row_bytes * shape[0];
      AddCopy(src->as<char>() + offset, dst->as<void>(), n);
      offset += n;
    }
  }
  FlushCopies(stream);
}

void BatchQueue::RunBatch(std::vector<Task>* batch) {
  std::string error;
  cudaStream_t stream = nullptr;
  try {
    CUDA_CHECK(cudaSetDevice(def_.device_option.device_id));
    if (!net_) {
      ws_.reset(new Workspace());
      ws_->Init(def_);
      ws_->SetSparsePuller(puller_);
      ws_->SetConstantStore(constants_);
      net_ = ws_->CreateNet();
    }
    stream = net_->stream();
    for (const auto& t : *batch) CUDA_CHECK(cudaStreamWaitEvent(stream, t.ready, 0));
    MergeInputs(*batch, stream);
    BLAZE_CONDITION_THROW(net_->Run(), "the merged net did not run");
    SplitOutputs(*batch, stream);
    CUDA_CHECK(cudaStreamSynchronize(stream));
    net_->CheckDeviceStatus();
    GlobalBatchingStats().batches += 1;
    GlobalBatchingStats().tasks += (int64_t)batch->size();
  } catch (const std::exception& e) {
    error = MakeString("batched forward failed: ", e.what());
    LOG_ERROR(error);
    if (stream) cudaStreamSynchronize(stream);
    if (copies_) { copies_->items.clear(); copies_->max_bytes = 0; }
  }
  for (auto& t : *batch) {
    if (t.ready) cudaEventDestroy(t.ready);
    t.ready = nullptr;
    if (t.done) t.done(error);
  }
}

}  // namespace blaze
