// Request batching: concurrent Forward(cb) calls on predictors of one model and device are stacked
// into one run of a merged net.
//
// The reference does this in blaze/blaze/graph/hybrid_net.cc:118-176 (queue per NetDef, merge, run
// the first net, split, call every task's callback), blaze/blaze/scheduler/batching.cc:131-191
// (Merge: concatenate every external input along dim 0; Split: hand each task its rows of every
// external output) and blaze/blaze/batching/shared_batch_scheduler.h (a batch closes when it holds
// max_batch_size tasks or batch_timeout_micros after its first task arrived). Here the queue owns a
// net of its own whose operators run on the batch thread's stream; inputs are stacked and outputs
// handed back with device-to-device copies on that stream, ordered after the submitters' feeds by
// an event per task.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "runtime.h"

namespace blaze {

// What InitScheduler was given (blaze/blaze/scheduler/scheduler_manager.h:32-51).
struct SchedulerOptions {
  bool enable_batching = false;
  int max_batch_size = 100;          // tasks per batch
  int batch_timeout_micros = 100;    // a batch closes this long after its first task arrived
  int max_enqueued_batches = 500;    // Schedule refuses once this many full batches are waiting
};
SchedulerOptions& GlobalSchedulerOptions();

struct BatchingStats {
  std::atomic<int64_t> batches{0};   // merged runs
  std::atomic<int64_t> tasks{0};     // tasks those runs carried
};
BatchingStats& GlobalBatchingStats();

class BatchQueue {
 public:
  struct Task {
    Workspace* ws = nullptr;                                   // the submitting predictor's blobs
    cudaEvent_t ready = nullptr;                               // recorded after its feeds
    std::function<void(const std::string& error)> done;        // error empty: outputs are in ws
    std::chrono::steady_clock::time_point enqueued;
    // first dimensions of the inputs that are one row per sample (everything but id / value lists),
    // followed by each input's trailing dimensions and data type: tasks stack only when these agree
    std::vector<TIndex> rows;
    std::vector<TIndex> rest;
    // The net declares an indicator input (input_type kInputIndicator, blaze/blaze/proto/blaze.proto:66-72): its
    // values are row numbers that stacking would have to shift (structured_batching.cc:49-60). No operator of
    // this runtime reads indicators, so such a request is run on its own instead of being rewritten.
    bool solo = false;
  };

  BatchQueue(const NetDef& def, std::shared_ptr<store::SparsePuller> puller, std::shared_ptr<ConstantStore> constants,
             const SchedulerOptions& options);
  ~BatchQueue();
  BatchQueue(const BatchQueue&) = delete;
  BatchQueue& operator=(const BatchQueue&) = delete;

  // Takes the task's event. False (task untouched) when the queue is full.
  bool Schedule(Task* task, std::string* why);

  // Which tasks of `queue` (positions, first one always 0) run together with its head: those whose
  // row counts are proportional to the head's and whose trailing shapes agree, at most `max_tasks`.
  static std::vector<size_t> PickBatch(const std::deque<Task>& queue, size_t max_tasks);
  // Fills rows / rest of a task from the workspace's external inputs.
  static void Describe(const NetDef& def, Task* task);

 private:
  void Loop();
  void RunBatch(std::vector<Task>* batch);
  void MergeInputs(const std::vector<Task>& batch, cudaStream_t stream);
  void SplitOutputs(const std::vector<Task>& batch, cudaStream_t stream);
  // All copies of a merge (or split) step go out as one descriptor table and one kernel launch
  // (xb_copy_segments) instead of one cudaMemcpyAsync per blob and request.
  void AddCopy(const void* src, void* dst, size_t bytes);
  void FlushCopies(cudaStream_t stream);
  struct CopyTable;

  NetDef def_;
  std::shared_ptr<store::SparsePuller> puller_;
  std::shared_ptr<ConstantStore> constants_;
  SchedulerOptions options_;
  std::unique_ptr<CopyTable> copies_;
  std::unique_ptr<Workspace> ws_;       // created and destroyed on the batch thread
  std::unique_ptr<Net> net_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Task> queue_;
  bool stop_ = false;
  std::thread thread_;
};

}  // namespace blaze
