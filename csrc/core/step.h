// Layer-ready pipeline of one engine step.
//
// A Step carries two monotone counters that sender threads block on:
//   recorded(i): the engine has *recorded* the CUDA event of layer i on its forward stream
//                (host-side fact).  A device transport may now order its own stream after
//                that event and enqueue the layer's transfer without any host wait.
//   ready(i):    the event of layer i has *completed* (the KV bytes exist).  Host-driven
//                transports (TCP, shared memory) wait for this before they read the cache.
// StepGuard is the engine-side handle: the forward thread calls after_record_one() per layer,
// a wait-layers thread turns completed events into ready(i).  Same protocol as the
// reference's Step/StepGuard (kvtransfer/src/step.cpp:42-81), plus the recorded counter.
#pragma once
#include <atomic>
#include <memory>
#include <vector>

#include "core/context.h"
#include "core/util.h"

namespace kvx {

class Step {
 public:
  const size_t step_idx;
  const Timepoint start_send_ts = SteadyClock::now();
  std::vector<int64_t> sub_queue_time_us;  // written by the target-manager thread
  Timepoint flush_send_ts;                 // written by the engine thread
  Timepoint wait_layers_start_ts;          // written by the wait-layers thread
  Timepoint wait_layers_end_ts;
  bool frozen = false;                     // born with every layer complete (freeze / migration steps)

  explicit Step(size_t idx) : step_idx(idx) {}
  ~Step();

  void wait_layer_ready(uint32_t layer) { data_signal_.wait(layer); }
  bool wait_layer_ready_for(uint32_t layer, std::chrono::milliseconds d) { return data_signal_.wait_for(layer, d); }
  uint32_t notify_layer_ready(uint32_t layers_done) { return data_signal_.release(layers_done); }
  void wait_layer_recorded(uint32_t layer) { record_signal_.wait(layer); }
  uint32_t notify_layer_recorded(uint32_t layers_recorded) { return record_signal_.release(layers_recorded); }
  void notify_one_recorded() { record_signal_.release(); }
  uint32_t layers_recorded() { return record_signal_.value(); }

  Timepoint last_send_finish_ts() const noexcept { return Timepoint(SteadyClock::duration(last_send_finish_.load())); }
  void update_last_send_finish_ts(Timepoint t) noexcept;

 private:
  SyncSemaphore data_signal_;
  SyncSemaphore record_signal_;
  std::atomic<int64_t> last_send_finish_{0};
};

class StepGuard {
 public:
  const uint32_t num_layers;
  StepGuard(uint32_t layers, ICudaBarrier* barrier, std::shared_ptr<Step> step);
  StepGuard(Context* ctx, std::shared_ptr<Step> step);

  size_t step_id() const { return step_->step_idx; }
  std::shared_ptr<Step>& step() { return step_; }
  void wait_layers();        // runs on the wait-layers thread
  void after_record_one();   // engine thread: one more layer event recorded
  void after_record_all();
  void layer_ready_all();    // flush: everything recorded (events still gate readiness)

 private:
  std::shared_ptr<Step> step_;
  ICudaBarrier* barrier_;
};

}  // namespace kvx
