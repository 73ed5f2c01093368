#include "core/step.h"

#include <algorithm>
#include <iomanip>
#include <numeric>

namespace kvx {

void Step::update_last_send_finish_ts(Timepoint t) noexcept {
  const int64_t v = t.time_since_epoch().count();
  int64_t cur = last_send_finish_.load(std::memory_order_relaxed);
  while (cur < v && !last_send_finish_.compare_exchange_weak(cur, v, std::memory_order_relaxed)) {
  }
}

Step::~Step() {
  // Destruction means every sender holding the step has finished: emit the step metrics line
  // (key names are part of the ops-script contract of the reference, step.cpp:29-39).
  if (sub_queue_time_us.empty()) return;
  const auto mn = *std::min_element(sub_queue_time_us.begin(), sub_queue_time_us.end());
  const auto mx = *std::max_element(sub_queue_time_us.begin(), sub_queue_time_us.end());
  const auto avg = std::accumulate(sub_queue_time_us.begin(), sub_queue_time_us.end(), int64_t{0}) /
                   static_cast<int64_t>(sub_queue_time_us.size());
  const Timepoint last = last_send_finish_ts();
  LOG(INFO) << "StepMetrics. StepIdx=" << step_idx << ",SubstepCnt=" << sub_queue_time_us.size()
            << ",SubQueueMinUs=" << mn << ",SubQueueMaxUs=" << mx << ",SubQueueAvgUs=" << avg
            << ",PythonExecUs=" << elapse_us(start_send_ts, flush_send_ts)
            << ",WaitLayerQueueUs=" << elapse_us(start_send_ts, wait_layers_start_ts)
            << ",ForwardExecUs=" << elapse_us(wait_layers_start_ts, wait_layers_end_ts)
            << ",SendNonoverlapUs=" << elapse_us(wait_layers_end_ts, last)
            << ",LastSendFlushTs=" << last.time_since_epoch().count();
}

StepGuard::StepGuard(uint32_t layers, ICudaBarrier* barrier, std::shared_ptr<Step> step)
    : num_layers(layers), step_(std::move(step)), barrier_(barrier) {
  RTASSERT(barrier_ != nullptr);
  RTASSERT(step_ != nullptr);
}

StepGuard::StepGuard(Context* ctx, std::shared_ptr<Step> step)
    : StepGuard(ctx->num_layers(), ctx->cuda_barrier(), std::move(step)) {}

void StepGuard::wait_layers() {
  uint32_t val = step_->notify_layer_ready(0);
  if (val > 0) return;  // a frozen step: born with every layer ready
  for (uint32_t layer = 0; layer < num_layers; ++layer) {
    step_->wait_layer_recorded(layer);
    barrier_->wait(layer);
    val = step_->notify_layer_ready(layer + 1);
    if (val > layer + 1) return;
  }
}

void StepGuard::after_record_one() { step_->notify_one_recorded(); }
void StepGuard::after_record_all() { step_->notify_layer_recorded(num_layers); }
void StepGuard::layer_ready_all() { after_record_all(); }

}  // namespace kvx
