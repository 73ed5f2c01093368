#include "core/client.h"

#include "core/envcfg.h"
#include "core/fault_inject.h"

namespace kvx {

// ---- TargetMgr ---------------------------------------------------------------------------------
KvTransferClient::TargetMgr::TargetMgr(Context* ctx, std::unique_ptr<ISendStubFactory> f)
    : ctx_(ctx), factory_(std::move(f)),
      send_pool_(std::make_unique<ThreadPool>(static_cast<size_t>(env_send_tpsize()), "clisend")),
      mgr_thd_(std::make_unique<ThreadPool>(1, "kvtmgr")) {}

KvTransferClient::TargetMgr::~TargetMgr() {
  mgr_thd_.reset();   // no new batches reach the sender pool
  send_pool_.reset(); // finish what is queued
}

void KvTransferClient::TargetMgr::submit(std::shared_ptr<Step> step, StepTasks tasks) {
  // counted here, on the caller's thread, so that a caller that asks "how far am I ahead" right after
  // submitting already sees these batches
  uint64_t n = 0;
  for (auto& [inst, per_worker] : tasks.tasks)
    for (auto& [wid, batch] : per_worker)
      if (!batch.tasks.empty()) {
        batch.inflight = &ctx_->inflight();
        ++n;
      }
  ctx_->inflight().add(n);
  auto shared_tasks = std::make_shared<StepTasks>(std::move(tasks));
  mgr_thd_->spawn([this, step = std::move(step), shared_tasks]() mutable { do_submit(step, *shared_tasks); });
}

void KvTransferClient::TargetMgr::drain() {
  mgr_thd_->drain();
  send_pool_->drain();
  // batches that complete on a device: every one of them is bounded by its own deadline
  ctx_->inflight().wait_at_most(0, std::chrono::milliseconds(env_completion_timeout_ms() + 2000));
}

void KvTransferClient::TargetMgr::shrink_sync(size_t cap) {
  mgr_thd_->spawn([this, cap] { shrink(cap); });
  mgr_thd_->drain();
}

KvTransferClient::Target* KvTransferClient::TargetMgr::get_or_create(const RequestInfo& req) {
  auto& slots = index_[req.dst_inst_id];
  if (req.dst_worker_id < slots.size() && slots[req.dst_worker_id].has_value()) {
    Iter it = *slots[req.dst_worker_id];
    targets_.splice(targets_.begin(), targets_, it);  // touch
    return &*it;
  }
  SendStub stub = factory_->create_stub(req.dst_inst_id, req.dst_worker_id, 0, ctx_->num_layers(), std::nullopt,
                                        req.dst_worker_info);
  targets_.emplace_front(std::move(stub));
  if (req.dst_worker_id >= slots.size()) slots.resize(req.dst_worker_id + 1);
  slots[req.dst_worker_id] = targets_.begin();
  n_targets_.store(targets_.size());
  LOG(INFO) << "TargetMgr.create: instid=" << req.dst_inst_id << " wid=" << req.dst_worker_id << " worker_info="
            << (req.dst_worker_info ? req.dst_worker_info->to_string() : std::string("NULL"));
  return &targets_.front();
}

void KvTransferClient::TargetMgr::do_submit(std::shared_ptr<Step>& step, StepTasks& st) {
  const auto submit_ts = SteadyClock::now();
  step->sub_queue_time_us.push_back(elapse_us(st.send_ts, submit_ts));
  for (auto& [inst, per_worker] : st.tasks) {
    for (auto& [wid, batch] : per_worker) {
      if (batch.tasks.empty()) continue;
      batch.step = step;
      batch.substepid = st.substepid;
      batch.send_ts = submit_ts;
      Target* target = nullptr;
      try {
        target = get_or_create(batch.tasks.front().req());
      } catch (const std::exception& ex) {
        LOG(ERROR) << "TargetMgr: cannot create stub for " << inst << "," << wid << ": " << ex.what();
        for (const auto& t : batch.tasks) t.set_state(ReqState::FAILED);
        if (batch.inflight != nullptr) batch.inflight->done(false);
        continue;
      }
      if (target->inflycnt.fetch_add(1, std::memory_order_acquire) == 0) target->thread_hint = ++next_hint_;
      auto shared_batch = std::make_shared<BatchSendTask>(std::move(batch));
      send_pool_->spawn(
          [target, shared_batch] {
            fault_inject_sleep(100 * 1000);
            target->stub->send_batch(std::move(*shared_batch));
            target->inflycnt.fetch_sub(1, std::memory_order_release);
          },
          target->thread_hint);
    }
  }
  shrink(static_cast<size_t>(env_txstub_cap()));
}

void KvTransferClient::TargetMgr::shrink(size_t cap) {
  // evict least-recently-used idle targets; stop at the first one still in flight
  while (targets_.size() > cap) {
    Target& victim = targets_.back();
    if (victim.inflycnt.load(std::memory_order_relaxed) > 0 || !victim.stub->idle()) break;
    const InstanceId inst = victim.stub->dstid();
    const WorkerId wid = victim.stub->dstworkerid();
    auto it = index_.find(inst);
    if (it != index_.end()) {
      if (wid < it->second.size()) it->second[wid] = std::nullopt;
      bool any = false;
      for (const auto& s : it->second) any = any || s.has_value();
      if (!any) index_.erase(it);
    }
    LOG(INFO) << "TargetMgr.shrink: instid=" << inst << " wid=" << wid;
    targets_.pop_back();
  }
  n_targets_.store(targets_.size());
}

// ---- client --------------------------------------------------------------------------------------
KvTransferClient::KvTransferClient(std::unique_ptr<Context> ctx, std::unique_ptr<ISendStubFactory> factory)
    : ctx_(std::move(ctx)), mgr_(ctx_.get(), std::move(factory)),
      wait_pool_(std::make_unique<ThreadPool>(static_cast<size_t>(env_waitlayer_tpsize()), "waitlayer")) {
  if (ctx_ == nullptr) throw std::runtime_error("can't create client with context=nullptr;");
}

KvTransferClient::~KvTransferClient() {
  // a step still open at destruction would leave senders blocked on its counters
  std::shared_ptr<StepGuard> g;
  {
    std::lock_guard<std::mutex> lk(coord_lock_);
    g = last_step_guard_;
  }
  if (g) {
    g->layer_ready_all();
    g->step()->notify_layer_ready(g->num_layers);
  }
  wait_pool_.reset();
}

void KvTransferClient::drain() { mgr_.drain(); }

static std::optional<WorkerInfo> parse_worker_info(const std::optional<std::string>& s) {
  if (!s.has_value() || s->empty()) return std::nullopt;
  return WorkerInfo::from_string(*s);
}

static void add_send_task(StepTasks& st, std::shared_ptr<RequestInfo> req, uint32_t seen, uint32_t new_tokens,
                          bool last) {
  auto& per_worker = st.tasks[req->dst_inst_id];
  BatchSendTask* batch = nullptr;
  for (auto& wt : per_worker)
    if (wt.first == req->dst_worker_id) batch = &wt.second;
  if (batch == nullptr) {
    per_worker.emplace_back(req->dst_worker_id, BatchSendTask());
    batch = &per_worker.back().second;
  }
  batch->tasks.emplace_back(std::move(req), seen, new_tokens, last);
}

static StepTasks make_step_tasks(size_t stepid, uint32_t substepid, std::vector<ReqMeta>& metas, bool freeze) {
  StepTasks st;
  st.stepid = stepid;
  st.substepid = substepid;
  for (auto& m : metas) {
    LOG(INFO) << "create_step_tasks: StepIdx=" << stepid << "." << substepid << ";req_id=" << m.reqid
              << ";dst_worker=" << m.dst_inst << ',' << m.dst_worker << ";freeze=" << freeze
              << ";seen_tokens=" << m.seen_tokens << ";new_tokens=" << m.new_tokens;
    RTASSERT(m.new_tokens > 0);
    auto info = std::make_shared<RequestInfo>(std::move(m.dst_inst), m.dst_worker, std::move(m.dst_worker_info),
                                              std::move(m.reqid), std::move(m.src_block_ids),
                                              std::move(m.dst_block_ids));
    add_send_task(st, std::move(info), m.seen_tokens, m.new_tokens, /*last=*/true);
  }
  return st;
}

void KvTransferClient::start_req_send(std::vector<ReqMeta>& metas, size_t stepid, uint32_t substepid) {
  StepTasks st = make_step_tasks(stepid, substepid, metas, true);
  if (st.empty()) return;
  auto step = std::make_shared<Step>(stepid);
  // the data is complete: the step is born with every layer recorded and ready
  step->frozen = true;
  step->notify_layer_recorded(ctx_->num_layers());
  step->notify_layer_ready(ctx_->num_layers());
  step->flush_send_ts = step->wait_layers_start_ts = step->wait_layers_end_ts = step->start_send_ts;
  mgr_.submit(std::move(step), std::move(st));
}

void KvTransferClient::submit_req_send(InstanceId dst_inst, WorkerId dst_worker, RequestId reqid, uint32_t seen,
                                       uint32_t new_tokens, bool last, BlockIds src_blocks, BlockIds dst_blocks,
                                       std::optional<std::string> dst_worker_info, size_t stepid, uint32_t substepid,
                                       uint32_t fanout) {
  RTASSERT(substepid == 0);
  RTASSERT(new_tokens > 0);
  auto parsed = parse_worker_info(dst_worker_info);
  if (!pending_buf_.empty()) {
    RTASSERT_EQ(pending_buf_.stepid, stepid);
    RTASSERT_EQ(pending_buf_.substepid, substepid);
  } else {
    pending_buf_.stepid = stepid;
    pending_buf_.substepid = substepid;
    pending_buf_.send_ts = SteadyClock::now();
  }
  auto info = std::make_shared<RequestInfo>(std::move(dst_inst), dst_worker, std::move(parsed), std::move(reqid),
                                            std::move(src_blocks), std::move(dst_blocks));
  info->replicas = fanout > 1 ? fanout : 1;
  add_send_task(pending_buf_, info, seen, new_tokens, last);
  LOG(INFO) << "submit_req_send: StepIdx=" << stepid << "." << substepid << ";req_id=" << info->req_id
            << ";dst_worker=" << info->dst_inst_id << ',' << dst_worker << ";seen_tokens=" << seen
            << ";new_tokens=" << new_tokens << ";has_last_token=" << last;
  if (!last) reqs_[info->req_id].push_back(std::move(info));  // later chunks arrive as deltas
}

void KvTransferClient::submit_delta_send(const RequestId& reqid, uint32_t seen, uint32_t new_tokens, bool last,
                                         size_t stepid, uint32_t substepid) {
  RTASSERT(substepid == 0);
  if (!pending_buf_.empty()) {
    RTASSERT_EQ(pending_buf_.stepid, stepid);
    RTASSERT_EQ(pending_buf_.substepid, substepid);
  } else {
    pending_buf_.stepid = stepid;
    pending_buf_.substepid = substepid;
    pending_buf_.send_ts = SteadyClock::now();
  }
  auto it = reqs_.find(reqid);
  if (it == reqs_.end()) {
    LOG(WARNING) << "KVT client: request not found for delta send;;req_id=" << reqid << ";seen_tokens=" << seen
                 << ";new_tokens=" << new_tokens << ";has_last_token=" << last;
    return;
  }
  if (new_tokens == 0) RTASSERT(last);  // the only zero-length delta is the closing marker
  for (auto& req : it->second) {
    add_send_task(pending_buf_, req, seen, new_tokens, last);
    LOG(INFO) << "submit_delta_send: StepIdx=" << stepid << "." << substepid << ";req_id=" << reqid
              << ";dst_worker=" << req->dst_inst_id << ',' << req->dst_worker_id << ";seen_tokens=" << seen
              << ";new_tokens=" << new_tokens << ";has_last_token=" << last;
  }
  if (last) reqs_.erase(it);
}

void KvTransferClient::start_send_substep(size_t stepid, uint32_t substepid, std::vector<ReqMeta>& metas) {
  if (metas.empty()) return;
  fault_inject_sleep(333 * 1000);
  enum class Action { ATTACH, FREEZE };
  Action action = Action::ATTACH;
  std::shared_ptr<Step> step;
  {
    std::lock_guard<std::mutex> g(coord_lock_);
    if (stepid < coord_step_id_) {
      action = Action::FREEZE;  // that step is over: its data is complete, send as a frozen step
    } else if (stepid > coord_step_id_) {
      // the worker has not opened that step yet: park until start_send(stepid)
      if (!pending_step_metas_.empty()) {
        RTASSERT_EQ(pending_step_metas_.back().stepid, stepid);
        RTASSERT(pending_step_metas_.back().substepid < substepid);
      }
      pending_step_metas_.push_back(StepMetas{stepid, substepid, std::move(metas)});
      return;
    } else if (last_step_guard_) {
      step = last_step_guard_->step();  // the step is running: ride along with its layer pipeline
    } else {
      action = Action::FREEZE;  // already flushed
    }
  }
  if (action == Action::FREEZE) {
    start_req_send(metas, stepid, substepid);
    return;
  }
  mgr_.submit(std::move(step), make_step_tasks(stepid, substepid, metas, false));
}

size_t KvTransferClient::start_send(size_t stepid, size_t sched_tokens) {
  if (sched_tokens == 0 && pending_buf_.empty()) return EMPTY_STEP_ID;
  fault_inject_sleep(777 * 1000);
  auto step = std::make_shared<Step>(stepid);
  auto guard = std::make_shared<StepGuard>(ctx_.get(), step);
  wait_pool_->spawn([guard] {
    fault_inject_sleep(10 * 1000);
    guard->step()->wait_layers_start_ts = SteadyClock::now();
    try {
      guard->wait_layers();
    } catch (const std::exception& ex) {
      // a failed event wait must not leave senders blocked: release them, the transfer will
      // then fail on its own checks
      LOG(ERROR) << "wait_layers failed: " << ex.what();
      guard->step()->notify_layer_ready(guard->num_layers);
    }
    guard->step()->wait_layers_end_ts = SteadyClock::now();
  });
  if (!pending_buf_.empty()) {
    StepTasks tmp;
    std::swap(tmp, pending_buf_);
    pending_buf_ = StepTasks{};
    mgr_.submit(step, std::move(tmp));
  }
  std::vector<StepMetas> parked;
  {
    std::lock_guard<std::mutex> g(coord_lock_);
    coord_step_id_ = stepid;
    last_step_guard_ = std::move(guard);
    parked.swap(pending_step_metas_);
  }
  for (auto& pm : parked) {
    RTASSERT_EQ(pm.stepid, stepid);
    mgr_.submit(step, make_step_tasks(pm.stepid, pm.substepid, pm.metas, false));
  }
  return stepid;
}

void KvTransferClient::notify_event_record(size_t step_id) {
  if (!last_step_guard_ || last_step_guard_->step_id() != step_id)
    throw KVTransferException(ErrorKind::INVALID_OPERATION, "event record before step start;");
  last_step_guard_->after_record_one();
}

void KvTransferClient::flush_send(size_t step_id) {
  if (!last_step_guard_ || last_step_guard_->step_id() != step_id)
    throw KVTransferException(ErrorKind::INVALID_OPERATION, "event record before step start;");
  last_step_guard_->layer_ready_all();
  last_step_guard_->step()->flush_send_ts = SteadyClock::now();
  std::lock_guard<std::mutex> g(coord_lock_);
  last_step_guard_.reset();
}

}  // namespace kvx
