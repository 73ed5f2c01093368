// KvTransferClient: the submit / step API the prefill worker drives.
//
//   submit_req_send / submit_delta_send   buffer request chunks for the coming step
//   start_send(stepid, sched_tokens)      open the step: layer-ready pipeline + dispatch of the
//                                         buffered chunks to their per-destination stubs
//   notify_event_record(stepid)           one more layer event recorded by the forward pass
//   flush_send(stepid)                    forward pass over: everything recorded
//   start_req_send(metas)                 "freeze" step: data already complete, born ready
//   start_send_substep(stepid, sub, m)    chunks added from another thread while a step runs
//
// Semantics, including the three-way race resolution of start_send_substep against the
// current step id, follow kvtransfer/src/client.cpp:307-543.  TargetMgr keeps an LRU of
// per-destination stubs on one manager thread and runs batches on a sender pool where one
// destination always maps to the same thread (batches of a destination stay ordered).
#pragma once
#include <list>
#include <mutex>
#include <optional>
#include <unordered_map>

#include "core/send_stub.h"

namespace kvx {

constexpr size_t EMPTY_STEP_ID = 9223372036854775807ull;

struct ReqMeta {
  InstanceId dst_inst;
  WorkerId dst_worker = 0;
  RequestId reqid;
  uint32_t seen_tokens = 0;
  uint32_t new_tokens = 0;
  BlockIds src_block_ids;
  BlockIds dst_block_ids;
  std::optional<WorkerInfo> dst_worker_info;
};

struct StepTasks {
  std::unordered_map<InstanceId, std::vector<std::pair<WorkerId, BatchSendTask>>> tasks;
  size_t stepid = 0;
  uint32_t substepid = 0;
  Timepoint send_ts = SteadyClock::now();
  bool empty() const noexcept { return tasks.empty(); }
};

class KvTransferClient {
 public:
  KvTransferClient(std::unique_ptr<Context> ctx, std::unique_ptr<ISendStubFactory> factory);
  ~KvTransferClient();
  KvTransferClient(const KvTransferClient&) = delete;

  void start_req_send(std::vector<ReqMeta>& metas, size_t stepid, uint32_t substepid);  // thread safe
  void submit_req_send(InstanceId dst_inst, WorkerId dst_worker, RequestId reqid, uint32_t seen_tokens,
                       uint32_t new_tokens, bool has_last_token, BlockIds src_block_ids, BlockIds dst_block_ids,
                       std::optional<std::string> dst_worker_info, size_t stepid, uint32_t substepid,
                       uint32_t fanout = 0);
  void submit_delta_send(const RequestId& reqid, uint32_t seen_tokens, uint32_t new_tokens, bool has_last_token,
                         size_t stepid, uint32_t substepid);
  size_t start_send(size_t stepid, size_t sched_tokens);
  void notify_event_record(size_t step_id);
  void flush_send(size_t step_id);
  void start_send_substep(size_t stepid, uint32_t substepid, std::vector<ReqMeta>& metas);  // thread safe

  Context* context() { return ctx_.get(); }
  size_t target_size() const noexcept { return mgr_.size(); }
  void target_try_shrink(size_t cap) { mgr_.shrink_sync(cap); }
  void drain();  // wait until every submitted batch has been processed (tests, shutdown)

 private:
  struct Target {
    std::atomic<int> inflycnt{0};
    int thread_hint = 0;
    SendStub stub;
    explicit Target(SendStub s) : stub(std::move(s)) {}
  };

  class TargetMgr {
   public:
    TargetMgr(Context* ctx, std::unique_ptr<ISendStubFactory> f);
    ~TargetMgr();
    size_t size() const noexcept { return n_targets_.load(); }
    void submit(std::shared_ptr<Step> step, StepTasks tasks);  // thread safe
    void shrink_sync(size_t cap);
    void drain();

   private:
    using Iter = std::list<Target>::iterator;
    Target* get_or_create(const RequestInfo& req);
    void do_submit(std::shared_ptr<Step>& step, StepTasks& tasks);
    void shrink(size_t cap);
    Context* const ctx_;
    std::unique_ptr<ISendStubFactory> factory_;
    std::list<Target> targets_;  // front = most recently used
    std::unordered_map<InstanceId, std::vector<std::optional<Iter>>> index_;
    std::atomic<size_t> n_targets_{0};
    int next_hint_ = 0;
    // Declared last: the pools' threads run tasks that touch the members above, and they are
    // joined first when the manager is destroyed.
    std::unique_ptr<ThreadPool> send_pool_;
    std::unique_ptr<ThreadPool> mgr_thd_;
  };

  std::unique_ptr<Context> ctx_;
  std::unordered_map<RequestId, std::vector<std::shared_ptr<RequestInfo>>> reqs_;
  StepTasks pending_buf_;  // chunks submitted for the next start_send (substep 0)
  TargetMgr mgr_;
  std::mutex coord_lock_;
  size_t coord_step_id_{0};
  std::shared_ptr<StepGuard> last_step_guard_;
  struct StepMetas {
    size_t stepid;
    uint32_t substepid;
    std::vector<ReqMeta> metas;
  };
  std::vector<StepMetas> pending_step_metas_;
  std::unique_ptr<ThreadPool> wait_pool_;
};

}  // namespace kvx
