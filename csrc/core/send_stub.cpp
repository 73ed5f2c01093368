#include "core/send_stub.h"

#include <arpa/inet.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cstring>
#include <thread>

#include "core/completion.h"
#include "core/envcfg.h"
#include "core/fault_inject.h"
#include "plan/device_plan.h"
#include "plan/planner.h"
#include "transport/verify.h"

namespace kvx {

static constexpr uint32_t SEND_DONE_REQ = 0x20181219u;
static constexpr uint32_t SAVE_DONE2_REQ = 0x20181223u;
static constexpr uint32_t HAS_VER2 = 0x40000000u;
static constexpr uint32_t CODE_INTERNALERROR = 500;

std::vector<char> SendDoneNotifier::encode(uint32_t worker_tp_rank, const std::vector<const ReqSendTask*>& reqs,
                                           int head_kind, int* resp_size) {
  std::vector<char> buf;
  auto put32 = [&](uint32_t v) {
    const char* p = reinterpret_cast<const char*>(&v);
    buf.insert(buf.end(), p, p + 4);
  };
  RTASSERT(worker_tp_rank < 0xffff);
  put32(SEND_DONE_REQ);
  put32(worker_tp_rank | HAS_VER2);
  put32(static_cast<uint32_t>(reqs.size()));
  for (const ReqSendTask* r : reqs) {
    put32(r->end_tokens());
    put32(r->state() == ReqState::OK ? 0u : CODE_INTERNALERROR);
    put32(static_cast<uint32_t>(r->req_id().size()));
    buf.insert(buf.end(), r->req_id().begin(), r->req_id().end());
  }
  *resp_size = 4;
  if (head_kind == SEND_SAVE_DONE_HEAD_KIND) {
    // the same body once more under the save-done header: the scheduler's connector half and
    // its backend half each consume one copy
    const size_t n = buf.size();
    buf.resize(2 * n);
    memcpy(buf.data() + n, buf.data(), n);
    const uint32_t h = SAVE_DONE2_REQ;
    memcpy(buf.data() + n, &h, 4);
    *resp_size = 8;
  }
  return buf;
}

void SendDoneNotifier::round_trip(const std::vector<char>& buf, int resp_size) {
  std::string ip_s;
  int port = 0;
  if (!addr_.empty()) {
    const auto pos = addr_.rfind(':');
    if (pos == std::string::npos) return;
    ip_s = addr_.substr(0, pos);
    port = atoi(addr_.c_str() + pos + 1);
  } else {
    const sockaddr_in* addr = env_send_done_addr();
    if (addr == nullptr) return;  // send-done RPC disabled
    char ip[64];
    inet_ntop(AF_INET, &addr->sin_addr, ip, sizeof(ip));
    ip_s = ip;
    port = ntohs(addr->sin_port);
  }
  if (!sock_.valid()) {
    int fd = tcp_connect(ip_s, port, env_rpc_timeout_s() * 1000);
    if (fd < 0) throw std::runtime_error("rpc send done: connect error. errno=" + std::to_string(errno));
    sock_ = FdGuard(fd);
  }
  if (write_full(sock_.fd(), buf.data(), buf.size(), env_rpc_timeout_s() * 1000) != static_cast<ssize_t>(buf.size()))
    throw std::runtime_error("rpc send done: write error. errno=" + std::to_string(errno));
  char resp[16];
  if (read_full(sock_.fd(), resp, static_cast<size_t>(resp_size), env_rpc_timeout_s() * 1000) != resp_size)
    throw std::runtime_error("rpc send done: invalid response");
}

void SendDoneNotifier::notify(const std::vector<const ReqSendTask*>& reqs) {
  if (reqs.empty()) return;
  std::lock_guard<std::mutex> g(mu_);
  int resp_size = 4;
  const std::vector<char> buf = encode(rank_, reqs, env_send_done_head_kind(), &resp_size);
  for (int attempt = 0; attempt < 2; ++attempt) {
    try {
      round_trip(buf, resp_size);
      return;
    } catch (const std::exception& ex) {
      LOG(ERROR) << "do_rpc_send_done failed. ex=" << ex.what();
      sock_.reset();  // a persistent connection may have gone stale: reconnect once
    }
  }
}

static bool same_dst(const WorkerInfo& a, const WorkerInfo& b) noexcept {
  return a.inst_id == b.inst_id && a.worker_id == b.worker_id && a.engine_tp_size == b.engine_tp_size &&
         a.worker_tp_rank == b.worker_tp_rank && a.block_sizes == b.block_sizes && a.token_sizes == b.token_sizes &&
         a.layer_num_blocks == b.layer_num_blocks && a.num_layers == b.num_layers &&
         a.transfer_protocols == b.transfer_protocols;
}

// One batch from "handed to the stub" to "finished": it owns the request chunks (the pointers below point
// into batch.tasks) and keeps the channel alive while a device transport still completes it.
struct PendingBatch {
  BatchSendTask batch;
  std::vector<const ReqSendTask*> send_req, finished_req;
  Channel ch;
  uint64_t ticket = 0;
  std::string flush_out;
  int64_t queue_us = 0, plan_us = 0, wait_us = 0;
  Timepoint iter_start, enqueued;
  // end-to-end check: the batch's byte ranges and the destination they were sent to (empty: not checked)
  std::vector<std::vector<IpcBlock>> check_blocks;
  AttnCheck check_src_rows, check_dst_rows;   // the row form, for a batch that changes the layout
  WorkerInfo check_dst;
};

struct KvSendStub::Impl {
  KvSendStub* stub;
  WorkerInfo src_info;
  std::shared_ptr<INamingWorkerClient> naming;
  uint32_t start_layer, num_layers;
  std::unique_ptr<IChannelFactory> channel_factory;
  int cache_shape;
  SendDoneNotifier notifier;

  std::optional<WorkerInfo> dstinfo;
  PlanEnv env;
  PlannerChoice planner;
  Channel ch;
  std::atomic<bool> drop_channel{false};   // set by the completion thread when a batch failed on the device
  std::atomic<int> completing{0};          // batches handed to the completion poller and not yet finished

  std::vector<std::vector<IpcBlock>> send_blocks;
  Context* check_ctx{nullptr};              // set: batches are verified end to end
  bool check_unavailable_logged{false};

  Impl(KvSendStub* s, const WorkerInfo& src, std::shared_ptr<INamingWorkerClient> n, uint32_t sl, uint32_t nl,
       std::unique_ptr<IChannelFactory> f, int shape, std::string sd_addr)
      : stub(s), src_info(src), naming(std::move(n)), start_layer(sl), num_layers(nl), channel_factory(std::move(f)),
        cache_shape(shape), notifier(src.worker_tp_rank, std::move(sd_addr)) {}

  void refresh_dst_info() {
    auto fresh = naming->get_worker_info(stub->dstid(), stub->dstworkerid());
    if (!fresh.has_value()) {
      if (dstinfo.has_value()) {
        LOG(WARNING) << "refresh_dst_info:use origdstinfo=" << dstinfo->to_string();
        return;
      }
      LOG(ERROR) << "refresh_dst_info:origdstinfo=none dstid=" << stub->dstid() << " dstwid=" << stub->dstworkerid();
      throw std::runtime_error("can't find target worker");
    }
    if (dstinfo.has_value()) {
      if (!same_dst(*dstinfo, *fresh)) {
        // a different worker took over the id: keep talking to the one this stub was bound to
        LOG(WARNING) << "TaskContext.dst_info: invalid dst: orig_dst_info=" << dstinfo->to_string()
                     << "bad_dst_info=" << fresh->to_string();
        return;
      }
      dstinfo->addr = fresh->addr;
      dstinfo->ext = fresh->ext;
      return;
    }
    dstinfo = std::move(fresh);
    env = PlanEnv{};
    env.src = &src_info;
    env.dst = &*dstinfo;
    env.cache_shape = cache_shape;
    env.cast_bf16_to_fp8 = env_bf162fp8_conversion();
    env.pad_last_attn_block = env_pad_last_attn_block();
    planner = bind_planner(env);
    LOG(INFO) << "Get valid_ranks. Src Info: valid_ranks=" << env.valid_ranks.to_string()
              << ",engine_tp_size=" << src_info.engine_tp_size << ",engine_tp_rank=" << src_info.worker_tp_rank
              << ",effective_kvt_tp_size=" << env.kvt_tp_size << ",effective_kvt_tp_rank=" << env.kvt_tp_rank
              << ",planner=" << planner.name << ",Dst Info: engine_tp_size=" << dstinfo->engine_tp_size
              << ",worker_tp_rank=" << dstinfo->worker_tp_rank;
  }

  void try_create_channel() {
    if (drop_channel.exchange(false)) ch.reset();
    if (ch && ch->is_active()) return;
    refresh_dst_info();
    env.dst = &*dstinfo;
    ch = channel_factory->create(*dstinfo);
    LOG(INFO) << "create channel. dst=" << dstinfo->to_string() << ";ch=" << ch.get() << ";proto=" << ch->name();
  }

  // End-to-end check, first half: remember the batch's byte ranges.  `planned` is the host plan of the
  // batch; a device-planned batch (nullptr) is planned once more here, on the CPU, for the check alone.
  void keep_check_blocks(PendingBatch& pb, const std::vector<std::vector<IpcBlock>>* planned) {
    const int dst_shape = dstinfo->cache_shape_or(cache_shape);
    const char* why = nullptr;
    if (dstinfo->ext_int("mx", env_dst_mxfp8()) != 0 || env.cast_bf16_to_fp8) {
      why = "it converts the dtype";
    } else if (dst_shape != cache_shape) {
      // no common byte ranges, but common rows: what the fused attention kernel moves
      DeviceAttnParams p;
      why = "it converts a cache layout that has no row description";
      if (planned == nullptr && check_ctx->device_id() >= 0 && device_attn_params(env, planner.kind, cache_shape, dst_shape, false, &p, nullptr)) {
        if (p.skip) return;          // this rank holds only replicas: it sent nothing
        pb.check_src_rows.layout = p.src;
        pb.check_src_rows.head0 = p.src_head0;
        pb.check_dst_rows.layout = p.dst;
        pb.check_dst_rows.head0 = p.dst_head0;
        pb.check_src_rows.n_heads = pb.check_dst_rows.n_heads = p.n_heads;
        uint32_t index = 0;
        for (const ReqSendTask* t : pb.send_req) {
          if (t->src_blocks().empty() || t->dst_blocks().empty()) continue;
          pb.check_src_rows.add(t->src_blocks()[0], t->seen_tokens, t->new_tokens, index);
          pb.check_dst_rows.add(t->dst_blocks()[0], t->seen_tokens, t->new_tokens, index);
          ++index;
        }
        pb.check_dst = *dstinfo;
        return;
      }
    }
    if (why == nullptr) {
      try {
        if (planned != nullptr) {
          pb.check_blocks = *planned;
        } else {
          for (const ReqSendTask* t : pb.send_req) plan_request(planner, env, *t, pb.check_blocks);
        }
        pb.check_dst = *dstinfo;
        return;
      } catch (const std::exception& ex) {
        pb.check_blocks.clear();
        why = "byte ranges cannot describe it";
      }
    }
    if (!check_unavailable_logged) {
      check_unavailable_logged = true;
      LOG(WARNING) << "KVT transfer check is on (BLLM_KVTRANS_CRC) but this transfer goes unchecked: " << why
                   << ". DstId=" << stub->dstid() << ",DstWorkerId=" << stub->dstworkerid();
    }
  }

  // Second half, when the batch has landed: compare the two caches.  False fails the batch.
  bool run_check(PendingBatch& pb) noexcept {
    try {
      const CheckOutcome o = pb.check_blocks.empty()
                                 ? verify_attn_transfer(check_ctx, pb.check_dst, start_layer, num_layers, pb.check_src_rows,
                                                        pb.check_dst_rows)
                                 : verify_transfer(check_ctx, pb.check_dst, start_layer, num_layers, pb.check_blocks);
      pb.flush_out += ",Check=" + std::string(o.ok ? "ok" : "MISMATCH") + ",CheckLocalUs=" + std::to_string(o.local_us) +
                      ",CheckRemoteUs=" + std::to_string(o.remote_us);
      if (!o.ok) {
        LOG(ERROR) << "KVT transfer check failed: source and destination differ. DstId=" << stub->dstid()
                   << ",DstWorkerId=" << stub->dstworkerid() << ",StepIdx=" << pb.batch.step->step_idx << "."
                   << pb.batch.substepid << ",local=" << o.local << ",remote=" << o.remote;
        drop_channel.store(true);
      }
      return o.ok;
    } catch (const std::exception& ex) {
      LOG(ERROR) << "KVT transfer check could not run. DstId=" << stub->dstid() << ",DstWorkerId=" << stub->dstworkerid()
                 << ",ex=" << ex.what();
      pb.flush_out += ",Check=error";
      return false;
    }
  }

  // Returns true when the batch completes asynchronously (pb.ticket names its completion record).
  bool do_send(PendingBatch& pb) {
    BatchSendTask& batch = pb.batch;
    pb.wait_us = 0;
    const bool by_record = ch->device_ordered();
    // a frozen step has nothing to wait for: let the channel move all layers in one go
    const bool whole = batch.step->frozen && ch->send_layers(start_layer, num_layers, batch.step.get());
    for (uint32_t i = start_layer; i < num_layers && !whole;) {
      TimeWatch w;
      if (by_record) batch.step->wait_layer_recorded(i); else batch.step->wait_layer_ready(i);
      pb.wait_us += w.get_elapse_us();
      if (by_record) {
        // layers recorded while the sender was busy go out together where the channel can do that
        const uint32_t ready = std::min<uint32_t>(num_layers, std::max<uint32_t>(i + 1, batch.step->layers_recorded()));
        i += static_cast<uint32_t>(ch->send_range(i, ready, batch.step.get()));
      } else {
        ch->send_data(i, batch.step.get());  // may be asynchronous
        ++i;
      }
    }
    fault_inject_throw();
    if (ch->async_flush()) {
      pb.ticket = ch->flush_async();
      pb.ch = ch;
      return true;
    }
    ch->flush(pb.flush_out);
    return false;
  }

  // Everything that follows a batch's data: request states, the send-done report, step and stub metrics.
  // Runs on the sender thread (host transports, failures) or on the completion poller's thread.
  void finish(PendingBatch& pb, bool ok) noexcept {
    BatchSendTask& batch = pb.batch;
    const size_t step_idx = batch.step->step_idx;
    Timepoint send_finish = SteadyClock::now();
    if (ok && (!pb.check_blocks.empty() || !pb.check_src_rows.reqs.empty())) {
      ok = run_check(pb);
      pb.check_blocks.clear();
      send_finish = SteadyClock::now();
    }
    const int64_t wait_and_send_us = elapse_us(pb.iter_start, send_finish);
    if (!ok) {
      for (const auto& task : batch.tasks) task.set_state(ReqState::FAILED);
    }
    for (const ReqSendTask* task : pb.finished_req) {
      if (task->state() == ReqState::INPROCESS) {
        // a request closed without ever sending a token counts as failed
        task->set_state(task->new_tokens == 0 ? ReqState::FAILED : ReqState::OK);
      }
      LOG(INFO) << "KVT tx_stub. DstId=" << stub->dstid() << ",DstWorkerId=" << stub->dstworkerid()
                << ",StepIdx=" << step_idx << "." << batch.substepid << ",State=" << static_cast<int>(task->state())
                << ",FinishedReq=" << task->req_id();
    }
    int64_t send_notify_us = 0;
    if (!pb.finished_req.empty()) {
      // a request that the destination relayed to k workers of its group reports k times: the scheduler counts one
      // completion per worker that this rank would otherwise have served itself
      bool relayed = false;
      for (const ReqSendTask* task : pb.finished_req) relayed = relayed || task->req().replicas > 1;
      if (relayed) {
        std::vector<const ReqSendTask*> expanded;
        for (const ReqSendTask* task : pb.finished_req) expanded.insert(expanded.end(), task->req().replicas, task);
        notifier.notify(expanded);
      } else {
        notifier.notify(pb.finished_req);
      }
      const auto now = SteadyClock::now();
      send_notify_us = elapse_us(send_finish, now);
      send_finish = now;
    }
    batch.step->update_last_send_finish_ts(send_finish);
    LOG(INFO) << "SendStubMetrics. DstId=" << stub->dstid() << ",DstWorkerId=" << stub->dstworkerid()
              << ",StepIdx=" << step_idx << "." << batch.substepid << ",FinishedReqSize=" << pb.finished_req.size() << ","
              << pb.flush_out << ",QueueUs=" << pb.queue_us << ",PlanUs=" << pb.plan_us << ",WaitUs=" << pb.wait_us
              << ",EnqueueUs=" << elapse_us(pb.iter_start, pb.enqueued) << ",WaitAndSendUs=" << wait_and_send_us
              << ",SendNotifyUs=" << send_notify_us << ",SendFinishTs=" << send_finish.time_since_epoch().count();
    if (batch.inflight != nullptr) batch.inflight->done(ok);
  }

  void do_task(std::shared_ptr<PendingBatch> pbp) noexcept {
    PendingBatch& pb = *pbp;
    BatchSendTask& batch = pb.batch;
    const size_t step_idx = batch.step->step_idx;
    fault_inject_sleep(300 * 1000);
    pb.iter_start = pb.enqueued = SteadyClock::now();
    pb.queue_us = elapse_us(batch.send_ts, pb.iter_start);
    for (const auto& task : batch.tasks) {
      if (task.reach_last_token) pb.finished_req.push_back(&task);
      if (task.new_tokens == 0) continue;            // a pure "close this request" marker
      if (task.state() == ReqState::FAILED) continue;  // an earlier chunk already failed
      pb.send_req.push_back(&task);
    }
    bool ok = true, async = false;
    if (!pb.send_req.empty()) {
      try {
        try_create_channel();
        for (const ReqSendTask* t : pb.send_req)
          if (t->req().replicas > 1 && !ch->relays_to_group())
            throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                      "a relayed transfer (fanout) needs the NVLINK transport and a destination in a multicast group");
        bool device_planned = ch->register_tasks(env, pb.send_req);
        bool have_data = device_planned;
        if (!device_planned) {
          // Byte ranges can only describe a transfer between caches of one layout and dtype: a
          // layout change or a block-scaled fp8 destination needs the fused kernel (NVLINK transport
          // between GPU caches).  Refuse instead of delivering misplaced bytes.
          const int dst_shape = dstinfo->cache_shape_or(cache_shape);
          if (dst_shape != cache_shape || dstinfo->ext_int("mx", 0) != 0) {
            throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                      "transfer from cache shape " + std::to_string(cache_shape) + " to shape " +
                                          std::to_string(dst_shape) + (dstinfo->ext_int("mx", 0) != 0 ? " (block-scaled fp8)" : "") +
                                          " needs the fused kernel of the NVLINK transport; channel is " + ch->name());
          }
          send_blocks.clear();
          for (const ReqSendTask* t : pb.send_req) plan_request(planner, env, *t, send_blocks);
          have_data = !send_blocks.empty() && !send_blocks[0].empty();
          if (have_data && check_ctx != nullptr) keep_check_blocks(pb, &send_blocks);
          if (have_data) ch->register_data(send_blocks, planner.kind);
        } else if (check_ctx != nullptr) {
          keep_check_blocks(pb, nullptr);
        }
        pb.plan_us = elapse_us(pb.iter_start, SteadyClock::now());   // channel, planning, descriptor upload
        if (have_data) async = do_send(pb);
        pb.enqueued = SteadyClock::now();
      } catch (const std::exception& ex) {
        LOG(ERROR) << "KVT tx_stub fail to send data. DstId=" << stub->dstid() << ",DstWorkerId=" << stub->dstworkerid()
                   << ",StepIdx=" << step_idx << "." << batch.substepid << ',' << pb.flush_out << ",ex=" << ex.what();
        ch.reset();
        ok = false;
        async = false;
      }
    }
    send_blocks.clear();
    send_blocks.shrink_to_fit();
    if (!async && completing.load(std::memory_order_acquire) == 0) {
      finish(pb, ok);
      return;
    }
    // The batch (or an earlier one of this stub) completes on the device: hand it to the completion poller,
    // which finishes this stub's batches in the order they were sent.
    completing.fetch_add(1, std::memory_order_acq_rel);
    CompletionPoller::Entry e;
    e.owner = this;
    e.deadline = SteadyClock::now() + std::chrono::milliseconds(env_completion_timeout_ms());
    Impl* self = this;
    if (async) {
      e.poll = [pbp] { return pbp->ch->poll_completion(pbp->ticket, pbp->flush_out); };
    } else {
      e.poll = [ok] { return ok ? PollResult::DONE : PollResult::FAILED; };
    }
    e.finish = [self, pbp](PollResult r) {
      if (r != PollResult::DONE) {
        LOG(ERROR) << "KVT tx_stub batch failed on completion. DstId=" << self->stub->dstid() << ",DstWorkerId="
                   << self->stub->dstworkerid() << ",StepIdx=" << pbp->batch.step->step_idx << "." << pbp->batch.substepid
                   << ',' << pbp->flush_out;
        if (pbp->ch) self->drop_channel.store(true);
      }
      self->finish(*pbp, r == PollResult::DONE);
      pbp->ch.reset();
      self->completing.fetch_sub(1, std::memory_order_acq_rel);
    };
    CompletionPoller::instance().add(std::move(e));
  }
};

KvSendStub::KvSendStub(InstanceId dstid, WorkerId dstworkerid, const WorkerInfo& src_info, uint32_t start_layer,
                       uint32_t num_layers, std::unique_ptr<IChannelFactory> channel_factory,
                       std::shared_ptr<INamingWorkerClient> naming, int cache_shape, std::string send_done_addr)
    : ISendStub(std::move(dstid), dstworkerid),
      impl_(std::make_unique<Impl>(this, src_info, std::move(naming), start_layer, num_layers,
                                   std::move(channel_factory), cache_shape, std::move(send_done_addr))) {}

KvSendStub::~KvSendStub() {
  // batches still completing hold pointers into this stub: wait for them (each one is bounded by its deadline)
  const Timepoint give_up = SteadyClock::now() + std::chrono::milliseconds(env_completion_timeout_ms() + 2000);
  while (impl_->completing.load(std::memory_order_acquire) > 0 && SteadyClock::now() < give_up)
    std::this_thread::sleep_for(std::chrono::microseconds(200));
}

void KvSendStub::enable_check(Context* ctx) { impl_->check_ctx = ctx; }

bool KvSendStub::idle() const { return impl_->completing.load(std::memory_order_acquire) == 0; }

void KvSendStub::send_batch(BatchSendTask batch) noexcept {
  auto pb = std::make_shared<PendingBatch>();
  pb->batch = std::move(batch);
  impl_->do_task(std::move(pb));
}

KvSendStubFactory::KvSendStubFactory(Context* ctx, std::shared_ptr<INamingClient> naming)
    : ctx_(ctx), naming_(std::move(naming)) {
  if (naming_) naming_worker_ = std::make_shared<WorkerNamingClient>(naming_);
}

SendStub KvSendStubFactory::create_stub(const InstanceId& dst, WorkerId dst_worker, uint32_t start_layer,
                                        uint32_t num_layers, std::optional<TransferProtocol> proto,
                                        const std::optional<WorkerInfo>& dst_info) {
  std::shared_ptr<INamingWorkerClient> nw;
  if (dst_info.has_value()) nw = std::make_shared<FakeNamingWorkerClient>(*dst_info);
  else nw = naming_worker_;
  if (!nw) throw std::runtime_error("no naming service and no destination info in the request");
  const int shape = ctx_->worker_info().cache_shape_or(env_cache_shape());
  auto stub = std::make_unique<KvSendStub>(dst, dst_worker, ctx_->worker_info(), start_layer, num_layers,
                                           std::make_unique<ChannelFactory>(ctx_, proto), std::move(nw), shape,
                                           ctx_->worker_info().ext_str("sdaddr"));
  if (env_crc() != 0) stub->enable_check(ctx_);
  return stub;
}

}  // namespace kvx
