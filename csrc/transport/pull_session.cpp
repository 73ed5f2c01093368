#include "transport/pull_session.h"

#include <thread>

#include <unistd.h>

#include "core/completion.h"
#include "core/envcfg.h"
#include "core/log.h"

namespace kvx {

PullSession::PullSession(Context* ctx, int fd, std::shared_ptr<std::mutex> write_mu)
    : ctx_(ctx), fd_(fd), write_mu_(std::move(write_mu)) {}

PullSession::~PullSession() {
  close();
  // completions still pending hold a reference to this session, so none is pending here
  eng_.reset();
  close_peer_events(ev_info_, events_);
}

void PullSession::close() { closed_.store(true); }

uint32_t PullSession::open(const char* body, size_t len) {
  const char* p = body;
  const char* end = body + len;
  uint32_t version = 0, n_caps = 0, mem_len = 0, ev_len = 0;
  if (!take(p, end, &version) || version != pull_protocol_version()) return WIRE_BAD_REQUEST;
  if (!take(p, end, &n_caps) || n_caps > KVT_WALK_MAX_TENSORS * 4u) return WIRE_BAD_REQUEST;
  std::vector<uint64_t> src_caps(n_caps);
  for (auto& c : src_caps)
    if (!take(p, end, &c)) return WIRE_BAD_REQUEST;
  if (!take(p, end, &mem_len) || static_cast<size_t>(end - p) < mem_len) return WIRE_BAD_REQUEST;
  PeerMemInfo mem;
  if (!PeerMemInfo::parse(p, mem_len, &mem)) return WIRE_BAD_REQUEST;
  p += mem_len;
  if (!take(p, end, &ev_len) || static_cast<size_t>(end - p) < ev_len) return WIRE_BAD_REQUEST;
  if (!PeerEvents::parse(p, ev_len, &ev_info_)) return WIRE_BAD_REQUEST;
  if (ctx_->device_id() < 0 || mem.num_layers != ctx_->num_layers()) return WIRE_BAD_REQUEST;
  // A pull between two caches on ONE GPU would make the kernels that wait for a layer and the kernels that
  // produce it share a device; the push path serves that case.
  if (mem.device == ctx_->device_id()) return WIRE_BAD_REQUEST;
  // Two workers inside ONE process (a test arrangement; serving engines run one process per GPU) stay with the
  // push path as well: this session would wait on the prefill worker's own event objects from another device's
  // stream, and with events created for interprocess use that wait crashed inside the driver.
  if (mem.pid == static_cast<int32_t>(getpid())) return WIRE_BAD_REQUEST;
  try {
    src_map_.map(mem, ctx_->device_id());
    events_ = open_peer_events(ev_info_);
    if (events_.size() != ctx_->num_layers()) {
      LOG(WARNING) << "pull session: the prefill worker's layer events cannot be shared (not created interprocess?)";
      return WIRE_BAD_REQUEST;
    }
    BatchEngineConfig cfg;
    cfg.device = ctx_->device_id();
    cfg.n_streams = std::max(1, env_nvlink_streams());
    const size_t table = (static_cast<size_t>(ctx_->layer_num_blocks()) * 2) * sizeof(uint32_t);
    cfg.plan_capacity = std::max<size_t>(table * 8 + (1u << 20), 2u << 20);
    cfg.stamps = env_device_timestamps();
    cfg.dst_remote = false;
    cfg.grid_ctas = env_nvlink_ctas();
    std::vector<uint64_t> dst_caps;
    for (size_t t = 0; t < ctx_->block_sizes().size(); ++t) dst_caps.push_back(ctx_->tensor_capacity(t));
    eng_ = std::make_unique<BatchEngine>(cfg, src_map_.ptrs(), ctx_->layer_data_address(), std::move(src_caps), std::move(dst_caps));
    if (!ctx_->multicast_address().empty()) eng_->set_multicast(ctx_->multicast_address());
  } catch (const std::exception& ex) {
    LOG(ERROR) << "pull session: open failed: " << ex.what();
    return WIRE_INTERNAL;
  }
  LOG(INFO) << "pull session open. src_pid=" << mem.pid << " src_device=" << mem.device << " device=" << ctx_->device_id()
            << " same_process=" << src_map_.same_process();
  return WIRE_OK;
}

void PullSession::on_plan(uint64_t seq, const char* body, size_t len) {
  cur_seq_ = seq;
  have_batch_ = false;
  error_.clear();
  try {
    if (!eng_ || len < sizeof(PullPlanHead)) throw std::runtime_error("bad plan message");
    memcpy(&head_, body, sizeof(PullPlanHead));
    if (head_.blob_bytes != len - sizeof(PullPlanHead)) throw std::runtime_error("plan blob length mismatch");
    if (head_.fanout != 0 && (head_.kind != PULL_KIND_WALK || !eng_->has_multicast()))
      throw std::runtime_error("fan-out asked of a worker whose cache is not in a multicast group");
    BatchEngine::SlotView sl = eng_->begin(head_.blob_bytes);
    memcpy(sl.h_plan, body + sizeof(PullPlanHead), head_.blob_bytes);
    eng_->upload(head_.blob_bytes);
    attn_plan_ = PackedPlan{};
    attn_plan_.n_reqs = head_.n_reqs;
    attn_plan_.total_tiles = head_.total_tiles;
    attn_plan_.pool_offset = head_.pool_offset;
    have_batch_ = true;
  } catch (const std::exception& ex) {
    error_ = ex.what();
    LOG(ERROR) << "pull session: plan of batch " << seq << " failed: " << ex.what();
  }
}

void PullSession::on_layers(uint64_t seq, const char* body, size_t len) {
  if (seq != cur_seq_ || !have_batch_ || !error_.empty()) return;
  uint32_t lo = 0, hi = 0;
  uint8_t one_launch = 0;
  const char* p = body;
  const char* end = body + len;
  if (!take(p, end, &lo) || !take(p, end, &hi) || !take(p, end, &one_launch) || hi > events_.size() || lo >= hi) {
    error_ = "bad layers message";
    return;
  }
  try {
    if (head_.kind == PULL_KIND_WALK) {
      // one launch for the range, behind the last of its layer events (recorded in order on one stream)
      const size_t stage = eng_->next_stage();
      eng_->launch_walk(head_.walk, head_.n_ops, head_.pool_len, lo, hi, stage, events_[hi - 1]);
      // the bytes are here: the switch delivers them to the other members of the group from this GPU
      if (head_.fanout != 0) eng_->launch_walk_fanout(head_.walk, head_.n_ops, head_.pool_len, lo, hi, stage);
    } else if (one_launch) {
      eng_->launch_attn(head_.attn, attn_plan_, lo, hi, 0, events_[hi - 1]);
    } else {
      for (uint32_t l = lo; l < hi; ++l) eng_->launch_attn(head_.attn, attn_plan_, l, l + 1, l % eng_->n_stages(), events_[l]);
    }
  } catch (const std::exception& ex) {
    error_ = ex.what();
    LOG(ERROR) << "pull session: layers [" << lo << ", " << hi << ") of batch " << seq << " failed: " << ex.what();
  }
}

void PullSession::send_done(uint64_t seq, uint32_t status, uint32_t detail, uint64_t t0, uint64_t t1) {
  std::string msg(RPC_HEADER, '\0');
  put_rpc_header(msg.data(), PULL_DONE, seq);
  put(msg, status);
  put(msg, detail);
  put(msg, t0);
  put(msg, t1);
  std::lock_guard<std::mutex> g(*write_mu_);
  if (closed_.load()) return;     // the connection's thread closes the descriptor after it has taken this lock once more
  if (!send_frame(fd_, msg.data(), msg.size(), env_rpc_timeout_s() * 1000)) closed_.store(true);
}

void PullSession::on_flush(uint64_t seq, const char* body, size_t len) {
  uint8_t drop = 0;
  if (len >= 1) drop = static_cast<uint8_t>(body[0]);
  if (seq != cur_seq_ || !have_batch_ || !error_.empty()) {
    // nothing was enqueued for this batch (or part of it failed): still let what was enqueued finish, and say so
    if (eng_ && eng_->in_batch()) {
      try {
        BatchEngine::Done d;
        eng_->wait(eng_->flush_async(""), &d);
      } catch (const std::exception&) {
      }
    }
    send_done(seq, 0xffffffffu, 0, 0, 0);
    have_batch_ = false;
    return;
  }
  have_batch_ = false;
  uint64_t ticket = 0;
  try {
    ticket = eng_->flush_async("", drop != 0);
  } catch (const std::exception& ex) {
    LOG(ERROR) << "pull session: flush of batch " << seq << " failed: " << ex.what();
    send_done(seq, 0xffffffffu, 0, 0, 0);
    return;
  }
  // the record is polled by the process's completion thread; the connection thread goes on with the next batch
  auto self = shared_from_this();
  pending_.fetch_add(1);
  CompletionPoller::Entry e;
  e.owner = this;
  e.deadline = SteadyClock::now() + std::chrono::milliseconds(env_completion_timeout_ms());
  auto done = std::make_shared<BatchEngine::Done>();
  e.poll = [self, ticket, done] { return self->eng_->poll(ticket, done.get()); };
  e.finish = [self, seq, done](PollResult r) {
    if (r == PollResult::DONE) self->send_done(seq, done->status, done->detail, done->t_start_ns, done->t_end_ns);
    else self->send_done(seq, 0xfffffffeu, 0, 0, 0);
    self->pending_.fetch_sub(1);
  };
  CompletionPoller::instance().add(std::move(e));
}

}  // namespace kvx
