#include "transport/batch_engine.h"

#include <algorithm>
#include <cstring>
#include <thread>

#include "core/envcfg.h"
#include "core/log.h"
#include "core/types.h"

namespace kvx {

template <typename T>
BatchEngine::DevArray<T>::~DevArray() {
  if (p != nullptr) cudaFree(p);
}

template <typename T>
void BatchEngine::DevArray<T>::upload(const std::vector<T>& v) {
  if (p != nullptr) cudaFree(p);
  p = nullptr;
  n = v.size();
  if (n == 0) return;
  cuda_check(cudaMalloc(reinterpret_cast<void**>(&p), n * sizeof(T)), "cudaMalloc");
  cuda_check(cudaMemcpy(p, v.data(), n * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
}

BatchEngine::BatchEngine(const BatchEngineConfig& cfg, std::vector<std::vector<uint64_t>> src_ptrs,
                         std::vector<std::vector<uint64_t>> dst_ptrs, std::vector<uint64_t> src_caps,
                         std::vector<uint64_t> dst_caps)
    : cfg_(cfg), src_ptrs_(std::move(src_ptrs)), dst_ptrs_(std::move(dst_ptrs)), src_caps_(std::move(src_caps)),
      dst_caps_(std::move(dst_caps)) {
  RTASSERT(src_ptrs_.size() == dst_ptrs_.size() && !src_ptrs_.empty());
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  for (int i = 0; i < std::max(1, cfg_.n_streams); ++i) stages_.emplace_back(std::make_unique<DeviceStage>(cfg_.device));
  alloc_slots(cfg_.plan_capacity);
}

BatchEngine::~BatchEngine() { close(); }

void BatchEngine::close() {
  if (stages_.empty() && slots_.empty()) return;
  cudaSetDevice(cfg_.device);
  // batches still in flight keep writing into the slots: let them finish (every kernel here bounds its own
  // waits) before the memory goes away
  for (Slot& sl : slots_)
    if (sl.stream != nullptr) cudaStreamSynchronize(sl.stream);
  stages_.clear();
  free_slots();
}

void BatchEngine::alloc_slots(size_t cap) {
  free_slots();
  plan_cap_ = (cap + 255) & ~size_t{255};
  cuda_check(cudaMalloc(reinterpret_cast<void**>(&d_plan_all_), plan_cap_ * kSlots), "cudaMalloc(plans)");
  cuda_check(cudaHostAlloc(reinterpret_cast<void**>(&h_plan_all_), plan_cap_ * kSlots, cudaHostAllocPortable), "cudaHostAlloc(plans)");
  cuda_check(cudaMalloc(reinterpret_cast<void**>(&d_status_all_), 64 * kSlots), "cudaMalloc(status)");
  cuda_check(cudaMemset(d_status_all_, 0, 64 * kSlots), "cudaMemset");
  void* h = nullptr;
  cuda_check(cudaHostAlloc(&h, 64 * kSlots, cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc(records)");
  memset(h, 0, 64 * kSlots);
  h_rec_all_ = static_cast<char*>(h);
  void* d = nullptr;
  cuda_check(cudaHostGetDevicePointer(&d, h, 0), "cudaHostGetDevicePointer");
  slots_.assign(kSlots, Slot{});
  for (size_t i = 0; i < kSlots; ++i) {
    Slot& sl = slots_[i];
    cuda_check(cudaStreamCreateWithFlags(&sl.stream, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_check(cudaEventCreateWithFlags(&sl.plan_event, cudaEventDisableTiming), "cudaEventCreate");
    cuda_check(cudaEventCreateWithFlags(&sl.done_event, cudaEventDisableTiming), "cudaEventCreate");
    sl.d_plan = d_plan_all_ + i * plan_cap_;
    sl.h_plan = h_plan_all_ + i * plan_cap_;
    sl.d_status = reinterpret_cast<uint32_t*>(d_status_all_ + 64 * i);
    sl.h_rec = reinterpret_cast<KvtCompletion*>(h_rec_all_ + 64 * i);
    sl.d_rec = reinterpret_cast<KvtCompletion*>(static_cast<char*>(d) + 64 * i);
  }
}

void BatchEngine::free_slots() {
  for (Slot& sl : slots_) {
    if (sl.plan_event != nullptr) cudaEventDestroy(sl.plan_event);
    if (sl.done_event != nullptr) cudaEventDestroy(sl.done_event);
    if (sl.stream != nullptr) cudaStreamDestroy(sl.stream);
  }
  slots_.clear();
  if (d_plan_all_ != nullptr) cudaFree(d_plan_all_);
  if (h_plan_all_ != nullptr) cudaFreeHost(h_plan_all_);
  if (d_status_all_ != nullptr) cudaFree(d_status_all_);
  if (h_rec_all_ != nullptr) cudaFreeHost(h_rec_all_);
  d_plan_all_ = h_plan_all_ = d_status_all_ = h_rec_all_ = nullptr;
  last_done_event_ = nullptr;
  batch_slot_ = -1;
}

bool BatchEngine::record_arrived(const Slot& sl) { return __atomic_load_n(&sl.h_rec->seq, __ATOMIC_ACQUIRE) == sl.seq; }

BatchEngine::Done BatchEngine::take_record(Slot& sl) {
  Done d;
  d.status = sl.h_rec->status;
  d.detail = sl.h_rec->detail;
  d.t_start_ns = sl.h_rec->t_start_ns;
  d.t_end_ns = sl.h_rec->t_end_ns;
  d.metrics = std::move(sl.metrics);
  sl.pending = false;
  return d;
}

BatchEngine::Slot& BatchEngine::cur() {
  RTASSERT(batch_slot_ >= 0);
  return slots_[static_cast<size_t>(batch_slot_)];
}

BatchEngine::SlotView BatchEngine::current() {
  Slot& sl = cur();
  return SlotView{sl.h_plan, sl.d_plan, sl.d_status, sl.seq};
}

// Waits (bounded) until the slot's previous batch has completed and parks its record for poll().
void BatchEngine::wait_slot(Slot& sl) {
  const Timepoint deadline = SteadyClock::now() + std::chrono::milliseconds(env_completion_timeout_ms());
  for (int spins = 0;; ++spins) {
    {
      std::lock_guard<std::mutex> g(slot_mu_);
      if (!sl.pending) return;
      if (record_arrived(sl)) {
        const uint64_t seq = sl.seq;
        finished_[seq] = take_record(sl);
        return;
      }
    }
    if (SteadyClock::now() > deadline)
      throw KVTransferException(ErrorKind::TRANSPORT, "an earlier batch never completed on the device");
    if (spins < 2000) std::this_thread::yield(); else std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
}

// A slot whose previous batch has not completed makes the caller wait here: the back-pressure of a sender
// running more than kSlots batches ahead of the GPU.  A plan larger than the slots re-allocates them (every
// batch drained first).
BatchEngine::SlotView BatchEngine::begin(size_t bytes) {
  RTASSERT(!slots_.empty());
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  if (bytes > plan_cap_) {
    LOG(WARNING) << "transfer plan of " << bytes << " bytes exceeds the slots sized at start (" << plan_cap_ << "); re-allocating";
    for (Slot& sl : slots_) wait_slot(sl);
    for (Slot& sl : slots_) cuda_check(cudaStreamSynchronize(sl.stream), "cudaStreamSynchronize");
    std::map<uint64_t, Done> keep;
    {
      std::lock_guard<std::mutex> g(slot_mu_);
      keep.swap(finished_);
    }
    alloc_slots(bytes * 2);
    std::lock_guard<std::mutex> g(slot_mu_);
    finished_.swap(keep);
  }
  slot_rr_ = (slot_rr_ + 1) % slots_.size();
  Slot& sl = slots_[slot_rr_];
  wait_slot(sl);
  {
    std::lock_guard<std::mutex> g(slot_mu_);
    sl.seq = ++next_seq_;
    sl.metrics.clear();
  }
  batch_slot_ = static_cast<int>(slot_rr_);
  begin_batch();
  return SlotView{sl.h_plan, sl.d_plan, sl.d_status, sl.seq};
}

void BatchEngine::upload(size_t bytes) {
  Slot& sl = cur();
  if (bytes != 0)
    cuda_check(cudaMemcpyAsync(sl.d_plan, sl.h_plan, bytes, cudaMemcpyHostToDevice, sl.stream), "cudaMemcpyAsync(plan)");
  if (cfg_.stamps) cuda_check(kvt_launch_stamp(reinterpret_cast<uint64_t*>(sl.d_status) + 1, sl.stream), "kvt_launch_stamp");
  cuda_check(cudaEventRecord(sl.plan_event, sl.stream), "cudaEventRecord");
}

DeviceStage& BatchEngine::stage(size_t i) {
  if (stage_used_.size() != stages_.size()) stage_used_.assign(stages_.size(), 0);
  if (!stage_used_[i]) {
    stages_[i]->wait_event(cur().plan_event);
    stage_used_[i] = 1;
  }
  return *stages_[i];
}

int BatchEngine::grid() const {
  if (cfg_.grid_ctas > 0) return cfg_.grid_ctas;
  return std::max(1, static_cast<int>(4 * kvt_sm_count(cfg_.device) * env_kernel_copy_sm_usage()));
}

void BatchEngine::ensure_attn_arrays(const DeviceAttnParams& p) {
  const bool same_maps = attn_ready_ && memcmp(&map_src_, &p.src, sizeof(KvtLayout)) == 0 &&
                         memcmp(&map_dst_, &p.dst, sizeof(KvtLayout)) == 0 && map_heads_ == p.n_heads &&
                         map_tile_ == p.tile_tokens;
  if (same_maps) return;
  std::vector<uint64_t> src, dst;
  for (const auto& l : src_ptrs_) src.push_back(l.at(0));
  for (const auto& l : dst_ptrs_) dst.push_back(l.at(0));
  if (!attn_ready_) {
    d_src_layers_.upload(src);
    d_dst_layers_.upload(dst);
  }
  use_tma_ = false;
  if (env_use_tma() != 0 && p.mode == KVT_MODE_COPY) {
    // a tile is kept in the destination's own order, so that it leaves as one linear store where the
    // destination page holds it contiguously (HND pages; NHD pages when every head moves)
    const int want_order = env_tile_order();
    tile_order_ = want_order >= 0 ? (want_order != 0 ? 1u : 0u) : (p.dst.token_stride < p.dst.head_stride ? 1u : 0u);
    const bool flat_ok = kvt_tile_is_flat(&p.dst, p.n_heads, p.tile_tokens, tile_order_) != 0;
    store_form_ = (flat_ok && env_store_form() != 0) ? 1u : 0u;
    std::vector<TensorMapBytes> sm(src.size()), dm(dst.size());
    bool ok = true;
    for (size_t i = 0; i < src.size() && ok; ++i) {
      ok = kvt_encode_tensor_map_ordered(sm[i].b, src[i], &p.src, p.n_heads, p.tile_tokens, tile_order_) == 0 &&
           kvt_encode_tensor_map_ordered(dm[i].b, dst[i], &p.dst, p.n_heads, p.tile_tokens, tile_order_) == 0;
    }
    if (ok) {
      // the previous maps may still be read by kernels in flight: those batches end before their slot is reused,
      // and a layout change between batches of one channel does not happen in practice; drain to be safe
      for (Slot& sl : slots_) cuda_check(cudaStreamSynchronize(sl.stream), "cudaStreamSynchronize");
      for (auto& st : stages_) cuda_check(cudaStreamSynchronize(static_cast<cudaStream_t>(st->stream())), "cudaStreamSynchronize");
      d_src_maps_.upload(sm);
      d_dst_maps_.upload(dm);
      use_tma_ = true;
    } else {
      LOG(WARNING) << "tensor maps not encodable for this layout, using the SIMT path";
    }
  }
  map_src_ = p.src;
  map_dst_ = p.dst;
  map_heads_ = p.n_heads;
  map_tile_ = p.tile_tokens;
  attn_ready_ = true;
}

void BatchEngine::launch_attn(const DeviceAttnParams& params, const PackedPlan& plan, size_t lo, size_t hi, size_t stage_idx,
                              void* wait_event) {
  if (plan.n_reqs == 0 || hi <= lo) return;
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  ensure_attn_arrays(params);
  DeviceStage& st = stage(stage_idx);
  if (wait_event != nullptr) st.wait_event(wait_event);
  Slot& sl = cur();
  KvtAttnLaunch a{};
  a.src_layers = d_src_layers_.p;
  a.dst_layers = d_dst_layers_.p;
  a.src_maps = use_tma_ ? d_src_maps_.p : nullptr;
  a.dst_maps = use_tma_ ? d_dst_maps_.p : nullptr;
  a.src = params.src;
  a.dst = params.dst;
  a.layer_begin = static_cast<uint32_t>(lo);
  a.layer_end = static_cast<uint32_t>(hi);
  a.reqs = reinterpret_cast<const KvtReqDesc*>(sl.d_plan);
  a.n_reqs = plan.n_reqs;
  a.total_tiles = plan.total_tiles;
  a.block_ids = reinterpret_cast<const uint32_t*>(sl.d_plan + plan.pool_offset);
  a.tile_tokens = params.tile_tokens;
  a.src_head0 = params.src_head0;
  a.dst_head0 = params.dst_head0;
  a.n_heads = params.n_heads;
  a.mode = params.mode;
  a.status = sl.d_status;
  a.dst_remote = cfg_.dst_remote ? 1u : 0u;
  a.tile_order = tile_order_;
  a.store_form = store_form_;
  cuda_check(kvt_launch_p2d_attn(&a, grid(), 0, use_tma_ ? 1 : 0, st.stream()), "kvt_launch_p2d_attn");
}

void BatchEngine::ensure_walk_arrays() {
  if (d_walk_src_.p != nullptr) return;
  std::vector<uint64_t> src, dst;
  for (const auto& l : src_ptrs_) src.insert(src.end(), l.begin(), l.end());
  for (const auto& l : dst_ptrs_) dst.insert(dst.end(), l.begin(), l.end());
  RTASSERT(src.size() == dst.size());
  d_walk_src_.upload(src);
  d_walk_dst_.upload(dst);
}

void BatchEngine::launch_walk(const KvtWalkCounts& c, size_t n_ops, size_t pool_len, size_t lo, size_t hi, size_t stage_idx,
                              void* wait_event) {
  if (n_ops == 0 || hi <= lo) return;
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  ensure_walk_arrays();
  DeviceStage& st = stage(stage_idx);
  if (wait_event != nullptr) st.wait_event(wait_event);
  Slot& sl = cur();
  KvtWalkLaunch a{};
  a.src_ptrs = d_walk_src_.p;
  a.dst_ptrs = d_walk_dst_.p;
  a.n_tensors = static_cast<uint32_t>(dst_ptrs_[0].size());
  RTASSERT(a.n_tensors <= KVT_WALK_MAX_TENSORS && src_caps_.size() >= a.n_tensors && dst_caps_.size() >= a.n_tensors);
  a.layer_begin = static_cast<uint32_t>(lo);
  a.layer_end = static_cast<uint32_t>(hi);
  a.shape = (static_cast<uint32_t>(std::max(0, env_walk_stages())) << 16) | (static_cast<uint32_t>(std::max(0, env_walk_threads())) & 0xffffu);
  for (uint32_t t = 0; t < a.n_tensors; ++t) {
    a.src_cap[t] = src_caps_[t];
    a.dst_cap[t] = dst_caps_[t];
  }
  a.ops = reinterpret_cast<const KvtWalkOp*>(sl.d_plan);
  a.n_bulk_ops = c.n_bulk;
  a.n_simt_ops = c.n_simt;
  a.bulk_units = c.bulk_units;
  a.simt_units = c.simt_units;
  a.pool = reinterpret_cast<const uint32_t*>(sl.d_plan + n_ops * sizeof(KvtWalkOp));
  a.pool_len = static_cast<uint32_t>(pool_len);
  a.status = sl.d_status;
  if (a.n_bulk_ops + a.n_simt_ops != 0) cuda_check(kvt_launch_walk(&a, grid(), st.stream()), "kvt_launch_walk");
  if (c.n_zero != 0) {
    // tail padding lands after the copies (same stream): where both touch a byte, the zero wins, as it does
    // when the byte ranges are applied in the planner's order
    a.ops += c.n_bulk + c.n_simt;
    a.n_bulk_ops = 0;
    a.bulk_units = 0;
    a.n_simt_ops = c.n_zero;
    a.simt_units = c.zero_units;
    cuda_check(kvt_launch_walk(&a, grid(), st.stream()), "kvt_launch_walk(zero fill)");
  }
}

void BatchEngine::set_multicast(std::vector<std::vector<uint64_t>> mc_ptrs) {
  RTASSERT(mc_ptrs.size() == dst_ptrs_.size());
  for (size_t l = 0; l < mc_ptrs.size(); ++l) RTASSERT(mc_ptrs[l].size() == dst_ptrs_[l].size());
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  mc_ptrs_ = std::move(mc_ptrs);
  std::vector<uint64_t> flat;
  for (const auto& l : mc_ptrs_) flat.insert(flat.end(), l.begin(), l.end());
  d_walk_mc_.upload(flat);
}

void BatchEngine::launch_walk_fanout(const KvtWalkCounts& c, size_t n_ops, size_t pool_len, size_t lo, size_t hi,
                                     size_t stage_idx) {
  if (n_ops == 0 || hi <= lo) return;
  RTASSERT(has_multicast());
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  ensure_walk_arrays();
  DeviceStage& st = stage(stage_idx);
  Slot& sl = cur();
  KvtWalkLaunch a{};
  a.src_ptrs = d_walk_src_.p;
  a.dst_ptrs = d_walk_dst_.p;
  a.n_tensors = static_cast<uint32_t>(dst_ptrs_[0].size());
  a.layer_begin = static_cast<uint32_t>(lo);
  a.layer_end = static_cast<uint32_t>(hi);
  for (uint32_t t = 0; t < a.n_tensors; ++t) {
    a.src_cap[t] = src_caps_[t];
    a.dst_cap[t] = dst_caps_[t];
  }
  a.ops = reinterpret_cast<const KvtWalkOp*>(sl.d_plan);
  a.n_bulk_ops = c.n_bulk;
  a.n_simt_ops = c.n_simt;
  a.bulk_units = c.bulk_units;
  a.simt_units = c.simt_units;
  a.pool = reinterpret_cast<const uint32_t*>(sl.d_plan + n_ops * sizeof(KvtWalkOp));
  a.pool_len = static_cast<uint32_t>(pool_len);
  a.status = sl.d_status;
  if (env_fanout_weak() != 0) a.shape |= 0x80000000u;
  cuda_check(kvt_launch_walk_fanout(&a, c.n_zero, c.zero_units, d_walk_mc_.p, grid(), st.stream()), "kvt_launch_walk_fanout");
}

void BatchEngine::launch_walk_multicast(const KvtWalkCounts& c, size_t n_ops, size_t pool_len, size_t lo, size_t hi,
                                        size_t stage_idx, void* wait_event) {
  if (n_ops == 0 || hi <= lo) return;
  RTASSERT(has_multicast());
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  ensure_walk_arrays();
  DeviceStage& st = stage(stage_idx);
  if (wait_event != nullptr) st.wait_event(wait_event);
  Slot& sl = cur();
  KvtWalkLaunch a{};
  a.src_ptrs = d_walk_src_.p;
  a.dst_ptrs = d_walk_dst_.p;
  a.n_tensors = static_cast<uint32_t>(dst_ptrs_[0].size());
  a.layer_begin = static_cast<uint32_t>(lo);
  a.layer_end = static_cast<uint32_t>(hi);
  for (uint32_t t = 0; t < a.n_tensors; ++t) {
    a.src_cap[t] = src_caps_[t];
    a.dst_cap[t] = dst_caps_[t];
  }
  a.ops = reinterpret_cast<const KvtWalkOp*>(sl.d_plan);
  a.n_bulk_ops = c.n_bulk;
  a.n_simt_ops = c.n_simt;
  a.bulk_units = c.bulk_units;
  a.simt_units = c.simt_units;
  a.pool = reinterpret_cast<const uint32_t*>(sl.d_plan + n_ops * sizeof(KvtWalkOp));
  a.pool_len = static_cast<uint32_t>(pool_len);
  a.status = sl.d_status;
  if (env_fanout_weak() != 0) a.shape |= 0x80000000u;
  cuda_check(kvt_launch_walk_multicast(&a, c.n_zero, c.zero_units, d_walk_mc_.p, grid(), st.stream()), "kvt_launch_walk_multicast");
}

uint64_t BatchEngine::flush_async(std::string metrics, bool drop_record) {
  cuda_check(cudaSetDevice(cfg_.device), "cudaSetDevice");
  if (batch_slot_ < 0) begin(0);     // a batch without data still completes through a record
  Slot& sl = cur();
  cudaStream_t ss = sl.stream;
  // the slot's stream joins the transfer streams the batch used, and the previous batch's record
  for (size_t i = 0; i < stages_.size() && i < stage_used_.size(); ++i)
    if (stage_used_[i])
      cuda_check(cudaStreamWaitEvent(ss, static_cast<cudaEvent_t>(stages_[i]->record_done()), 0), "cudaStreamWaitEvent");
  if (last_done_event_ != nullptr && last_done_event_ != sl.done_event)
    cuda_check(cudaStreamWaitEvent(ss, last_done_event_, 0), "cudaStreamWaitEvent");
  if (!drop_record) cuda_check(kvt_launch_complete(sl.d_status, sl.d_rec, sl.seq, ss), "kvt_launch_complete");
  cuda_check(cudaEventRecord(sl.done_event, ss), "cudaEventRecord");
  last_done_event_ = sl.done_event;
  {
    std::lock_guard<std::mutex> g(slot_mu_);
    sl.metrics = std::move(metrics);
    sl.pending = true;
  }
  const uint64_t ticket = sl.seq;
  batch_slot_ = -1;
  begin_batch();
  return ticket;
}

PollResult BatchEngine::poll(uint64_t ticket, Done* out) {
  std::lock_guard<std::mutex> g(slot_mu_);
  auto it = finished_.find(ticket);
  if (it != finished_.end()) {
    *out = std::move(it->second);
    finished_.erase(it);
    return PollResult::DONE;
  }
  for (Slot& sl : slots_) {
    if (sl.seq != ticket) continue;
    if (!sl.pending) return PollResult::FAILED;      // never flushed
    if (!record_arrived(sl)) return PollResult::PENDING;
    *out = take_record(sl);
    return PollResult::DONE;
  }
  return PollResult::FAILED;
}

bool BatchEngine::wait(uint64_t ticket, Done* out) {
  const Timepoint deadline = SteadyClock::now() + std::chrono::milliseconds(env_completion_timeout_ms());
  for (int spins = 0;; ++spins) {
    const PollResult r = poll(ticket, out);
    if (r == PollResult::DONE) return true;
    if (r == PollResult::FAILED || SteadyClock::now() > deadline) return false;
    if (spins < 2000) std::this_thread::yield(); else std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
}

}  // namespace kvx
