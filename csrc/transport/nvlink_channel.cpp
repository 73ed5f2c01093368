// NVLink transport: the KV of a prefill GPU reaches the decode GPU's paged cache through peer-mapped
// memory (NVLink 5 / NVSwitch).  No staging buffer, no library copy.
//
// connect() asks the destination's server for the CUDA IPC handles of its layer tensors
// (MEM_HANDLES_REQ); a push channel maps them (a destination in the same process is used by pointer
// after enabling peer access), a pull channel never touches the destination's memory.  One of two
// modes serves the channel:
//
//   push   the transfer kernels run on the prefill GPU: local loads, stores into the peer cache.  Serves a
//          destination on the same GPU, a block-scaled fp8 destination (the quantiser halves the bytes that
//          cross the link) and a destination whose server offers no pull session.
//   pull   the kernels run on the DECODE GPU: a session on the destination's server maps this worker's cache
//          and layer events, and executes the plans this channel sends (transport/pull_session.h).  TMA loads
//          over NVLink run at the copy engine's rate (measured 772 against 705 GB/s for SM-issued stores of any
//          form), and the prefill GPU spends no SM on the transfer.
//
// Requests for a whole multicast group (RequestInfo::replicas > 1: data that every worker of a decode group
// holds identically) take one of two further forms, both through walk ops:
//   relay      over a pull session: the destination worker loads the request and stores what the ops wrote to
//              its group's multicast mapping (kvt_walk_fanout);
//   multicast  when THIS worker's GPU is bound to that multicast object and holds a mapping of it
//              (Context::multicast_address): the source pieces leave as multicast stores from here
//              (kvt_walk_multicast), whatever serves the channel's other requests.
//
// In both modes the kernels are the same two:
//   * kvt_p2d_attn walks the requests' block tables, converts the layout (NHD<->HND), re-shards heads for
//     TP-mismatched pairs and optionally quantises to block-scaled e4m3: cache shapes 1, 2 and 5;
//   * kvt_walk expands the planner's walk ops (hybrid GDN / MLA / KDA pages, any TP relation).
// A third, push-only path takes the planner's IpcBlocks (BLLM_KVTRANS_NVLINK_WALK=0, or a layer of more
// tensors than the walk kernel addresses) and runs the descriptor copy kernel over them.
//
// The channel is device ordered: a layer's kernel is enqueued behind the layer's CUDA event, nothing on the
// host waits for the forward pass.  Nothing on the host waits for the transfer either: flush_async()
// enqueues a completion record behind the batch and returns; the completion poller reads it and finishes
// the batch.  Only plain peer loads and stores and multimem stores are used; loads with cluster multicast
// are never issued.
#include <cuda_runtime.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <sstream>
#include <thread>

#include "core/envcfg.h"
#include "core/fault_inject.h"
#include "core/util.h"
#include "kernels/kvt_kernels.h"
#include "plan/device_plan.h"
#include "transport/batch_engine.h"
#include "transport/channel.h"
#include "transport/device_stage.h"
#include "transport/peer_memory.h"
#include "transport/pull_session.h"
#include "transport/wire.h"

namespace kvx {

namespace {

class NvlinkChannel : public IChannel {
 public:
  explicit NvlinkChannel(Context* ctx) : ctx_(ctx) {}
  ~NvlinkChannel() override { close(); }
  const char* name() const override { return "nvlink"; }
  bool device_ordered() const override { return true; }

  void connect(const WorkerInfo& dst) override {
    RTASSERT(ctx_->device_id() >= 0);
    dst_ = dst;
    fault_inject_throw();
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    // ---- fetch and map the destination's memory ------------------------------------------
    const std::string ip = dst.addr.empty() ? "127.0.0.1" : dst.addr;
    FdGuard sock(tcp_connect(ip, server_port_of(dst), env_rpc_timeout_s() * 1000));
    if (!sock.valid()) throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: cannot reach destination control port");
    std::string req(RPC_HEADER, '\0');
    put_rpc_header(req.data(), MEM_HANDLES_REQ, new_id());
    std::string resp;
    if (!send_frame(sock.fd(), req.data(), req.size(), env_rpc_timeout_s() * 1000) ||
        !recv_frame(sock.fd(), resp, env_rpc_timeout_s() * 1000) || resp.size() < RPC_HEADER + 4) {
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: memory-handle exchange failed");
    }
    uint32_t status = 0;
    memcpy(&status, resp.data() + RPC_HEADER, 4);
    PeerMemInfo info;
    if (status != WIRE_OK || !PeerMemInfo::parse(resp.data() + RPC_HEADER + 4, resp.size() - RPC_HEADER - 4, &info)) {
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: destination has no device memory to map");
    }
    if (info.host_id != this_host_id()) {
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: destination is on another host");
    }
    RTASSERT(info.num_layers == ctx_->num_layers());
    dst_remote_ = info.device != ctx_->device_id();
    same_process_ = info.pid == static_cast<int32_t>(getpid());
    n_tensors_ = info.num_tensors;
    src_shape_ = ctx_->worker_info().cache_shape_or(env_cache_shape());
    dst_shape_ = dst.cache_shape_or(src_shape_);
    dst_mx_ = dst.ext_int("mx", env_dst_mxfp8()) != 0;
    for (size_t t = 0; t < ctx_->block_sizes().size(); ++t) src_caps_.push_back(ctx_->tensor_capacity(t));
    for (size_t t = 0; t < dst.block_sizes.size(); ++t)
      dst_caps_.push_back(dst.block_sizes[t] * static_cast<uint64_t>(dst.layer_num_blocks));
    // ---- pull session on the destination, where that is the faster way ----------------------------
    pull_ = false;
    push_unavailable_ = false;
    if (dst_remote_ && !dst_mx_ && env_nvlink_pull() != 0) pull_ = open_pull(sock);
    if (pull_) {
      // the decode GPU reads this worker's cache; its own cache is never mapped here, so it may live in memory that
      // has no IPC handle (a symmetric allocation bound to a multicast group)
      pull_sock_ = std::move(sock);
    } else {
      // ---- push: the destination's cache mapped here, streams and plan slots on this GPU ------------
      const bool can_multicast = !ctx_->multicast_address().empty() && dst.ext_int("mcn", 0) > 1 && !dst_mx_;
      try {
        dst_map_.map(info, ctx_->device_id());
      } catch (const std::exception& ex) {
        // a cache in a symmetric allocation has no IPC handle; with a mapping of its multicast object this worker
        // can still serve the requests meant for the whole group
        if (!can_multicast) throw;
        LOG(INFO) << "nvlink: destination cache cannot be mapped (" << ex.what() << "); multicast transfers only";
        push_unavailable_ = true;
      }
      if (!push_unavailable_) {
        BatchEngineConfig cfg;
        cfg.device = ctx_->device_id();
        cfg.n_streams = std::max(1, env_nvlink_streams());
        // A plan holds one descriptor per request and the block tables of both sides.  Sized for every block of
        // both caches in every block group, plus room for a few thousand request descriptors / walk ops.
        const size_t groups = std::max<size_t>(1, ctx_->worker_info().num_gdn_layers + ctx_->worker_info().num_ple_layers + 2);
        const size_t table = (static_cast<size_t>(ctx_->layer_num_blocks()) + dst.layer_num_blocks) * sizeof(uint32_t);
        cfg.plan_capacity = std::max<size_t>(table * std::min<size_t>(groups, 8) + (1u << 20), 2u << 20);
        cfg.stamps = env_device_timestamps();
        cfg.dst_remote = dst_remote_;
        cfg.grid_ctas = env_nvlink_ctas();
        eng_ = std::make_unique<BatchEngine>(cfg, ctx_->layer_data_address(), dst_map_.ptrs(), src_caps_, dst_caps_);
      }
    }
    // ---- this worker's GPU is bound to the destination group's multicast object: relayed requests leave as
    //      multicast stores from here, whichever of pull and push serves the others ----------------------------
    mc_eng_.reset();
    if (!ctx_->multicast_address().empty() && dst.ext_int("mcn", 0) > 1 && !dst_mx_) {
      BatchEngineConfig cfg;
      cfg.device = ctx_->device_id();
      cfg.n_streams = std::max(1, env_nvlink_streams());
      const size_t table = (static_cast<size_t>(ctx_->layer_num_blocks()) + dst.layer_num_blocks) * sizeof(uint32_t);
      cfg.plan_capacity = std::max<size_t>(table * 8 + (1u << 20), 2u << 20);
      cfg.stamps = env_device_timestamps();
      cfg.dst_remote = true;
      cfg.grid_ctas = env_nvlink_ctas();
      mc_eng_ = std::make_unique<BatchEngine>(cfg, ctx_->layer_data_address(), ctx_->multicast_address(), src_caps_, dst_caps_);
      mc_eng_->set_multicast(ctx_->multicast_address());
    }
    active_ = true;
    LOG(INFO) << "nvlink channel connected. dst=" << dst.to_string() << " same_process=" << same_process_
              << " src_shape=" << src_shape_ << " dst_shape=" << dst_shape_ << " dst_mx=" << dst_mx_
              << " mode=" << (pull_ ? "pull" : "push") << (mc_eng_ ? "+multicast" : "");
  }

  bool register_tasks(const PlanEnv& env, const std::vector<const ReqSendTask*>& tasks) override {
    fused_ = false;
    walk_ = false;
    generic_.clear();
    origin_blocks_ = merged_blocks_ = 0;
    if (n_tensors_ == 0) return false;
    PlanEnv e = env;
    e.cache_shape = src_shape_;
    PlannerChoice choice;
    try {
      choice = bind_planner(e);
    } catch (const std::exception&) {
      return false;
    }
    // requests that the destination relays to its multicast group: all of a batch or none of it
    fanout_ = 0;
    mc_batch_ = false;
    for (const ReqSendTask* t : tasks) fanout_ = std::max(fanout_, t->req().replicas > 1 ? t->req().replicas : 0u);
    if (fanout_ != 0) {
      for (const ReqSendTask* t : tasks)
        if (t->req().replicas != fanout_)
          throw KVTransferException(ErrorKind::INVALID_OPERATION, "nvlink: a batch mixes relayed and plain requests");
      const uint32_t group = static_cast<uint32_t>(dst_.ext_int("mcn", 0));
      if (mc_eng_ && group >= fanout_) {
        if (src_shape_ != dst_shape_)
          throw KVTransferException(ErrorKind::INVALID_OPERATION, "nvlink: a multicast transfer keeps the cache layout");
        mc_batch_ = true;
        return register_walk(e, choice, tasks);
      }
      if (!pull_ || group < fanout_)
        throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                  "nvlink: the destination cannot relay to " + std::to_string(fanout_) +
                                      " workers (multicast group of " + std::to_string(group) + ", pull session " +
                                      (pull_ ? "open" : "absent") + ")");
      if (src_shape_ != dst_shape_ || dst_mx_)
        throw KVTransferException(ErrorKind::INVALID_OPERATION, "nvlink: a relayed transfer keeps the cache layout");
      // the relay replicates what walk ops wrote, so these batches take the walk path whatever their shape
      return register_walk(e, choice, tasks);
    }
    if (!pull_ && !eng_)
      throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                "nvlink: this destination is reachable by multicast only (submit with fanout)");
    DeviceAttnParams p;
    std::string why = "the layer has several cache tensors";
    if (n_tensors_ != 1 || !device_attn_params(e, choice.kind, src_shape_, dst_shape_, dst_mx_, &p, &why)) {
      if (src_shape_ != dst_shape_ || dst_mx_) {
        throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                  "nvlink: cross-layout / fp8 transfer needs the fused kernel but " + why);
      }
      // every other shape (hybrid pages, MLA, KDA): the planner records walk ops and the kernel walks the
      // block tables itself; no per-piece descriptor is built or uploaded
      return register_walk(e, choice, tasks);
    }
    params_ = p;
    fused_ = true;
    plan_ = p.skip ? PackedPlan{} : pack_device_plan(tasks, 0, p.tile_tokens, p.dst.ntpb, false);
    if (plan_.n_reqs == 0) return true;     // this rank holds only replicas, or nothing is due
    moved_bytes_per_layer_ = 0;
    for (const ReqSendTask* t : tasks)
      moved_bytes_per_layer_ += static_cast<size_t>(t->new_tokens) * 2 * p.n_heads * p.src.head_bytes;
    if (pull_) {
      PullPlanHead h{};
      h.kind = PULL_KIND_ATTN;
      h.n_reqs = plan_.n_reqs;
      h.total_tiles = plan_.total_tiles;
      h.pool_offset = plan_.pool_offset;
      h.attn = p;
      send_plan(h, plan_.blob.data(), plan_.blob.size(), nullptr, 0);
      return true;
    }
    BatchEngine::SlotView sl = eng_->begin(plan_.blob.size());
    memcpy(sl.h_plan, plan_.blob.data(), plan_.blob.size());
    eng_->upload(plan_.blob.size());
    return true;
  }

  bool register_walk(const PlanEnv& e, const PlannerChoice& choice, const std::vector<const ReqSendTask*>& tasks) {
    if (env_nvlink_walk() == 0 || e.cast_bf16_to_fp8 || n_tensors_ > KVT_WALK_MAX_TENSORS) {
      if (pull_ || mc_batch_) throw KVTransferException(ErrorKind::INVALID_OPERATION, "nvlink: the pull mode needs the walk kernel for this shape");
      return false;
    }
    walk_plan_.clear();
    for (const ReqSendTask* t : tasks) plan_request_ops(choice, e, *t, walk_plan_);
    walk_plan_.finalize(ctx_->layer_num_blocks(), dst_.layer_num_blocks);
    plan_ = PackedPlan{};
    moved_bytes_per_layer_ = walk_plan_.bytes;
    origin_blocks_ = walk_plan_.ops.size();
    walk_ = true;
    walk_counts_ = KvtWalkCounts{walk_plan_.n_bulk, walk_plan_.n_simt, walk_plan_.n_zero, 0, walk_plan_.bulk_units,
                                 walk_plan_.simt_units, walk_plan_.zero_units};
    if (walk_plan_.empty()) return true;       // this rank has nothing to send (not a representative rank)
    const size_t ops_bytes = walk_plan_.ops.size() * sizeof(KvtWalkOp);
    const size_t pool_bytes = walk_plan_.pool.size() * sizeof(uint32_t);
    if (pull_ && !mc_batch_) {
      PullPlanHead h{};
      h.kind = PULL_KIND_WALK;
      h.n_ops = static_cast<uint32_t>(walk_plan_.ops.size());
      h.pool_len = static_cast<uint32_t>(walk_plan_.pool.size());
      h.walk = walk_counts_;
      h.fanout = fanout_;
      send_plan(h, walk_plan_.ops.data(), ops_bytes, walk_plan_.pool.data(), pool_bytes);
      return true;
    }
    BatchEngine& eng = mc_batch_ ? *mc_eng_ : *eng_;
    BatchEngine::SlotView sl = eng.begin(ops_bytes + pool_bytes);
    memcpy(sl.h_plan, walk_plan_.ops.data(), ops_bytes);
    memcpy(sl.h_plan + ops_bytes, walk_plan_.pool.data(), pool_bytes);
    eng.upload(ops_bytes + pool_bytes);
    return true;
  }

  void register_data(std::vector<std::vector<IpcBlock>>& data, TPKind kind) override {
    if (env_bf162fp8_conversion() && kind == TPKind::PGTD) {
      throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                "nvlink: the unscaled bf16->fp8 cast belongs to the host-staged transports; over NVLink an "
                                "fp8 decode cache is filled by the block-scaled quantiser (BLLM_KVTRANS_DST_MXFP8)");
    }
    if (pull_ || !eng_) throw KVTransferException(ErrorKind::INVALID_OPERATION, "nvlink: byte-range descriptors are a push-mode path");
    fused_ = false;
    walk_ = false;
    generic_.assign(data.size(), {});
    moved_bytes_per_layer_ = 0;
    origin_blocks_ = merged_blocks_ = 0;
    for (size_t t = 0; t < data.size(); ++t) {
      origin_blocks_ += data[t].size();
      validate_ipc_block_bounds(data[t], ctx_->tensor_capacity(t), IpcBlockOffset::SOURCE, "nvlink", 0, t);
      const MergeStats st = merge_interval(data[t]);
      merged_blocks_ += st.count;
      moved_bytes_per_layer_ += st.total_len;
      generic_[t].reserve(data[t].size());
      for (const auto& b : data[t]) generic_[t].push_back(Triple{b.src_offset, b.dst_offset, b.length});
    }
    data.clear();
    upload_generic();
  }

  // The descriptor lists are the same for every layer of the batch: upload them once instead of once per layer.
  void upload_generic() {
    size_t total = 0;
    generic_off_.assign(generic_.size(), 0);
    generic_rounds_ = 1;
    for (size_t t = 0; t < generic_.size(); ++t) {
      generic_off_[t] = total;
      total += generic_[t].size();
      if (generic_[t].empty()) continue;
      uint64_t longest = 0;
      for (const Triple& tr : generic_[t]) longest = std::max<uint64_t>(longest, tr.len);
      generic_rounds_ = std::max(generic_rounds_, kvt_bulk_rounds(generic_[t][0].len, longest));
    }
    if (total == 0) return;
    const size_t bytes = total * sizeof(Triple);
    BatchEngine::SlotView sl = eng_->begin(bytes);
    for (size_t t = 0; t < generic_.size(); ++t)
      if (!generic_[t].empty())
        memcpy(sl.h_plan + generic_off_[t] * sizeof(Triple), generic_[t].data(), generic_[t].size() * sizeof(Triple));
    eng_->upload(bytes);
  }

  bool nothing_to_send() const { return (fused_ && plan_.n_reqs == 0) || (walk_ && walk_plan_.empty()); }

  bool send_layers(size_t layer_begin, size_t layer_end, Step* step) override {
    (void)step;
    if ((!fused_ && !walk_) || layer_end <= layer_begin) return false;
    if (nothing_to_send()) return true;
    // One launch saves ~100 us of launch and event overhead, which is what matters for a small
    // migration; a large one is faster layer by layer over several streams (measured crossover
    // around half a GiB).
    if (moved_bytes_per_layer_ * (layer_end - layer_begin) > (512ull << 20)) return false;
    if (mc_batch_) {
      void* mev = ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer_end - 1));
      mc_eng_->launch_walk_multicast(walk_counts_, walk_plan_.ops.size(), walk_plan_.pool.size(), layer_begin, layer_end, 0, mev);
      return true;
    }
    if (pull_) {
      send_layers_msg(layer_begin, layer_end, true);
      return true;
    }
    // layer events are recorded in order on one stream, so the last one implies the others
    void* ev = ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer_end - 1));
    if (walk_) eng_->launch_walk(walk_counts_, walk_plan_.ops.size(), walk_plan_.pool.size(), layer_begin, layer_end, 0, ev);
    else eng_->launch_attn(params_, plan_, layer_begin, layer_end, 0, ev);
    return true;
  }

  void send_data(size_t layer, Step* step) override {
    (void)step;
    if (nothing_to_send()) return;
    if (mc_batch_) {
      mc_eng_->launch_walk_multicast(walk_counts_, walk_plan_.ops.size(), walk_plan_.pool.size(), layer, layer + 1,
                                     layer % mc_eng_->n_stages(), ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer)));
      return;
    }
    if (pull_) {
      send_layers_msg(layer, layer + 1, false);
      return;
    }
    void* ev = ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer));
    if (fused_) {
      eng_->launch_attn(params_, plan_, layer, layer + 1, layer % eng_->n_stages(), ev);
      return;
    }
    if (walk_) {
      eng_->launch_walk(walk_counts_, walk_plan_.ops.size(), walk_plan_.pool.size(), layer, layer + 1, layer % eng_->n_stages(), ev);
      return;
    }
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    DeviceStage& st = eng_->stage(layer % eng_->n_stages());
    st.wait_event(ev);
    const auto& addrs = ctx_->layer_data_address();
    RTASSERT(layer < addrs.size() && layer < dst_map_.ptrs().size());
    if (launch_generic_multi(layer, layer + 1, st)) return;
    for (size_t t = 0; t < generic_.size(); ++t) {
      if (generic_[t].empty()) continue;
      const uint64_t* d = reinterpret_cast<const uint64_t*>(eng_->current().d_plan) + generic_off_[t] * 3;
      st.launch_resident(addrs[layer][t], dst_map_.ptrs()[layer][t], d, generic_[t].size(), src_caps_.at(t), dst_caps_.at(t), 0,
                         eng_->current().d_status);
    }
  }

  // Every tensor of layers [lo, hi) in one launch when they fit the kernel's entry table.
  bool launch_generic_multi(size_t lo, size_t hi, DeviceStage& st) {
    size_t per_layer = 0;
    for (const auto& g : generic_) per_layer += g.empty() ? 0 : 1;
    if (per_layer == 0) return true;
    if (per_layer * (hi - lo) > KVT_COPY_MAX_TENSORS) return false;
    const auto& addrs = ctx_->layer_data_address();
    KvtCopyMulti m{};
    uint32_t e = 0;
    for (size_t layer = lo; layer < hi; ++layer) {
      for (size_t t = 0; t < generic_.size(); ++t) {
        if (generic_[t].empty()) continue;
        m.src_base[e] = addrs[layer][t];
        m.dst_base[e] = dst_map_.ptrs()[layer][t];
        m.src_cap[e] = src_caps_.at(t);
        m.dst_cap[e] = dst_caps_.at(t);
        m.first[e] = static_cast<uint32_t>(generic_off_[t]);
        m.count[e] = static_cast<uint32_t>(generic_[t].size());
        ++e;
      }
    }
    m.n_tensors = e;
    m.triples = reinterpret_cast<const uint64_t*>(eng_->current().d_plan);
    m.status = eng_->current().d_status;
    if (env_use_tma() != 0) {
      // pages are long 16-byte aligned runs: the TMA engine moves them, four CTAs per SM
      const int grid = std::max(1, static_cast<int>(4 * kvt_sm_count(ctx_->device_id()) * env_kernel_copy_sm_usage()));
      cuda_check(kvt_launch_copy_blocks_bulk(&m, generic_rounds_, grid, st.stream()), "kvt_launch_copy_blocks_bulk");
      return true;
    }
    const int grid = std::max(1, static_cast<int>(2 * kvt_sm_count(ctx_->device_id()) * env_kernel_copy_sm_usage()));
    cuda_check(kvt_launch_copy_blocks_multi(&m, grid, st.stream()), "kvt_launch_copy_blocks_multi");
    return true;
  }

  size_t send_range(size_t lo, size_t hi, Step* step) override {
    if (nothing_to_send()) return hi - lo;
    if (mc_batch_) {
      // the layers recorded so far in one launch, behind the last of their events
      const size_t n = std::min<size_t>(hi - lo, 8);
      mc_eng_->launch_walk_multicast(walk_counts_, walk_plan_.ops.size(), walk_plan_.pool.size(), lo, lo + n, mc_eng_->next_stage(),
                                     ctx_->cuda_barrier()->event(static_cast<uint32_t>(lo + n - 1)));
      return n;
    }
    if (pull_) {
      // one message for everything recorded so far; the session launches layer by layer (attention) or once (walk)
      const size_t n = walk_ ? std::min<size_t>(hi - lo, 8) : hi - lo;
      send_layers_msg(lo, lo + n, false);
      return n;
    }
    if (fused_ || hi <= lo + 1) {   // the fused kernel gains nothing from longer launches (measured)
      send_data(lo, step);
      return 1;
    }
    if (walk_) {
      // the layers recorded so far leave in one launch: short per-layer work (state pages, MLA tokens) would
      // otherwise be bounded by the launch rate
      const size_t n = std::min<size_t>(hi - lo, 8);
      eng_->launch_walk(walk_counts_, walk_plan_.ops.size(), walk_plan_.pool.size(), lo, lo + n, eng_->next_stage(),
                        ctx_->cuda_barrier()->event(static_cast<uint32_t>(lo + n - 1)));
      return n;
    }
    size_t per_layer = 0;
    for (const auto& g : generic_) per_layer += g.empty() ? 0 : 1;
    const size_t fit = per_layer == 0 ? hi - lo : KVT_COPY_MAX_TENSORS / per_layer;
    const size_t n = std::max<size_t>(1, std::min(hi - lo, fit));
    if (n == 1) {
      send_data(lo, step);
      return 1;
    }
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    const auto& addrs = ctx_->layer_data_address();
    RTASSERT(lo + n <= addrs.size() && lo + n <= dst_map_.ptrs().size());
    DeviceStage& st = eng_->stage(eng_->next_stage());
    // layer events are recorded in order on one stream: the last of the range implies the others
    st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(lo + n - 1)));
    if (!launch_generic_multi(lo, lo + n, st)) {
      send_data(lo, step);
      return 1;
    }
    return n;
  }

  bool async_flush() const override { return true; }
  bool relays_to_group() const override { return (pull_ || mc_eng_) && dst_.ext_int("mcn", 0) > 1; }

  std::string metrics_prefix() const {
    std::ostringstream ss;
    ss << "Proto=nvlink,Mode=" << (mc_batch_ ? "multicast" : (pull_ ? "pull" : "push")) << ",Path="
       << (fused_ ? "fused" : (walk_ ? "walk" : "descriptors"))
       << ",OriginSbNum=" << origin_blocks_ << ",MergedSbNum=" << merged_blocks_ << ",BytesPerLayer=" << moved_bytes_per_layer_
       << ",Tiles=" << (walk_ ? walk_plan_.bulk_units + walk_plan_.simt_units : plan_.total_tiles);
    if (fanout_ > 1) ss << ",Fanout=" << fanout_;
    return ss.str();
  }

  // Enqueue the batch's completion record and return its ticket; nothing here waits for the GPU.
  uint64_t flush_async() override {
    fault_inject_throw();
    const bool drop = fault_inject_drop_completion();
    TimeWatch tw;
    uint64_t ticket = 0;
    if (mc_batch_) {
      cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
      ticket = mc_eng_->flush_async(metrics_prefix(), drop) | kMcTicket;
      mc_batch_ = false;
      std::lock_guard<std::mutex> g(pull_mu_);
      pull_metrics_[ticket] = ",FlushUs=" + std::to_string(tw.get_elapse_us());
    } else if (pull_) {
      if (!pull_batch_open_) {        // a batch without data still completes through the session, in order
        PullPlanHead h{};
        h.kind = PULL_KIND_WALK;
        send_plan(h, nullptr, 0, nullptr, 0);
      }
      std::string msg(RPC_HEADER, '\0');
      put_rpc_header(msg.data(), PULL_FLUSH_REQ, pull_seq_);
      put(msg, static_cast<uint8_t>(drop ? 1 : 0));
      send_msg(msg);
      ticket = pull_seq_;
      pull_batch_open_ = false;
      std::lock_guard<std::mutex> g(pull_mu_);
      pull_metrics_[ticket] = metrics_prefix() + ",FlushUs=" + std::to_string(tw.get_elapse_us());
    } else {
      cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
      ticket = eng_->flush_async(metrics_prefix(), drop);
      std::lock_guard<std::mutex> g(pull_mu_);
      pull_metrics_[ticket] = ",FlushUs=" + std::to_string(tw.get_elapse_us());
    }
    generic_.clear();
    return ticket;
  }

  PollResult poll_completion(uint64_t ticket, std::string& out) override {
    BatchEngine::Done d;
    std::string tail;
    if ((ticket & kMcTicket) != 0) {
      const PollResult r = mc_eng_ ? mc_eng_->poll(ticket & ~kMcTicket, &d) : PollResult::FAILED;
      if (r == PollResult::PENDING) return r;
      if (r == PollResult::FAILED) {
        out = "completion ticket unknown";
        return r;
      }
      std::lock_guard<std::mutex> g(pull_mu_);
      auto mt = pull_metrics_.find(ticket);
      if (mt != pull_metrics_.end()) {
        tail = mt->second;
        pull_metrics_.erase(mt);
      }
    } else if (pull_) {
      std::lock_guard<std::mutex> g(pull_mu_);
      drain_done_frames();
      auto it = pull_done_.find(ticket);
      if (it == pull_done_.end()) {
        if (pull_broken_) {
          out = "the pull session's connection broke";
          active_ = false;
          return PollResult::FAILED;
        }
        return PollResult::PENDING;
      }
      d = it->second;
      pull_done_.erase(it);
      auto mt = pull_metrics_.find(ticket);
      if (mt != pull_metrics_.end()) {
        d.metrics = mt->second;
        pull_metrics_.erase(mt);
      }
    } else {
      const PollResult r = eng_->poll(ticket, &d);
      if (r == PollResult::PENDING) return r;
      if (r == PollResult::FAILED) {
        out = "completion ticket unknown";
        return r;
      }
      std::lock_guard<std::mutex> g(pull_mu_);
      auto mt = pull_metrics_.find(ticket);
      if (mt != pull_metrics_.end()) {
        tail = mt->second;
        pull_metrics_.erase(mt);
      }
    }
    std::ostringstream ss;
    ss << d.metrics << tail;
    if (d.t_start_ns != 0 && d.t_end_ns >= d.t_start_ns) ss << ",DeviceUs=" << (d.t_end_ns - d.t_start_ns) / 1000;
    if (d.status != 0) {
      ss << ",KernelStatus=" << d.status << ",Detail=" << d.detail;
      out = ss.str();
      active_ = false;     // the next batch gets a fresh channel
      return PollResult::FAILED;
    }
    out = ss.str();
    return PollResult::DONE;
  }

  // The synchronous form, for callers that have nothing else to do: the same record, polled here.
  void flush(std::string& out) override {
    const uint64_t ticket = flush_async();
    const Timepoint deadline = SteadyClock::now() + std::chrono::milliseconds(env_completion_timeout_ms());
    for (int spins = 0;; ++spins) {
      const PollResult r = poll_completion(ticket, out);
      if (r == PollResult::DONE) return;
      if (r == PollResult::FAILED) throw KVTransferException(ErrorKind::CUDA, "transfer failed: " + out);
      if (SteadyClock::now() > deadline) {
        active_ = false;
        throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: the completion record of a batch did not arrive");
      }
      if (spins < 2000) std::this_thread::yield(); else std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
  }

  bool is_active() override { return active_; }

  void close() override {
    active_ = false;
    if (ctx_->device_id() >= 0) cudaSetDevice(ctx_->device_id());
    if (eng_) eng_->close();
    eng_.reset();
    if (mc_eng_) mc_eng_->close();
    mc_eng_.reset();
    pull_sock_.reset();      // the server ends the session when the connection goes away
    dst_map_.release();
  }

 private:
  // ---- pull mode: messages to the session ------------------------------------------------------------
  bool open_pull(FdGuard& sock) {
    const PeerMemInfo mine = export_peer_mem_info(ctx_);
    const PeerEvents evs = export_peer_events(ctx_);
    if (evs.events.size() != ctx_->num_layers()) return false;
    if (!same_process_)
      for (const auto& e : evs.events)
        if (!e.has_handle) return false;      // layer events were not created for interprocess use
    std::string msg(RPC_HEADER, '\0');
    put_rpc_header(msg.data(), PULL_OPEN_REQ, new_id());
    put(msg, pull_protocol_version());
    put(msg, static_cast<uint32_t>(src_caps_.size()));
    for (uint64_t c : src_caps_) put(msg, c);
    const std::string mem = mine.serialize(), ev = evs.serialize();
    put(msg, static_cast<uint32_t>(mem.size()));
    msg += mem;
    put(msg, static_cast<uint32_t>(ev.size()));
    msg += ev;
    std::string resp;
    if (!send_frame(sock.fd(), msg.data(), msg.size(), env_rpc_timeout_s() * 1000) ||
        !recv_frame(sock.fd(), resp, env_rpc_timeout_s() * 1000) || resp.size() < RPC_HEADER + 4) {
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: pull-session request failed");
    }
    uint32_t status = 0;
    memcpy(&status, resp.data() + RPC_HEADER, 4);
    if (status != WIRE_OK) LOG(INFO) << "nvlink: destination offers no pull session (status " << status << "), pushing";
    return status == WIRE_OK;
  }

  void send_msg(const std::string& msg) {
    if (!send_frame(pull_sock_.fd(), msg.data(), msg.size(), env_rpc_timeout_s() * 1000)) {
      active_ = false;
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: the pull session's connection broke");
    }
  }

  void send_plan(const PullPlanHead& head, const void* a, size_t a_len, const void* b, size_t b_len) {
    PullPlanHead h = head;
    h.blob_bytes = a_len + b_len;
    ++pull_seq_;
    std::string msg(RPC_HEADER, '\0');
    put_rpc_header(msg.data(), PULL_PLAN_REQ, pull_seq_);
    msg.append(reinterpret_cast<const char*>(&h), sizeof(h));
    if (a_len) msg.append(static_cast<const char*>(a), a_len);
    if (b_len) msg.append(static_cast<const char*>(b), b_len);
    send_msg(msg);
    pull_batch_open_ = true;
  }

  void send_layers_msg(size_t lo, size_t hi, bool one_launch) {
    std::string msg(RPC_HEADER, '\0');
    put_rpc_header(msg.data(), PULL_LAYERS_REQ, pull_seq_);
    put(msg, static_cast<uint32_t>(lo));
    put(msg, static_cast<uint32_t>(hi));
    put(msg, static_cast<uint8_t>(one_launch ? 1 : 0));
    send_msg(msg);
  }

  // pull_mu_ held.  Reads whatever PULL_DONE frames have arrived, without blocking.
  void drain_done_frames() {
    if (!pull_sock_.valid() || pull_broken_) return;
    for (;;) {
      char tmp[4096];
      const ssize_t n = ::recv(pull_sock_.fd(), tmp, sizeof(tmp), MSG_DONTWAIT);
      if (n > 0) {
        pull_rx_.append(tmp, static_cast<size_t>(n));
        continue;
      }
      if (n == 0 || (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) pull_broken_ = true;
      break;
    }
    size_t off = 0;
    while (pull_rx_.size() - off >= 4) {
      uint32_t len = 0;
      memcpy(&len, pull_rx_.data() + off, 4);
      if (pull_rx_.size() - off - 4 < len) break;
      const char* p = pull_rx_.data() + off + 4;
      if (len >= RPC_HEADER + 24) {
        uint32_t magic = 0;
        uint64_t seq = 0;
        get_rpc_header(p, &magic, &seq);
        if (magic == PULL_DONE) {
          BatchEngine::Done d;
          memcpy(&d.status, p + RPC_HEADER, 4);
          memcpy(&d.detail, p + RPC_HEADER + 4, 4);
          memcpy(&d.t_start_ns, p + RPC_HEADER + 8, 8);
          memcpy(&d.t_end_ns, p + RPC_HEADER + 16, 8);
          pull_done_[seq] = d;
        }
      }
      off += 4 + len;
    }
    if (off) pull_rx_.erase(0, off);
  }

  Context* ctx_;
  WorkerInfo dst_;
  bool active_{false};
  PeerMapping dst_map_;
  uint32_t n_tensors_{0};
  std::vector<uint64_t> src_caps_, dst_caps_;
  std::unique_ptr<BatchEngine> eng_;     // push mode
  std::unique_ptr<BatchEngine> mc_eng_;  // this GPU holds a mapping of the destination group's multicast object
  bool mc_batch_{false};                 // the batch being assembled leaves through mc_eng_
  bool push_unavailable_{false};         // the destination cache has no IPC handle and no pull session serves it
  static constexpr uint64_t kMcTicket = 1ull << 63;   // marks the tickets of such batches
  int src_shape_{0}, dst_shape_{0};
  bool dst_mx_{false};
  bool dst_remote_{false};       // the destination cache lives on another GPU
  bool same_process_{false};
  // what the current batch is
  bool fused_{false}, walk_{false};
  uint32_t fanout_{0};           // > 1: the destination relays this batch to that many workers of its group
  DeviceAttnParams params_{};
  PackedPlan plan_;
  WalkPlan walk_plan_;
  KvtWalkCounts walk_counts_{};
  // pull mode
  bool pull_{false};
  FdGuard pull_sock_;
  uint64_t pull_seq_{0};
  bool pull_batch_open_{false};
  std::mutex pull_mu_;                                   // shared with the completion poller's thread
  std::string pull_rx_;
  std::map<uint64_t, BatchEngine::Done> pull_done_;
  std::map<uint64_t, std::string> pull_metrics_;
  bool pull_broken_{false};
  // descriptor path (push only)
  uint32_t generic_rounds_{1};   // bulk copy kernel: segment rounds the longest descriptor needs
  std::vector<std::vector<Triple>> generic_;
  std::vector<size_t> generic_off_;   // first descriptor of each tensor inside the uploaded buffer
  size_t origin_blocks_{0}, merged_blocks_{0}, moved_bytes_per_layer_{0};
};

}  // namespace

Channel make_nvlink_channel(Context* ctx) { return std::make_shared<NvlinkChannel>(ctx); }

Channel ChannelFactory::create(const WorkerInfo& dst) {
  const uint8_t mine = ctx_->worker_info().transfer_protocols;
  const uint8_t theirs = dst.transfer_protocols;
  auto both = [&](TransferProtocol::Kind k) { return (mine & k) != 0 && (theirs & k) != 0; };
  const std::string host = dst.ext_str("host");
  const bool same_host = !host.empty() && host == std::to_string(this_host_id());
  TransferProtocol::Kind pick = TransferProtocol::UNKNOWN;
  if (proto_.has_value()) {
    pick = proto_->type;
  } else if (both(TransferProtocol::NVLINK) && same_host && ctx_->device_id() >= 0 && dst.ext_int("dev", -1) >= 0) {
    pick = TransferProtocol::NVLINK;
  } else if (both(TransferProtocol::SHM) && same_host) {
    pick = TransferProtocol::SHM;
  } else if (both(TransferProtocol::TCP)) {
    pick = TransferProtocol::TCP;
  }
  Channel ch;
  switch (pick) {
    case TransferProtocol::NVLINK: ch = make_nvlink_channel(ctx_); break;
    case TransferProtocol::SHM: ch = make_tcp_channel(ctx_, true); break;
    case TransferProtocol::TCP: ch = make_tcp_channel(ctx_, false); break;
    default:
      throw KVTransferException(ErrorKind::TRANSPORT, "no transfer protocol in common with " + dst.to_string());
  }
  ch->connect(dst);
  return ch;
}

}  // namespace kvx
