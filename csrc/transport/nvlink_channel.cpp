// NVLink transport: kernels on the prefill GPU store straight into the decode GPU's paged
// cache through peer-mapped memory (NVLink 5 / NVSwitch).  No staging buffer, no library copy.
//
// connect() asks the destination's server for the CUDA IPC handles of its layer tensors
// (MEM_HANDLES_REQ) and maps them; a destination in the same process is used by pointer after
// enabling peer access.  Two data paths share the channel:
//   * fused:   register_tasks() packs the requests' block tables; send_data(layer) launches
//              kvt_p2d_attn, which walks the tables, converts the layout (NHD<->HND), re-shards
//              heads for TP-mismatched pairs, optionally quantises to block-scaled e4m3 and
//              stores into the peer cache.  Serves cache shapes 1, 2 and 5 on either side.
//   * generic: register_data() takes the planner's IpcBlocks (any cache shape, including hybrid
//              GDN / MLA / KDA pages) and send_data(layer) runs the descriptor-driven copy
//              kernel from the local tensor into the peer tensor.
// The channel is device ordered: send_data(layer) makes its stream wait for the layer's CUDA
// event and returns; nothing on the host waits for the forward pass.  Nothing on the host waits for
// the transfer either: flush_async() enqueues a completion record (sequence number, kernel status
// words, GPU timer stamps, written into mapped host memory by a one-thread kernel) behind the batch
// and returns; the completion poller reads the record and finishes the batch.  Every batch runs in
// one of a few plan slots (device + pinned plan buffer, status block, record, a small stream), sized
// once at connect from the caches' block counts, so the step path neither allocates nor frees.
// Only plain peer stores are used here; loads with cluster multicast are never issued.
#include <cuda_runtime.h>
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
#include "transport/channel.h"
#include "transport/device_stage.h"
#include "transport/wire.h"

namespace kvx {

namespace {

// IPC mappings are per process: a handle is opened once and shared by every channel that maps the same
// allocation, and closed when the last of them goes away.  The key is the handle itself, which names one
// allocation of one process: a peer that restarted (even with a recycled pid and the same addresses) hands
// out different handles, so nothing is ever written through a mapping of memory that no longer exists.
struct IpcCache {
  struct Mapping {
    uint64_t local = 0;
    uint32_t refs = 0;
  };
  std::mutex mu;
  std::map<std::string, Mapping> mapped;   // 64 handle bytes -> local address
  uint64_t acquire(const char* handle64) {
    std::lock_guard<std::mutex> g(mu);
    const std::string key(handle64, 64);
    auto it = mapped.find(key);
    if (it == mapped.end()) {
      uint64_t local = 0;
      cuda_check(kvt_ipc_open_handle(handle64, &local), "cudaIpcOpenMemHandle");
      it = mapped.emplace(key, Mapping{local, 0}).first;
    }
    ++it->second.refs;
    return it->second.local;
  }
  void release(const std::string& key) {
    std::lock_guard<std::mutex> g(mu);
    auto it = mapped.find(key);
    if (it == mapped.end()) return;
    if (--it->second.refs == 0) {
      kvt_ipc_close(it->second.local);
      mapped.erase(it);
    }
  }
  size_t size() {
    std::lock_guard<std::mutex> g(mu);
    return mapped.size();
  }
};
IpcCache& ipc_cache() {
  static IpcCache& c = *new IpcCache;   // never destroyed: channels may close while the process exits
  return c;
}

template <typename T>
struct DevArray {
  T* p{nullptr};
  size_t n{0};
  ~DevArray() {
    if (p != nullptr) cudaFree(p);
  }
  void upload(const std::vector<T>& v) {
    if (p != nullptr) cudaFree(p);
    p = nullptr;
    n = v.size();
    if (n == 0) return;
    cuda_check(cudaMalloc(reinterpret_cast<void**>(&p), n * sizeof(T)), "cudaMalloc");
    cuda_check(cudaMemcpy(p, v.data(), n * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
  }
};

struct alignas(64) TensorMapBytes {
  char b[128];
};

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
    const bool same_process = info.pid == static_cast<int32_t>(getpid());
    dst_remote_ = info.device != ctx_->device_id();
    if (info.device != ctx_->device_id() && same_process) {
      if (!kvt_can_access_peer(ctx_->device_id(), info.device))
        throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: no peer access to the destination GPU");
      cuda_check(kvt_enable_peer_access(ctx_->device_id(), info.device), "cudaDeviceEnablePeerAccess");
    }
    dst_ptrs_.assign(info.num_layers, std::vector<uint64_t>(info.num_tensors, 0));
    for (uint32_t l = 0; l < info.num_layers; ++l) {
      for (uint32_t t = 0; t < info.num_tensors; ++t) {
        const PeerTensor& pt = info.tensors[static_cast<size_t>(l) * info.num_tensors + t];
        if (same_process) {
          dst_ptrs_[l][t] = pt.ptr;
          continue;
        }
        if (!pt.has_handle) throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: destination tensor has no IPC handle");
        const std::string key(pt.ipc_handle, 64);
        uint64_t local = 0;
        for (size_t k = 0; k < ipc_keys_.size() && local == 0; ++k)
          if (ipc_keys_[k] == key) local = ipc_locals_[k];
        if (local == 0) {      // one reference per allocation and channel
          local = ipc_cache().acquire(pt.ipc_handle);
          ipc_keys_.push_back(key);
          ipc_locals_.push_back(local);
        }
        dst_ptrs_[l][t] = local + (pt.ptr - pt.alloc_base);
      }
    }
    // ---- streams and plan slots -------------------------------------------------------------
    const int n_streams = std::max(1, env_nvlink_streams());
    for (int i = 0; i < n_streams; ++i) stages_.emplace_back(std::make_unique<DeviceStage>(ctx_->device_id()));
    // A plan holds one descriptor per request and the block tables of both sides.  Sized for every block of
    // both caches in every block group, plus room for a few thousand request descriptors.
    const size_t groups = std::max<size_t>(1, ctx_->worker_info().num_gdn_layers + ctx_->worker_info().num_ple_layers + 2);
    const size_t table = (static_cast<size_t>(ctx_->layer_num_blocks()) + dst.layer_num_blocks) * sizeof(uint32_t);
    alloc_slots(std::max<size_t>(table * std::min<size_t>(groups, 8) + (1u << 20), 2u << 20));
    src_shape_ = ctx_->worker_info().cache_shape_or(env_cache_shape());
    dst_shape_ = dst.cache_shape_or(src_shape_);
    dst_mx_ = dst.ext_int("mx", env_dst_mxfp8()) != 0;
    active_ = true;
    LOG(INFO) << "nvlink channel connected. dst=" << dst.to_string() << " same_process=" << same_process
              << " src_shape=" << src_shape_ << " dst_shape=" << dst_shape_ << " dst_mx=" << dst_mx_;
  }

  bool register_tasks(const PlanEnv& env, const std::vector<const ReqSendTask*>& tasks) override {
    fused_ = false;
    walk_ = false;
    generic_.clear();
    origin_blocks_ = merged_blocks_ = 0;
    if (dst_ptrs_.empty()) return false;
    PlanEnv e = env;
    e.cache_shape = src_shape_;
    PlannerChoice choice;
    try {
      choice = bind_planner(e);
    } catch (const std::exception&) {
      return false;
    }
    DeviceAttnParams p;
    std::string why = "the layer has several cache tensors";
    if (dst_ptrs_[0].size() != 1 || !device_attn_params(e, choice.kind, src_shape_, dst_shape_, dst_mx_, &p, &why)) {
      if (src_shape_ != dst_shape_ || dst_mx_) {
        throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                  "nvlink: cross-layout / fp8 transfer needs the fused kernel but " + why);
      }
      // every other shape (hybrid pages, MLA, KDA): the planner records walk ops and the kernel walks the
      // block tables itself; no per-piece descriptor is built or uploaded
      return register_walk(e, choice, tasks);
    }
    params_ = p;
    if (p.skip) {
      plan_ = PackedPlan{};
      fused_ = true;
      return true;
    }
    plan_ = pack_device_plan(tasks, 0, p.tile_tokens, p.dst.ntpb, false);
    if (plan_.n_reqs == 0) {
      fused_ = true;
      return true;
    }
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    ensure_layer_arrays();
    // upload the plan on the slot's stream; the transfer streams wait for it when the batch first uses them
    Slot& sl = begin_slot(plan_.blob.size());
    memcpy(sl.h_plan, plan_.blob.data(), plan_.blob.size());
    upload_slot(sl, plan_.blob.size());
    fused_ = true;
    moved_bytes_per_layer_ = 0;
    for (const ReqSendTask* t : tasks)
      moved_bytes_per_layer_ += static_cast<size_t>(t->new_tokens) * 2 * p.n_heads * p.src.head_bytes;
    return true;
  }

  bool register_walk(const PlanEnv& e, const PlannerChoice& choice, const std::vector<const ReqSendTask*>& tasks) {
    if (env_nvlink_walk() == 0 || e.cast_bf16_to_fp8 || dst_ptrs_[0].size() > KVT_WALK_MAX_TENSORS) return false;
    walk_plan_.clear();
    for (const ReqSendTask* t : tasks) plan_request_ops(choice, e, *t, walk_plan_);
    walk_plan_.finalize(ctx_->layer_num_blocks(), dst_.layer_num_blocks);
    plan_ = PackedPlan{};
    moved_bytes_per_layer_ = walk_plan_.bytes;
    walk_ = true;
    if (walk_plan_.empty()) return true;       // this rank has nothing to send (not a representative rank)
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    ensure_walk_arrays();
    const size_t ops_bytes = walk_plan_.ops.size() * sizeof(KvtWalkOp);
    const size_t bytes = ops_bytes + walk_plan_.pool.size() * sizeof(uint32_t);
    Slot& sl = begin_slot(bytes);
    memcpy(sl.h_plan, walk_plan_.ops.data(), ops_bytes);
    memcpy(sl.h_plan + ops_bytes, walk_plan_.pool.data(), walk_plan_.pool.size() * sizeof(uint32_t));
    upload_slot(sl, bytes);
    origin_blocks_ = walk_plan_.ops.size();
    return true;
  }

  void launch_walk(size_t layer_begin, size_t layer_end, DeviceStage& st) {
    KvtWalkLaunch a{};
    a.src_ptrs = d_walk_src_.p;
    a.dst_ptrs = d_walk_dst_.p;
    a.n_tensors = static_cast<uint32_t>(dst_ptrs_[0].size());
    a.layer_begin = static_cast<uint32_t>(layer_begin);
    a.layer_end = static_cast<uint32_t>(layer_end);
    for (uint32_t t = 0; t < a.n_tensors; ++t) {
      a.src_cap[t] = ctx_->tensor_capacity(t);
      a.dst_cap[t] = dst_.block_sizes.at(t) * static_cast<uint64_t>(dst_.layer_num_blocks);
    }
    a.ops = reinterpret_cast<const KvtWalkOp*>(cur().d_plan);
    a.n_bulk_ops = walk_plan_.n_bulk;
    a.n_simt_ops = walk_plan_.n_simt;
    a.bulk_units = walk_plan_.bulk_units;
    a.simt_units = walk_plan_.simt_units;
    a.pool = reinterpret_cast<const uint32_t*>(cur().d_plan + walk_plan_.ops.size() * sizeof(KvtWalkOp));
    a.pool_len = static_cast<uint32_t>(walk_plan_.pool.size());
    a.status = cur().d_status;
    int grid = env_nvlink_ctas();
    if (grid <= 0) grid = std::max(1, static_cast<int>(4 * kvt_sm_count(ctx_->device_id()) * env_kernel_copy_sm_usage()));
    if (a.n_bulk_ops + a.n_simt_ops != 0) cuda_check(kvt_launch_walk(&a, grid, st.stream()), "kvt_launch_walk");
    if (walk_plan_.n_zero != 0) {
      // tail padding lands after the copies (same stream): where both touch a byte, the zero wins, as it does
      // when the byte ranges are applied in the planner's order
      a.ops += walk_plan_.n_bulk + walk_plan_.n_simt;
      a.n_bulk_ops = 0;
      a.bulk_units = 0;
      a.n_simt_ops = walk_plan_.n_zero;
      a.simt_units = walk_plan_.zero_units;
      cuda_check(kvt_launch_walk(&a, grid, st.stream()), "kvt_launch_walk(zero fill)");
    }
  }

  void ensure_walk_arrays() {
    if (d_walk_src_.p != nullptr) return;
    std::vector<uint64_t> src, dst;
    for (const auto& l : ctx_->layer_data_address()) src.insert(src.end(), l.begin(), l.end());
    for (const auto& l : dst_ptrs_) dst.insert(dst.end(), l.begin(), l.end());
    RTASSERT(src.size() == dst.size());
    d_walk_src_.upload(src);
    d_walk_dst_.upload(dst);
  }

  void register_data(std::vector<std::vector<IpcBlock>>& data, TPKind kind) override {
    if (env_bf162fp8_conversion() && kind == TPKind::PGTD) {
      throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                "nvlink: the unscaled bf16->fp8 cast belongs to the host-staged transports; over NVLink an "
                                "fp8 decode cache is filled by the block-scaled quantiser (BLLM_KVTRANS_DST_MXFP8)");
    }
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

  // The descriptor lists are the same for every layer of the batch: upload them once (on stream 0,
  // the other streams wait for the upload) instead of once per layer.
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
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    const size_t bytes = total * sizeof(Triple);
    Slot& sl = begin_slot(bytes);
    for (size_t t = 0; t < generic_.size(); ++t)
      if (!generic_[t].empty())
        memcpy(sl.h_plan + generic_off_[t] * sizeof(Triple), generic_[t].data(), generic_[t].size() * sizeof(Triple));
    upload_slot(sl, bytes);
  }

  bool send_layers(size_t layer_begin, size_t layer_end, Step* step) override {
    (void)step;
    if ((!fused_ && !walk_) || layer_end <= layer_begin) return false;
    if (walk_ ? walk_plan_.empty() : plan_.n_reqs == 0) return true;
    // One launch saves ~100 us of launch and event overhead, which is what matters for a small
    // migration; a large one is faster layer by layer over several streams (measured crossover
    // around half a GiB).
    if (moved_bytes_per_layer_ * (layer_end - layer_begin) > (512ull << 20)) return false;
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    // one launch over the layer range on the stream that carried the plan; layer events are
    // recorded in order on one stream, so the last one implies the others
    DeviceStage& st = use_stage(0);
    st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer_end - 1)));
    if (walk_) launch_walk(layer_begin, layer_end, st); else launch_fused(layer_begin, layer_end, st);
    return true;
  }

  void launch_fused(size_t layer_begin, size_t layer_end, DeviceStage& st) {
    {
      KvtAttnLaunch a{};
      a.src_layers = d_src_layers_.p;
      a.dst_layers = d_dst_layers_.p;
      a.src_maps = use_tma_ ? d_src_maps_.p : nullptr;
      a.dst_maps = use_tma_ ? d_dst_maps_.p : nullptr;
      a.src = params_.src;
      a.dst = params_.dst;
      a.layer_begin = static_cast<uint32_t>(layer_begin);
      a.layer_end = static_cast<uint32_t>(layer_end);
      a.reqs = reinterpret_cast<const KvtReqDesc*>(cur().d_plan);
      a.n_reqs = plan_.n_reqs;
      a.total_tiles = plan_.total_tiles;
      a.block_ids = reinterpret_cast<const uint32_t*>(cur().d_plan + plan_.pool_offset);
      a.tile_tokens = params_.tile_tokens;
      a.src_head0 = params_.src_head0;
      a.dst_head0 = params_.dst_head0;
      a.n_heads = params_.n_heads;
      a.mode = params_.mode;
      a.status = cur().d_status;
      a.dst_remote = dst_remote_ ? 1u : 0u;
      a.tile_order = tile_order_;
      a.store_form = store_form_;
      int grid = env_nvlink_ctas();
      // four small CTAs per SM, scaled by the SM-usage knob that bounds what a transfer may take from the forward pass
      if (grid <= 0) grid = std::max(1, static_cast<int>(4 * kvt_sm_count(ctx_->device_id()) * env_kernel_copy_sm_usage()));
      cuda_check(kvt_launch_p2d_attn(&a, grid, 0, use_tma_ ? 1 : 0, st.stream()), "kvt_launch_p2d_attn");
    }
  }

  void send_data(size_t layer, Step* step) override {
    (void)step;
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    if ((fused_ && plan_.n_reqs == 0) || (walk_ && walk_plan_.empty())) return;   // nothing to send from this rank
    DeviceStage& st = use_stage(layer % stages_.size());
    st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer)));
    if (fused_) {
      if (plan_.n_reqs != 0) launch_fused(layer, layer + 1, st);
      return;
    }
    if (walk_) {
      if (!walk_plan_.empty()) launch_walk(layer, layer + 1, st);
      return;
    }
    const auto& addrs = ctx_->layer_data_address();
    RTASSERT(layer < addrs.size() && layer < dst_ptrs_.size());
    if (launch_generic_multi(layer, layer + 1, st)) return;
    for (size_t t = 0; t < generic_.size(); ++t) {
      if (generic_[t].empty()) continue;
      const size_t dst_cap = dst_.block_sizes.at(t) * static_cast<size_t>(dst_.layer_num_blocks);
      const uint64_t* d = reinterpret_cast<const uint64_t*>(cur().d_plan) + generic_off_[t] * 3;
      st.launch_resident(addrs[layer][t], dst_ptrs_[layer][t], d, generic_[t].size(), ctx_->tensor_capacity(t), dst_cap, 0,
                         cur().d_status);
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
        m.dst_base[e] = dst_ptrs_[layer][t];
        m.src_cap[e] = ctx_->tensor_capacity(t);
        m.dst_cap[e] = dst_.block_sizes.at(t) * static_cast<uint64_t>(dst_.layer_num_blocks);
        m.first[e] = static_cast<uint32_t>(generic_off_[t]);
        m.count[e] = static_cast<uint32_t>(generic_[t].size());
        ++e;
      }
    }
    m.n_tensors = e;
    m.triples = reinterpret_cast<const uint64_t*>(cur().d_plan);
    m.status = cur().d_status;
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
    if (fused_ || hi <= lo + 1) {   // the fused kernel gains nothing from longer launches (measured)
      send_data(lo, step);
      return 1;
    }
    if (walk_) {
      // the layers recorded so far leave in one launch: short per-layer work (state pages, MLA tokens) would
      // otherwise be bounded by the launch rate
      if (walk_plan_.empty()) return hi - lo;
      cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
      const size_t n = std::min<size_t>(hi - lo, 8);
      DeviceStage& st = use_stage((range_rr_++) % stages_.size());
      st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(lo + n - 1)));
      launch_walk(lo, lo + n, st);
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
    RTASSERT(lo + n <= addrs.size() && lo + n <= dst_ptrs_.size());
    DeviceStage& st = use_stage((range_rr_++) % stages_.size());
    // layer events are recorded in order on one stream: the last of the range implies the others
    st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(lo + n - 1)));
    if (!launch_generic_multi(lo, lo + n, st)) {
      send_data(lo, step);
      return 1;
    }
    return n;
  }

  bool async_flush() const override { return true; }

  // Enqueue the batch's completion record and return its ticket; nothing here waits for the GPU.
  uint64_t flush_async() override {
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    fault_inject_throw();
    if (batch_slot_ < 0) begin_slot(0);     // a batch without data still completes through a record
    Slot& sl = cur();
    cudaStream_t ss = sl.stream;
    // the slot's stream joins the transfer streams the batch used, and the previous batch's record
    for (size_t i = 0; i < stages_.size() && i < stage_used_.size(); ++i)
      if (stage_used_[i]) cuda_check(cudaStreamWaitEvent(ss, static_cast<cudaEvent_t>(stages_[i]->record_done()), 0), "cudaStreamWaitEvent");
    if (last_done_event_ != nullptr && last_done_event_ != sl.done_event)
      cuda_check(cudaStreamWaitEvent(ss, last_done_event_, 0), "cudaStreamWaitEvent");
    if (!fault_inject_drop_completion())
      cuda_check(kvt_launch_complete(sl.d_status, sl.d_rec, sl.seq, ss), "kvt_launch_complete");
    cuda_check(cudaEventRecord(sl.done_event, ss), "cudaEventRecord");
    last_done_event_ = sl.done_event;
    std::ostringstream ss_m;
    ss_m << "Proto=nvlink,Path=" << (fused_ ? "fused" : (walk_ ? "walk" : "descriptors")) << ",OriginSbNum=" << origin_blocks_
         << ",MergedSbNum=" << merged_blocks_ << ",BytesPerLayer=" << moved_bytes_per_layer_ << ",Tiles=" << (walk_ ? walk_plan_.bulk_units + walk_plan_.simt_units : plan_.total_tiles);
    {
      std::lock_guard<std::mutex> g(slot_mu_);
      sl.metrics = ss_m.str();
      sl.flushed_at = SteadyClock::now();
      sl.pending = true;
    }
    const uint64_t ticket = sl.seq;
    batch_slot_ = -1;
    generic_.clear();
    begin_batch();
    return ticket;
  }

  PollResult poll_completion(uint64_t ticket, std::string& out) override {
    std::lock_guard<std::mutex> g(slot_mu_);
    Done d;
    bool have = false;
    auto it = finished_.find(ticket);
    if (it != finished_.end()) {
      d = it->second;
      finished_.erase(it);
      have = true;
    } else {
      for (Slot& sl : slots_) {
        if (sl.seq != ticket) continue;
        if (!sl.pending) return PollResult::FAILED;      // never flushed
        if (!record_arrived(sl)) return PollResult::PENDING;
        d = take_record(sl);
        have = true;
        break;
      }
    }
    if (!have) {
      out = "completion ticket unknown";
      return PollResult::FAILED;
    }
    std::ostringstream ss;
    ss << d.metrics << ",FlushUs=" << d.flush_us;
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
    if (!active_ && stages_.empty() && slots_.empty()) return;
    active_ = false;
    if (ctx_->device_id() >= 0) cudaSetDevice(ctx_->device_id());
    // batches still in flight keep writing into the slots: let them finish (bounded by the device itself;
    // every kernel here bounds its own waits) before the memory goes away
    for (Slot& sl : slots_)
      if (sl.stream != nullptr) cudaStreamSynchronize(sl.stream);
    stages_.clear();
    free_slots();
    for (const std::string& key : ipc_keys_) ipc_cache().release(key);
    ipc_keys_.clear();
    ipc_locals_.clear();
  }

 private:
  static constexpr size_t kSlots = 4;
  struct Slot {
    cudaStream_t stream{nullptr};      // carries the plan upload and the completion record of its batch
    cudaEvent_t plan_event{nullptr};   // the plan is on the device
    cudaEvent_t done_event{nullptr};   // behind the completion record
    char* d_plan{nullptr};
    char* h_plan{nullptr};             // pinned
    uint32_t* d_status{nullptr};       // 64 bytes: code, detail, start stamp
    KvtCompletion* h_rec{nullptr};     // mapped host memory ...
    KvtCompletion* d_rec{nullptr};     // ... and its device address
    uint64_t seq{0};                   // ticket of the batch that last used the slot
    bool pending{false};               // flushed, record not yet consumed
    std::string metrics;
    Timepoint flushed_at;
  };
  struct Done {
    uint32_t status{0}, detail{0};
    uint64_t t_start_ns{0}, t_end_ns{0};
    int64_t flush_us{0};
    std::string metrics;
  };

  void alloc_slots(size_t cap) {
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

  void free_slots() {
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

  static bool record_arrived(const Slot& sl) {
    return __atomic_load_n(&sl.h_rec->seq, __ATOMIC_ACQUIRE) == sl.seq;
  }

  // slot_mu_ held.  Moves an arrived record out of its slot.
  Done take_record(Slot& sl) {
    Done d;
    d.status = sl.h_rec->status;
    d.detail = sl.h_rec->detail;
    d.t_start_ns = sl.h_rec->t_start_ns;
    d.t_end_ns = sl.h_rec->t_end_ns;
    d.flush_us = 0;
    d.metrics = std::move(sl.metrics);
    sl.pending = false;
    return d;
  }

  Slot& cur() {
    RTASSERT(batch_slot_ >= 0);
    return slots_[static_cast<size_t>(batch_slot_)];
  }

  // Takes the next slot for a new batch.  A slot whose previous batch has not completed makes the sender
  // wait here (bounded): that is the back-pressure of a sender running more than kSlots batches ahead of
  // the GPU.  A plan larger than the slots were sized for re-allocates them (all batches drained first).
  Slot& begin_slot(size_t bytes) {
    RTASSERT(!slots_.empty());
    if (bytes > plan_cap_) {
      LOG(WARNING) << "nvlink: plan of " << bytes << " bytes exceeds the slots sized at connect (" << plan_cap_
                   << "); re-allocating";
      for (size_t i = 0; i < slots_.size(); ++i) wait_slot(slots_[i]);
      for (Slot& sl : slots_) cuda_check(cudaStreamSynchronize(sl.stream), "cudaStreamSynchronize");
      std::map<uint64_t, Done> keep;
      uint64_t seq = next_seq_;
      {
        std::lock_guard<std::mutex> g(slot_mu_);
        keep.swap(finished_);
      }
      alloc_slots(bytes * 2);
      std::lock_guard<std::mutex> g(slot_mu_);
      finished_.swap(keep);
      next_seq_ = seq;
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
    return sl;
  }

  // Waits (bounded) until the slot's previous batch has completed and parks its record for the poller.
  void wait_slot(Slot& sl) {
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
      if (SteadyClock::now() > deadline) {
        active_ = false;
        throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: an earlier batch never completed; dropping the channel");
      }
      if (spins < 2000) std::this_thread::yield(); else std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
  }

  void upload_slot(Slot& sl, size_t bytes) {
    if (bytes != 0)
      cuda_check(cudaMemcpyAsync(sl.d_plan, sl.h_plan, bytes, cudaMemcpyHostToDevice, sl.stream), "cudaMemcpyAsync(plan)");
    if (stamps_) cuda_check(kvt_launch_stamp(reinterpret_cast<uint64_t*>(sl.d_status) + 1, sl.stream), "kvt_launch_stamp");
    cuda_check(cudaEventRecord(sl.plan_event, sl.stream), "cudaEventRecord");
  }

  // The slot's stream carries the plan; a transfer stream joins it (waits for the upload) when the batch first
  // uses it, and the completion record joins back only the streams that were used.
  void begin_batch() { stage_used_.assign(stages_.size(), 0); }

  DeviceStage& use_stage(size_t i) {
    if (stage_used_.size() != stages_.size()) stage_used_.assign(stages_.size(), 0);
    if (!stage_used_[i]) {
      stages_[i]->wait_event(cur().plan_event);
      stage_used_[i] = 1;
    }
    return *stages_[i];
  }

  void ensure_layer_arrays() {
    if (d_src_layers_.p != nullptr) return;
    std::vector<uint64_t> src, dst;
    for (const auto& l : ctx_->layer_data_address()) src.push_back(l.at(0));
    for (const auto& l : dst_ptrs_) dst.push_back(l.at(0));
    d_src_layers_.upload(src);
    d_dst_layers_.upload(dst);
    use_tma_ = false;
    if (env_use_tma() != 0 && params_.mode == KVT_MODE_COPY) {
      // a tile is kept in the destination's own order, so that it leaves as one linear store where the
      // destination page holds it contiguously (HND pages; NHD pages when every head moves)
      const int want_order = env_tile_order();
      tile_order_ = want_order >= 0 ? (want_order != 0 ? 1u : 0u)
                                    : (params_.dst.token_stride < params_.dst.head_stride ? 1u : 0u);
      const bool flat_ok = kvt_tile_is_flat(&params_.dst, params_.n_heads, params_.tile_tokens, tile_order_) != 0;
      store_form_ = (flat_ok && env_store_form() != 0) ? 1u : 0u;
      std::vector<TensorMapBytes> sm(src.size()), dm(dst.size());
      bool ok = true;
      for (size_t i = 0; i < src.size() && ok; ++i) {
        ok = kvt_encode_tensor_map_ordered(sm[i].b, src[i], &params_.src, params_.n_heads, params_.tile_tokens, tile_order_) == 0 &&
             kvt_encode_tensor_map_ordered(dm[i].b, dst[i], &params_.dst, params_.n_heads, params_.tile_tokens, tile_order_) == 0;
      }
      if (ok) {
        d_src_maps_.upload(sm);
        d_dst_maps_.upload(dm);
        use_tma_ = true;
      } else {
        LOG(WARNING) << "nvlink: tensor maps not encodable for this layout, using the SIMT path";
      }
    }
  }

  Context* ctx_;
  WorkerInfo dst_;
  bool active_{false};
  std::vector<std::vector<uint64_t>> dst_ptrs_;
  std::vector<std::unique_ptr<DeviceStage>> stages_;
  int src_shape_{0}, dst_shape_{0};
  bool dst_mx_{false};
  // fused path
  bool fused_{false};
  bool use_tma_{false};
  uint32_t tile_order_{0}, store_form_{0};
  DeviceAttnParams params_{};
  PackedPlan plan_;
  bool walk_{false};
  WalkPlan walk_plan_;
  DevArray<uint64_t> d_walk_src_, d_walk_dst_;   // [layer][tensor] base addresses
  std::vector<Slot> slots_;
  size_t plan_cap_{0}, slot_rr_{0};
  int batch_slot_{-1};
  uint64_t next_seq_{0};
  char* d_plan_all_{nullptr};
  char* h_plan_all_{nullptr};
  char* d_status_all_{nullptr};
  char* h_rec_all_{nullptr};
  cudaEvent_t last_done_event_{nullptr};
  std::mutex slot_mu_;                    // slot bookkeeping is shared with the completion poller's thread
  std::map<uint64_t, Done> finished_;     // records taken out of a slot that was needed again before they were polled
  std::vector<std::string> ipc_keys_;     // mappings this channel holds a reference to
  std::vector<uint64_t> ipc_locals_;
  DevArray<uint64_t> d_src_layers_, d_dst_layers_;
  DevArray<TensorMapBytes> d_src_maps_, d_dst_maps_;
  size_t range_rr_{0};
  bool dst_remote_{false};       // the destination cache lives on another GPU
  std::vector<char> stage_used_;
  uint32_t generic_rounds_{1};   // bulk copy kernel: segment rounds the longest descriptor needs
  const bool stamps_{env_device_timestamps()};
  // generic path
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
